// The exchange step of a sharded sum, inside the kernel that produced this GPU's share: every rank stores its f32
// value into every peer's slot over NVLink (plain peer stores into symmetric memory; no multicast, no collective
// library), raises a flag behind it, waits - BOUNDED - for the flags of all peers and adds the values in rank order,
// so every rank gets the same bits. It replaces the all-reduce that would follow the kernel as a launch of its own
// (in the reference a problem runs on one GPU; sharding its element range is this backend's addition).
//
// Memory per rank (symmetric: the same layout at every rank, mapped into every peer):
//   float    value[2][EMB_MAX_PEERS]   slot [q & 1][r] = rank r's value of step q
//   unsigned flag [2][EMB_MAX_PEERS]   slot [q & 1][r] = q once that value is there
// Two parities: a rank one step ahead writes the other parity, and it cannot get two steps ahead, because its wait
// of the step between needs this rank's flag, which this rank raises only after it has read the older values.
#pragma once
#include <stdint.h>

#define EMB_MAX_PEERS 8

namespace emb {

struct PeerExchange {
    float* value[EMB_MAX_PEERS];     // value[r]: rank r's value slots (a peer pointer for r != rank)
    unsigned* flag[EMB_MAX_PEERS];   // flag[r]: rank r's flag slots
    unsigned rank, world;
    unsigned step;                   // steps completed by this rank (touched by this rank's kernels only)
    unsigned status;                 // 0, or 1 + the peer whose flag did not arrive in time (the result is then invalid)
};

constexpr unsigned long long PEER_WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ void peer_store_release(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned peer_load_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long peer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Called by every thread of a ONE-block kernel with the same `mine`; returns the sum over all ranks (`mine` itself
// when there is no exchange). `bcast` is one float of shared memory.
__device__ __forceinline__ float peer_all_sum(float mine, PeerExchange* px, float* bcast) {
    if (px == nullptr) return mine;
    if (*static_cast<volatile unsigned*>(&px->status)) return mine;  // an earlier wait gave up: no further waiting, the host reports it
    __syncthreads();  // earlier uses of `bcast` are over
    if (threadIdx.x < 32) {
        const unsigned lane = threadIdx.x, world = px->world, rank = px->rank;
        const unsigned q = px->step + 1, slot = (q & 1u) * EMB_MAX_PEERS;
        __syncwarp();  // every lane has read `step` before lane 0 moves it on
        if (lane < world) {
            volatile float* there = px->value[lane] + slot + rank;
            *there = mine;
            peer_store_release(px->flag[lane] + slot + rank, q);  // the value is visible before the flag
            const unsigned* f = px->flag[rank] + slot + lane;
            if (peer_load_acquire(f) != q) {
                const unsigned long long t0 = peer_ns();
                for (unsigned i = 1; peer_load_acquire(f) != q; ++i) {
                    if ((i & 63u) == 0 && peer_ns() - t0 > PEER_WAIT_LIMIT_NS) {
                        atomicCAS(&px->status, 0u, lane + 1);
                        break;
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) {
            const volatile float* here = px->value[rank] + slot;
            float total = here[0];
            for (unsigned r = 1; r < world; ++r) total = __fadd_rn(total, here[r]);  // rank order on every rank
            px->step = q;
            *bcast = total;
        }
    }
    __syncthreads();
    return *bcast;
}

}  // namespace emb
