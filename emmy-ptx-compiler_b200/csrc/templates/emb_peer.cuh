// The exchange step of a sharded sum, inside the kernel that produced this GPU's share: every rank stores its f32
// value into every peer's slot over NVLink (plain peer stores into symmetric memory; no multicast, no collective
// library), waits - BOUNDED - for the slots of all peers and adds the values in rank order, so every rank gets the
// same bits. It replaces the all-reduce that would follow the kernel as a launch of its own (in the reference a
// problem runs on one GPU; sharding its element range is this backend's addition).
//
// Memory per rank (symmetric: the same layout at every rank, mapped into every peer):
//   u64 slot[2][EMB_MAX_PEERS]   slot [q & 1][r] = (q << 32) | bits of rank r's value of step q
// Value and step number travel in ONE 8-byte store, which is atomic: no fence between a value and its flag, one
// NVLink crossing per peer. Two parities: a rank one step ahead writes the other parity, and it cannot get two steps
// ahead, because its wait of the step between needs this rank's store, which this rank issues only after it has read
// the older values.
#pragma once
#include <stdint.h>

#define EMB_MAX_PEERS 8

namespace emb {

struct PeerExchange {
    unsigned long long* slot[EMB_MAX_PEERS];  // slot[r]: rank r's slots (a peer pointer for r != rank)
    unsigned rank, world;
    unsigned step;    // steps completed by this rank (touched by this rank's kernels only)
    unsigned status;  // 0, or 1 + the peer whose value did not arrive in time (results are invalid from then on)
    unsigned wait_limit_us;  // how long a wait for a peer may last (the host sets 2 s; a test of the time-out far less)
    unsigned reserved;
};

__device__ __forceinline__ void peer_store(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long peer_load(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
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
    if (*reinterpret_cast<volatile unsigned*>(&px->status)) return mine;  // an earlier wait gave up: no more waiting, the host reports it
    __syncthreads();  // earlier uses of `bcast` are over
    if (threadIdx.x < 32) {
        const unsigned lane = threadIdx.x, world = px->world, rank = px->rank;
        const unsigned q = px->step + 1, parity = (q & 1u) * EMB_MAX_PEERS;
        __syncwarp();  // every lane has read `step` before lane 0 moves it on
        float theirs = 0.0f;
        if (lane < world) {
            peer_store(px->slot[lane] + parity + rank, (static_cast<unsigned long long>(q) << 32) | __float_as_uint(mine));
            const unsigned long long* from = px->slot[rank] + parity + lane;
            unsigned long long got = peer_load(from);
            if (static_cast<unsigned>(got >> 32) != q) {
                const unsigned long long t0 = peer_ns(), limit = 1000ull * px->wait_limit_us;
                for (unsigned i = 1; static_cast<unsigned>((got = peer_load(from)) >> 32) != q; ++i) {
                    if ((i & 63u) == 0 && peer_ns() - t0 > limit) {
                        atomicCAS(&px->status, 0u, lane + 1);
                        break;
                    }
                }
            }
            theirs = __uint_as_float(static_cast<unsigned>(got));
        }
        __syncwarp();
        float total = __shfl_sync(0xffffffffu, theirs, 0);
        for (unsigned r = 1; r < world; ++r) total = __fadd_rn(total, __shfl_sync(0xffffffffu, theirs, r));  // rank order on every rank
        if (lane == 0) {
            px->step = q;
            *bcast = total;
        }
    }
    __syncthreads();
    return *bcast;
}

}  // namespace emb
