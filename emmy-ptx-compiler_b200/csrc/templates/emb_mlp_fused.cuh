// Cluster-fused GELU MLP for sm_100a: y = s2 * (gelu_tanh(s1 * x w1)) w2 with the hidden activations never
// leaving the thread-block cluster. A cluster of C CTAs owns a tile of 128 token rows; every CTA holds the f32
// accumulators of its own d_model / C columns of y in tensor memory. The hidden dimension is walked in rounds of
// C chunks of 128 units: in a round CTA r computes ONE chunk, h_r = gelu(s1 * x_tile w1[:, chunk r]) (tcgen05.mma into
// tensor memory, the activation on the way out, bf16 into its own shared memory), and then every CTA needs all C
// chunks for its columns of y: it reads the other CTAs' chunks out of THEIR shared memory (distributed shared memory:
// mapa + ld.shared::cluster), stages them locally and accumulates y += h_j w2[chunk j, own columns] on tcgen05.mma.
//
// This is the reference's cluster rewrite (emmy_ptx/cluster.py:120-164, statements emmy_ptx/lower.py:1147-1163: the
// loop over hidden units is split into the part that does not depend on the output column - computed once per
// cluster, a slice per CTA rank, stashed in the rank's shared memory - and the column's own part, which gathers the
// stashed values from the owners' shared memory between two cluster barriers), carried from scalar FMAs and four f32
// values per iteration to 128 x 128 tensor-core tiles and 32 KB chunks.
//
// The weights arrive as bf16 K-major copies (w1t [hidden, d_model], w2t [d_model, hidden]) made from the e4m3 codes by
// the decode kernels of emb_dequant.cuh: there is no tcgen05 kind that multiplies bf16 by e4m3.
//
//   warp 0     TMA producer of the first product: x [128 x 64] and w1t [128 x 64] K-slices, two stages
//   warp 1     TMA producer of the second product: w2t [own columns x 64] K-slices, two stages
//   warp 2     one thread issues every tcgen05.mma: chunk n + 1 of the first product BEFORE the second product of
//              chunk n, so the tensor pipe has work while chunk n is activated, published and gathered
//   warp 3     allocates and frees the tensor memory (512 columns: y 256, two h accumulators of 128)
//   warps 4-7  activation (TMEM -> gelu -> bf16 -> 128-byte-swizzled shared memory), publication to the cluster,
//              the gather of the peers' chunks, and at the end of a token tile the epilogue of y
//
// Cluster-wide hand-offs use mbarriers with remote arrivals (mbarrier.arrive.release.cluster on every CTA's
// barrier) and BOUNDED acquire.cluster waits instead of barrier.cluster, whose wait cannot give up: a CTA whose
// wait runs out records it in the status word and walks on idle, its peers' waits run out in turn, and every CTA
// reaches the one barrier.cluster at the very end, where nothing can be missing any more.
#pragma once
#include <cuda_bf16.h>

#include "emb_gemm.cuh"

namespace emb {

struct MlpShape {
    int tokens, d_model, hidden;
};

namespace mlpf {

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(tc::smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// As tc::mbar_wait, for a barrier that CTAs of the whole cluster arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const tc::Guard& g, unsigned detail) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = tc::global_ns();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((i & 255u) == 0) {
            if (*g.abort_flag) return false;
            if (tc::global_ns() - t0 > tc::WAIT_LIMIT_NS) break;
        }
    }
    tc::wait_failed(g, tc::WAIT_OTHER, detail);
    return false;
}

__device__ __forceinline__ uint4 ld_cluster_16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void fence_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }

// The 128 threads of warps 4-7 meet (named barrier 1).
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

}  // namespace mlpf

// C: CTAs per cluster; NCOLS: columns of y per CTA (d_model / C, a multiple of 16, at most 256).
template <int C, int NCOLS>
__device__ __forceinline__ void mlp_fused_kernel(const CUtensorMap* __restrict__ map_x, const CUtensorMap* __restrict__ map_w1t,
                                                 const CUtensorMap* __restrict__ map_w2t, __nv_bfloat16* __restrict__ y_out,
                                                 MlpShape shape, const float* __restrict__ s1_ptr, const float* __restrict__ s2_ptr,
                                                 unsigned* status) {
    constexpr int BM = 128, HC = 128, BK = 64, UMMA_K = 16;
    constexpr uint32_t HALF_BYTES = 128 * 128;              // 128 rows x 64 bf16: 16 KB
    constexpr uint32_t G1_STAGE = 2 * HALF_BYTES;           // x slice + w1t slice
    constexpr uint32_t W2_STAGE = 256 * 128;                // up to 256 rows x 64 bf16 (NCOLS * 128 bytes are used)
    constexpr uint32_t CHUNK = 2 * HALF_BYTES;              // 128 x 128 bf16, two 64-wide halves
    constexpr uint32_t W2_BYTES = NCOLS * 128;
    constexpr uint32_t TMEM_COLS = 512, Y_COL = 0, H_COL = 256;
    static_assert(NCOLS % 16 == 0 && NCOLS >= 16 && NCOLS <= 256, "columns of y per CTA");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* g1_smem = smem;                         // 2 stages
    uint8_t* w2_smem = g1_smem + 2 * G1_STAGE;       // 2 stages
    uint8_t* h_own = w2_smem + 2 * W2_STAGE;         // this CTA's chunk of the round
    uint8_t* h_stage = h_own + CHUNK;                // 2 slots for the peers' chunks
    uint64_t* bars = reinterpret_cast<uint64_t*>(h_stage + 2 * CHUNK);
    uint64_t* g1_full = bars;            // 2
    uint64_t* g1_empty = bars + 2;       // 2
    uint64_t* w2_full = bars + 4;        // 2
    uint64_t* w2_empty = bars + 6;       // 2
    uint64_t* hacc_full = bars + 8;      // 2: a chunk's accumulator is complete
    uint64_t* hacc_empty = bars + 10;    // 2: ... and has been read out (4 warps)
    uint64_t* hs_full = bars + 12;       // 2: a peer's chunk is staged (4 warps)
    uint64_t* hs_empty = bars + 14;      // 2: ... and consumed
    uint64_t* own_ready = bars + 16;     // this CTA's chunk is in h_own
    uint64_t* own_done = bars + 17;      // ... and this CTA's second product has read it
    uint64_t* h_ready = bars + 18;       // every CTA's chunk of the round is in place (C remote arrivals)
    uint64_t* h_free = bars + 19;        // every CTA has gathered this CTA's chunk (C remote arrivals)
    uint64_t* y_full = bars + 20;
    uint64_t* y_empty = bars + 21;       // 4 warps
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 22);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    const tc::Guard guard{status, abort_flag};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int cluster = tc::cluster_id_x(), clusters = tc::cluster_count_x();
    const int tiles = (shape.tokens + BM - 1) / BM;
    const int rounds = shape.hidden / (HC * C);
    const int k_blocks = shape.d_model / BK;
    int my_tiles = 0;
    for (int t = cluster; t < tiles; t += clusters) ++my_tiles;
    const int total_rounds = my_tiles * rounds;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(&g1_full[s], 1);
            tc::mbar_init(&g1_empty[s], 1);
            tc::mbar_init(&w2_full[s], 1);
            tc::mbar_init(&w2_empty[s], 1);
            tc::mbar_init(&hacc_full[s], 1);
            tc::mbar_init(&hacc_empty[s], 4);
            tc::mbar_init(&hs_full[s], 4);
            tc::mbar_init(&hs_empty[s], 1);
        }
        tc::mbar_init(own_ready, 1);
        tc::mbar_init(own_done, 1);
        tc::mbar_init(h_ready, C);
        tc::mbar_init(h_free, C);
        tc::mbar_init(y_full, 1);
        tc::mbar_init(y_empty, 4);
        *abort_flag = 0;
        tc::mbar_init_fence();
        tc::tma_prefetch_desc(map_x);
        tc::tma_prefetch_desc(map_w1t);
        tc::tma_prefetch_desc(map_w2t);
    }
    if (warp == 3) tc::tmem_alloc(tmem_holder, TMEM_COLS);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::cluster_sync();  // every CTA's barriers exist before anything arrives on them
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer of x and w1t slices
        if (tc::elect_one()) {
            uint32_t it = 0;
            bool alive = true;
            for (int t = cluster; alive && t < tiles; t += clusters)
                for (int q = 0; alive && q < rounds; ++q) {
                    const int chunk = q * C + static_cast<int>(rank);
                    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                        const uint32_t s = it & 1, ph = (it >> 1) & 1;
                        if (!tc::mbar_wait(&g1_empty[s], ph ^ 1, guard, tc::WAIT_SMEM_EMPTY, it)) {
                            alive = false;
                            break;
                        }
                        tc::mbar_arrive_expect_tx(&g1_full[s], G1_STAGE);
                        uint8_t* stage = g1_smem + s * G1_STAGE;
                        tc::tma_load_2d(stage, map_x, &g1_full[s], kb * BK, t * BM);
                        tc::tma_load_2d(stage + HALF_BYTES, map_w1t, &g1_full[s], kb * BK, chunk * HC);
                    }
                }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- producer of w2t slices, in the order they are consumed
        if (tc::elect_one()) {
            uint32_t it = 0;
            bool alive = true;
            for (int n = 0; alive && n < total_rounds; ++n) {
                const int q = n % rounds;
                for (int j = 0; alive && j < C; ++j) {
                    const int chunk = q * C + static_cast<int>((rank + j) % C);
                    for (int half = 0; half < 2; ++half, ++it) {
                        const uint32_t s = it & 1, ph = (it >> 1) & 1;
                        if (!tc::mbar_wait(&w2_empty[s], ph ^ 1, guard, tc::WAIT_SMEM_EMPTY, 100000 + it)) {
                            alive = false;
                            break;
                        }
                        tc::mbar_arrive_expect_tx(&w2_full[s], W2_BYTES);
                        tc::tma_load_2d(w2_smem + s * W2_STAGE, map_w2t, &w2_full[s], chunk * HC + half * BK, static_cast<int>(rank) * NCOLS);
                    }
                }
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- MMA issuer
        if (tc::elect_one()) {
            constexpr uint32_t idesc_g1 = tc::idesc_f16(BM, HC, true);
            constexpr uint32_t idesc_g2 = tc::idesc_f16(BM, NCOLS, true);
            uint32_t g1_it = 0, w2_it = 0, hs_it = 0;
            bool alive = true;
            // first product of global round n: its chunk's accumulator h_acc[n & 1]
            auto first_product = [&](int n) {
                const uint32_t buf = n & 1;
                if (!tc::mbar_wait(&hacc_empty[buf], ((n >> 1) & 1) ^ 1, guard, tc::WAIT_TMEM_EMPTY, n)) return false;
                tc::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + H_COL + buf * HC;
                for (int kb = 0; kb < k_blocks; ++kb, ++g1_it) {
                    const uint32_t s = g1_it & 1;
                    if (!tc::mbar_wait(&g1_full[s], (g1_it >> 1) & 1, guard, tc::WAIT_SMEM_FULL, g1_it)) return false;
                    tc::tc_fence_after_sync();
                    const uint8_t* stage = g1_smem + s * G1_STAGE;
                    const uint64_t a_desc = tc::smem_desc_k128(stage), b_desc = tc::smem_desc_k128(stage + HALF_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc::mma_f16_ss(d_tmem, a_desc + (k * 32 >> 4), b_desc + (k * 32 >> 4), idesc_g1, (kb | k) != 0);
                    tc::mma_commit(&g1_empty[s]);
                }
                tc::mma_commit(&hacc_full[buf]);
                return true;
            };
            // second product of global round n: y += h_j w2[chunk j, own columns] for this CTA's own chunk, then the peers'
            auto second_product = [&](int n) {
                const int q = n % rounds, tile_local = n / rounds;
                if (q == 0) {  // the previous token tile's y has been read out
                    if (!tc::mbar_wait(y_empty, (tile_local & 1) ^ 1, guard, tc::WAIT_TMEM_EMPTY, 200000 + n)) return false;
                    tc::tc_fence_after_sync();
                }
                for (int j = 0; j < C; ++j) {
                    const uint8_t* a_base;
                    uint32_t slot = 0;
                    if (j == 0) {
                        if (!tc::mbar_wait(own_ready, n & 1, guard, tc::WAIT_SMEM_FULL, 300000 + n)) return false;
                        a_base = h_own;
                    } else {
                        slot = hs_it & 1;
                        if (!tc::mbar_wait(&hs_full[slot], (hs_it >> 1) & 1, guard, tc::WAIT_SMEM_FULL, 400000 + hs_it)) return false;
                        a_base = h_stage + slot * CHUNK;
                    }
                    tc::tc_fence_after_sync();
                    for (int half = 0; half < 2; ++half, ++w2_it) {
                        const uint32_t s = w2_it & 1;
                        if (!tc::mbar_wait(&w2_full[s], (w2_it >> 1) & 1, guard, tc::WAIT_SMEM_FULL, 500000 + w2_it)) return false;
                        tc::tc_fence_after_sync();
                        const uint64_t a_desc = tc::smem_desc_k128(a_base + half * HALF_BYTES);
                        const uint64_t b_desc = tc::smem_desc_k128(w2_smem + s * W2_STAGE);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            tc::mma_f16_ss(tmem_base + Y_COL, a_desc + (k * 32 >> 4), b_desc + (k * 32 >> 4), idesc_g2,
                                           (q | j | half | k) != 0);
                        tc::mma_commit(&w2_empty[s]);
                    }
                    if (j == 0) {
                        tc::mma_commit(own_done);
                    } else {
                        tc::mma_commit(&hs_empty[slot]);
                        ++hs_it;
                    }
                }
                if (q == rounds - 1) tc::mma_commit(y_full);
                return true;
            };
            if (total_rounds > 0) alive = first_product(0);
            for (int n = 0; alive && n < total_rounds; ++n) {
                if (n + 1 < total_rounds) alive = first_product(n + 1);
                if (alive) alive = second_product(n);
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- activation, publication, gather, epilogue of y
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int tid = threadIdx.x - 128;  // 0..127 among the epilogue threads
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const float s1 = __ldg(s1_ptr), s2 = __ldg(s2_ptr);
        uint32_t hs_cnt = 0;
        bool alive = true;  // a thread whose wait ran out walks on idle: the named barriers below still need it
        int n = 0;
        for (int t = cluster; t < tiles; t += clusters) {
            for (int q = 0; q < rounds; ++q, ++n) {
                const uint32_t buf = n & 1;
                if (alive) alive = tc::mbar_wait(&hacc_full[buf], (n >> 1) & 1, guard, tc::WAIT_TMEM_FULL, 600000 + n);
                if (alive && n > 0) {  // h_own is free again: this CTA's second product and every peer's gather have read round n - 1
                    alive = tc::mbar_wait(own_done, (n - 1) & 1, guard, tc::WAIT_SMEM_EMPTY, 700000 + n);
                    if (alive) alive = mlpf::mbar_wait_cluster(h_free, (n - 1) & 1, guard, 800000 + n);
                }
                if (alive) {
                    tc::tc_fence_after_sync();
                    const uint32_t taddr = tmem_base + lane_addr + H_COL + buf * HC;
#pragma unroll 1
                    for (int cb = 0; cb < HC; cb += 32) {
                        uint32_t v[32];
                        tc::tmem_ld_32x32(taddr + cb, v);
                        tc::tmem_ld_wait();
                        // row `row` of the chunk, columns cb .. cb + 31, as bf16: 64 bytes = four 16-byte pieces of the row's
                        // 128-byte line in the half (cb / 64); the 128-byte swizzle XORs the piece index with (row % 8)
                        uint8_t* line = h_own + (cb >> 6) * HALF_BYTES + row * 128;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 p;
                            p.x = pack2<true>(gelu_tanh_fast(__uint_as_float(v[8 * i + 0]) * s1), gelu_tanh_fast(__uint_as_float(v[8 * i + 1]) * s1));
                            p.y = pack2<true>(gelu_tanh_fast(__uint_as_float(v[8 * i + 2]) * s1), gelu_tanh_fast(__uint_as_float(v[8 * i + 3]) * s1));
                            p.z = pack2<true>(gelu_tanh_fast(__uint_as_float(v[8 * i + 4]) * s1), gelu_tanh_fast(__uint_as_float(v[8 * i + 5]) * s1));
                            p.w = pack2<true>(gelu_tanh_fast(__uint_as_float(v[8 * i + 6]) * s1), gelu_tanh_fast(__uint_as_float(v[8 * i + 7]) * s1));
                            const int piece = (((cb & 63) >> 3) + i) ^ (row & 7);
                            *reinterpret_cast<uint4*>(line + piece * 16) = p;
                        }
                    }
                    tc::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&hacc_empty[buf]);
                    tc::fence_async_smem();   // the chunk is read by this CTA's tensor pipe ...
                    mlpf::fence_cluster();    // ... and by the peers' loads
                }
                mlpf::epilogue_sync();
                if (tid == 0 && alive) {
                    tc::mbar_arrive(own_ready);
#pragma unroll
                    for (int c = 0; c < C; ++c) tc::mbar_arrive_cluster(tc::smem_of_cta(h_ready, c));
                }
                if (alive) alive = mlpf::mbar_wait_cluster(h_ready, n & 1, guard, 900000 + n);
                // gather: peer (rank + j) % C's chunk into a staging slot, 16 bytes per thread and step (the layout is kept)
                for (int j = 1; j < C; ++j, ++hs_cnt) {
                    const uint32_t slot = hs_cnt & 1;
                    if (alive) alive = tc::mbar_wait(&hs_empty[slot], ((hs_cnt >> 1) & 1) ^ 1, guard, tc::WAIT_SMEM_EMPTY, 1000000 + hs_cnt);
                    if (alive) {
                        const uint32_t src = tc::smem_of_cta(h_own, (rank + j) % C);
                        uint8_t* dst = h_stage + slot * CHUNK;
                        constexpr int PIECES = static_cast<int>(CHUNK / 16 / 128);  // 16 per thread: all loads in flight, then the stores
                        uint4 piece[PIECES];
#pragma unroll
                        for (int i = 0; i < PIECES; ++i) piece[i] = mlpf::ld_cluster_16(src + (i * 128 + tid) * 16);
#pragma unroll
                        for (int i = 0; i < PIECES; ++i) *reinterpret_cast<uint4*>(dst + (i * 128 + tid) * 16) = piece[i];
                        tc::fence_async_smem();
                        __syncwarp();
                        if (lane == 0) tc::mbar_arrive(&hs_full[slot]);
                    }
                }
                mlpf::epilogue_sync();  // all of this CTA's gathers of the round are done
                if (tid == 0 && alive) {
#pragma unroll
                    for (int c = 0; c < C; ++c) tc::mbar_arrive_cluster(tc::smem_of_cta(h_free, c));
                }
            }
            // epilogue of the token tile: this CTA's columns of y
            const int tile_local = n / rounds - 1;
            if (alive) alive = tc::mbar_wait(y_full, tile_local & 1, guard, tc::WAIT_TMEM_FULL, 1100000 + n);
            if (alive) {
                tc::tc_fence_after_sync();
                const int grow = t * BM + row;
                const uint32_t taddr = tmem_base + lane_addr + Y_COL;
#pragma unroll 1
                for (int cb = 0; cb < NCOLS; cb += 16) {
                    uint32_t v[16];
                    tc::tmem_ld_32x16(taddr + cb, v);
                    tc::tmem_ld_wait();
                    if (grow < shape.tokens) {
                        __nv_bfloat16* dst = y_out + static_cast<size_t>(grow) * shape.d_model + rank * NCOLS + cb;
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            uint4 p;
                            p.x = pack2<true>(__uint_as_float(v[8 * i + 0]) * s2, __uint_as_float(v[8 * i + 1]) * s2);
                            p.y = pack2<true>(__uint_as_float(v[8 * i + 2]) * s2, __uint_as_float(v[8 * i + 3]) * s2);
                            p.z = pack2<true>(__uint_as_float(v[8 * i + 4]) * s2, __uint_as_float(v[8 * i + 5]) * s2);
                            p.w = pack2<true>(__uint_as_float(v[8 * i + 6]) * s2, __uint_as_float(v[8 * i + 7]) * s2);
                            *reinterpret_cast<uint4*>(dst + 8 * i) = p;
                        }
                    }
                }
                tc::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(y_empty);
            }
        }
    }

    // teardown: nobody leaves while a peer may still read its shared memory or arrive on its barriers
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::cluster_sync();
    if (warp == 3) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace emb
