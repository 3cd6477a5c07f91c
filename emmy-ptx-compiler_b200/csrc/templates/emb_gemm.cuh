// Tensor-core matmul template for sm_100a: C[M,N] = A[M,K] * B[N,K]^T, A and B 16-bit (f16 or bf16),
// both K-major ("row-major A, column-major B"), f32 accumulation in tensor memory, C rounded once to
// the output type.
//
// It takes the place of the reference's tensor-core lowering, which turns emmy's fragment statements
// into ldmatrix / mma.sync.m16n8k16 on 16x8 warp tiles (emmy_ptx/tensorcore.py:165-279,376-420) fed by
// cp.async (emmy_ptx/lower.py:1057-1102) or, with --bulk-copy, by untiled cp.async.bulk on eight
// round-robin mbarriers (emmy_ptx/bulk.py:34-57, emmy_ptx/lower.py:1167-1238). Here one persistent CTA
// per SM walks 128 x 256 output tiles:
//
//   warp 0    producer  one thread issues TMA tensor-map loads of the A (128 x 64) and B (256 x 64)
//                       K-slices into a ring of STAGES shared-memory stages; a stage's mbarrier counts
//                       the bytes landed (full) and the MMAs that consumed it (empty)
//   warp 1    MMA       one thread issues tcgen05.mma 128x256x16 (four per stage) accumulating into one
//                       of two 256-column TMEM buffers; tcgen05.commit releases the stage and, after the
//                       last K-slice, hands the buffer to the epilogue
//   warps 2-5 epilogue  tcgen05.ld 32 lanes x 32 columns per warp, convert, 16-byte global stores; the
//                       other TMEM buffer is being accumulated meanwhile
//
// No multicast, no clusters: every CTA loads its own tiles; reuse comes from L2 through the tile order
// (GROUP_M row-blocks share each B panel while it is resident).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "emb_math.cuh"
#include "emb_tc.cuh"

namespace emb {

template <bool BF16> struct Half16 { using type = __half; };
template <> struct Half16<true> { using type = __nv_bfloat16; };

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<false>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<true>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <bool BF16> __device__ __forceinline__ void unpack2(uint32_t v, float& lo, float& hi);
template <> __device__ __forceinline__ void unpack2<false>(uint32_t v, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
    lo = f.x, hi = f.y;
}
template <> __device__ __forceinline__ void unpack2<true>(uint32_t v, float& lo, float& hi) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
    lo = f.x, hi = f.y;
}

struct GemmShape {
    int m, n, k;
    int splits = 1;  // K is cut into this many slabs (each a multiple of 64 when there are several); C is [splits, m, n]
};

// What the epilogue does to an accumulator before it is rounded to the output type.
enum GemmEpilogue : int {
    EPI_NONE = 0,        // c = acc
    EPI_SCALE = 1,       // c = acc * scale[0]
    EPI_SCALE_GELU = 2,  // c = gelu_tanh(acc * scale[0])
};

// A per-cell epilogue given by the caller: f(acc, row, column) -> value (the statements an IR has between its
// contraction loop and its Write, lowered one by one). The default does nothing.
struct NoCellEpilogue {
    __device__ __forceinline__ float operator()(float acc, int, int) const { return acc; }
};
template <class F> struct HasCellEpilogue { static constexpr bool value = true; };
template <> struct HasCellEpilogue<NoCellEpilogue> { static constexpr bool value = false; };

template <int EPI> __device__ __forceinline__ float gemm_epilogue(float acc, float scale) {
    if (EPI == EPI_SCALE) return acc * scale;
    if (EPI == EPI_SCALE_GELU) return gelu_tanh_fast(acc * scale);
    return acc;
}

// FP8: the operands are e4m3 byte codes (tcgen05 kind::f8f6f4, 128 elements per 128-byte row, K = 32 per MMA);
// otherwise 16-bit (kind::f16, 64 elements per row, K = 16 per MMA). BF16 names the OUTPUT type (and, for the
// 16-bit kind, the operand type).
// B_NMAJOR: B is stored [K, N] (N contiguous) instead of [N, K]: its stage is four boxes of 64 columns x 64 k, read
// through an MN-major descriptor. OUT_F32: C is f32 (the partial slabs of a split-K schedule) instead of 16-bit.
template <int STAGES, int GROUP_M, bool BF16, int EPI = EPI_NONE, bool FP8 = false, bool B_NMAJOR = false, bool OUT_F32 = false,
          class CellEpilogue = NoCellEpilogue>
__device__ __forceinline__ void gemm_tn_kernel(const CUtensorMap* __restrict__ map_a, const CUtensorMap* __restrict__ map_b,
                                               void* __restrict__ c_out, GemmShape shape, unsigned* status,
                                               const float* __restrict__ scale_ptr = nullptr, CellEpilogue cell = CellEpilogue()) {
    constexpr int ELEM = FP8 ? 1 : 2;                       // bytes per operand element
    constexpr int BM = 128, BN = 256, BK = 128 / ELEM, UMMA_K = 32 / ELEM;  // a stage row and an MMA step are 128 and 32 bytes
    constexpr uint32_t A_BYTES = BM * BK * ELEM, B_BYTES = BN * BK * ELEM, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 512;
    using out_t = typename Half16<BF16>::type;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // the operand tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tmem_full = bars + 2 * STAGES;
    uint64_t* tmem_empty = bars + 2 * STAGES + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    const tc::Guard guard{status, abort_flag};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (shape.m + BM - 1) / BM, tiles_n = (shape.n + BN - 1) / BN;
    const int tiles_mn = tiles_m * tiles_n;
    const int num_tiles = tiles_mn * shape.splits;
    const int k_slab = shape.k / shape.splits;
    const int k_blocks = (k_slab + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&tmem_full[b], 1);
            tc::mbar_init(&tmem_empty[b], 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        tc::mbar_init_fence();
        tc::tma_prefetch_desc(map_a);
        tc::tma_prefetch_desc(map_b);
    }
    if (warp == 1) tc::tmem_alloc(tmem_holder, TMEM_COLS);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    // tile order: GROUP_M row-blocks at a time, all column-blocks under them, so that the CTAs running
    // together share A and B panels in L2
    auto tile_coords = [&](int t, int& tm, int& tn, int& slab) {
        slab = t / tiles_mn;
        t -= slab * tiles_mn;
        const int per_group = GROUP_M * tiles_n;
        const int g = t / per_group, r = t % per_group;
        const int rows = min(GROUP_M, tiles_m - g * GROUP_M);
        tm = g * GROUP_M + r % rows;
        tn = r / rows;
    };

    if (warp == 0) {
        if (tc::elect_one()) {
            uint32_t it = 0;
            bool alive = true;
            for (int t = blockIdx.x; alive && t < num_tiles; t += gridDim.x) {
                int tm, tn, slab;
                tile_coords(t, tm, tn, slab);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (!tc::mbar_wait(&empty[s], ph ^ 1, guard, tc::WAIT_SMEM_EMPTY, it)) {
                        alive = false;
                        break;
                    }
                    tc::mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                    uint8_t* stage = smem + s * STAGE_BYTES;
                    const int k0 = slab * k_slab + kb * BK;
                    tc::tma_load_2d(stage, map_a, &full[s], k0, tm * BM);
                    if (B_NMAJOR) {
#pragma unroll
                        for (int b = 0; b < BN / 64; ++b)
                            tc::tma_load_2d(stage + A_BYTES + b * (B_BYTES / (BN / 64)), map_b, &full[s], tn * BN + b * 64, k0);
                    } else {
                        tc::tma_load_2d(stage + A_BYTES, map_b, &full[s], k0, tn * BN);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (tc::elect_one()) {
            constexpr uint32_t idesc = (FP8 ? tc::idesc_e4m3(BM, BN) : tc::idesc_f16(BM, BN, BF16)) | (B_NMAJOR ? 1u << 16 : 0u);
            uint32_t it = 0, local = 0;
            bool alive = true;
            for (int t = blockIdx.x; alive && t < num_tiles; t += gridDim.x, ++local) {
                const uint32_t buf = local & 1, use = local >> 1;
                if (!tc::mbar_wait(&tmem_empty[buf], (use & 1) ^ 1, guard, tc::WAIT_TMEM_EMPTY, local)) break;
                tc::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (!tc::mbar_wait(&full[s], ph, guard, tc::WAIT_SMEM_FULL, it)) {
                        alive = false;
                        break;
                    }
                    tc::tc_fence_after_sync();
                    const uint8_t* stage = smem + s * STAGE_BYTES;
                    const uint64_t a_desc = tc::smem_desc_k128(stage), b_desc = tc::smem_desc_k128(stage + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        if (FP8)
                            tc::mma_e4m3_ss(d_tmem, a_desc + (k * 32 >> 4), b_desc + (k * 32 >> 4), idesc, (kb | k) != 0);
                        else if (B_NMAJOR)  // 16 k = 16 rows of 128 bytes further on; 64-column groups 8 KB apart
                            tc::mma_f16_ss(d_tmem, a_desc + (k * 32 >> 4),
                                           tc::smem_desc_mn128(stage + A_BYTES + k * UMMA_K * 128, B_BYTES / (BN / 64)), idesc, (kb | k) != 0);
                        else
                            tc::mma_f16_ss(d_tmem, a_desc + (k * 32 >> 4), b_desc + (k * 32 >> 4), idesc, (kb | k) != 0);
                    }
                    tc::mma_commit(&empty[s]);  // the stage is free once these MMAs have read it
                }
                if (alive) tc::mma_commit(&tmem_full[buf]);
            }
        }
    } else {
        // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        uint32_t local = 0;
        out_t* c = static_cast<out_t*>(c_out);
        const bool vec_ok = (shape.n % 8) == 0;
        const float scale = (EPI != EPI_NONE && scale_ptr) ? __ldg(scale_ptr) : 1.0f;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++local) {
            int tm, tn, slab;
            tile_coords(t, tm, tn, slab);
            const uint32_t buf = local & 1, use = local >> 1;
            if (!tc::mbar_wait(&tmem_full[buf], use & 1, guard, tc::WAIT_TMEM_FULL, local)) break;
            tc::tc_fence_after_sync();
            const int row = tm * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int cb = 0; cb < BN; cb += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(taddr + cb, r);
                tc::tmem_ld_wait();
                if (EPI != EPI_NONE) {
#pragma unroll
                    for (int x = 0; x < 32; ++x) r[x] = __float_as_uint(gemm_epilogue<EPI>(__uint_as_float(r[x]), scale));
                }
                const int col = tn * BN + cb;
                if (HasCellEpilogue<CellEpilogue>::value && row < shape.m) {
#pragma unroll
                    for (int x = 0; x < 32; ++x)
                        if (col + x < shape.n) r[x] = __float_as_uint(cell(__uint_as_float(r[x]), row, col + x));
                }
                if (OUT_F32) {
                    if (row < shape.m) {
                        float* dst = static_cast<float*>(c_out) + (static_cast<size_t>(slab) * shape.m + row) * shape.n + col;
                        if ((shape.n % 4) == 0 && col + 32 <= shape.n) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                *reinterpret_cast<uint4*>(dst + 4 * q) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (col + j < shape.n) dst[j] = __uint_as_float(r[j]);
                        }
                    }
                } else if (row < shape.m) {
                    out_t* dst = c + (static_cast<size_t>(slab) * shape.m + row) * shape.n + col;
                    if (vec_ok && col + 32 <= shape.n) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint4 v;
                            v.x = pack2<BF16>(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1]));
                            v.y = pack2<BF16>(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
                            v.z = pack2<BF16>(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
                            v.w = pack2<BF16>(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                            *reinterpret_cast<uint4*>(dst + 8 * q) = v;
                        }
                    } else {
                        for (int j = 0; j < 32; ++j)
                            if (col + j < shape.n) {
                                uint32_t p = pack2<BF16>(__uint_as_float(r[j]), 0.0f);
                                dst[j] = *reinterpret_cast<out_t*>(&p);
                            }
                    }
                }
            }
            tc::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&tmem_empty[buf]);
        }
    }

    // teardown: everyone meets, then the allocating warp frees the tensor memory
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// The same matmul on CTA PAIRS: a cluster of two CTAs (the two SMs of a TPC) owns a 256 x 256 output tile and
// runs it as ONE tcgen05.mma.cta_group::2 of 256 x 256 x 16 per step. CTA r of the pair loads rows
// 128 r .. 128 r + 127 of the tile's A panel and of its B panel (half of what a lone CTA would load for the same
// amount of tensor work, so a stage is 32 KB and the ring can be deeper) and holds lanes = rows 128 r .. of
// the accumulator in its own tensor memory. Roles per CTA as above, with these differences:
//
//   producer  both CTAs load their halves; the bytes of both are counted on the LEADER's (rank 0) full barrier
//   MMA       only the leader issues; its commits arrive on the empty / accumulator-full barriers of BOTH CTAs
//   epilogue  both CTAs drain their own 128 lanes; every epilogue warp of both arrives on the leader's
//             accumulator-empty barrier (8 arrivals)
//
// The tensor maps must have boxes of 128 rows for A and for B.
template <int STAGES, int GROUP_M, bool BF16, int EPI = EPI_NONE, bool FP8 = false, class CellEpilogue = NoCellEpilogue>
__device__ __forceinline__ void gemm_tn_pair_kernel(const CUtensorMap* __restrict__ map_a, const CUtensorMap* __restrict__ map_b,
                                                    void* __restrict__ c_out, GemmShape shape, unsigned* status,
                                                    const float* __restrict__ scale_ptr = nullptr, CellEpilogue cell = CellEpilogue()) {
    constexpr int ELEM = FP8 ? 1 : 2;
    constexpr int BM = 256, BN = 256, HALF = 128, BK = 128 / ELEM, UMMA_K = 32 / ELEM;
    constexpr uint32_t A_BYTES = HALF * BK * ELEM, B_BYTES = HALF * BK * ELEM, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 512;
    using out_t = typename Half16<BF16>::type;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // the same offsets in both CTAs: the MMA applies one descriptor to both shared memories
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                    // used in the leader only
    uint64_t* empty = bars + STAGES;          // one set per CTA
    uint64_t* tmem_full = bars + 2 * STAGES;  // one set per CTA
    uint64_t* tmem_empty = bars + 2 * STAGES + 2;  // used in the leader only
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    const tc::Guard guard{status, abort_flag};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = tc::cluster_id_x(), pairs = tc::cluster_count_x();
    const int tiles_m = (shape.m + BM - 1) / BM, tiles_n = (shape.n + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int k_blocks = (shape.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&tmem_full[b], 1);
            tc::mbar_init(&tmem_empty[b], 8);  // one arrival per epilogue warp of both CTAs
        }
        *abort_flag = 0;
        tc::mbar_init_fence();
        tc::tma_prefetch_desc(map_a);
        tc::tma_prefetch_desc(map_b);
    }
    if (warp == 1) tc::tmem_alloc_pair(tmem_holder, TMEM_COLS);
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::cluster_sync();  // the peer's barriers exist before anything arrives on them
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    auto tile_coords = [&](int t, int& tm, int& tn) {
        const int per_group = GROUP_M * tiles_n;
        const int g = t / per_group, r = t % per_group;
        const int rows = min(GROUP_M, tiles_m - g * GROUP_M);
        tm = g * GROUP_M + r % rows;
        tn = r / rows;
    };

    if (warp == 0) {
        if (tc::elect_one()) {
            uint32_t it = 0;
            bool alive = true;
            for (int t = pair; alive && t < num_tiles; t += pairs) {
                int tm, tn;
                tile_coords(t, tm, tn);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (!tc::mbar_wait(&empty[s], ph ^ 1, guard, tc::WAIT_SMEM_EMPTY, it)) {
                        alive = false;
                        break;
                    }
                    if (rank == 0) tc::mbar_arrive_expect_tx(&full[s], 2 * STAGE_BYTES);
                    const uint32_t leader_full = tc::smem_of_cta(&full[s], 0);
                    uint8_t* stage = smem + s * STAGE_BYTES;
                    tc::tma_load_2d_pair(stage, map_a, leader_full, kb * BK, tm * BM + rank * HALF);
                    tc::tma_load_2d_pair(stage + A_BYTES, map_b, leader_full, kb * BK, tn * BN + rank * HALF);
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && tc::elect_one()) {
            constexpr uint32_t idesc = FP8 ? tc::idesc_e4m3(BM, BN) : tc::idesc_f16(BM, BN, BF16);
            uint32_t it = 0, local = 0;
            bool alive = true;
            for (int t = pair; alive && t < num_tiles; t += pairs, ++local) {
                const uint32_t buf = local & 1, use = local >> 1;
                if (!tc::mbar_wait(&tmem_empty[buf], (use & 1) ^ 1, guard, tc::WAIT_TMEM_EMPTY, local)) break;
                tc::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (!tc::mbar_wait(&full[s], ph, guard, tc::WAIT_SMEM_FULL, it)) {
                        alive = false;
                        break;
                    }
                    tc::tc_fence_after_sync();
                    const uint8_t* stage = smem + s * STAGE_BYTES;
                    const uint64_t a_desc = tc::smem_desc_k128(stage), b_desc = tc::smem_desc_k128(stage + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        if (FP8)
                            tc::mma_e4m3_ss_pair(d_tmem, a_desc + (k * 32 >> 4), b_desc + (k * 32 >> 4), idesc, (kb | k) != 0);
                        else
                            tc::mma_f16_ss_pair(d_tmem, a_desc + (k * 32 >> 4), b_desc + (k * 32 >> 4), idesc, (kb | k) != 0);
                    }
                    tc::mma_commit_pair(&empty[s], 3);  // the stage is free in both CTAs once these MMAs have read it
                }
                if (alive) tc::mma_commit_pair(&tmem_full[buf], 3);
            }
        }
    } else {
        const int quarter = warp & 3;
        uint32_t local = 0;
        out_t* c = static_cast<out_t*>(c_out);
        const bool vec_ok = (shape.n % 8) == 0;
        const float scale = (EPI != EPI_NONE && scale_ptr) ? __ldg(scale_ptr) : 1.0f;
        for (int t = pair; t < num_tiles; t += pairs, ++local) {
            int tm, tn;
            tile_coords(t, tm, tn);
            const uint32_t buf = local & 1, use = local >> 1;
            if (!tc::mbar_wait(&tmem_full[buf], use & 1, guard, tc::WAIT_TMEM_FULL, local)) break;
            tc::tc_fence_after_sync();
            const int row = tm * BM + rank * HALF + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int cb = 0; cb < BN; cb += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(taddr + cb, r);
                tc::tmem_ld_wait();
                if (EPI != EPI_NONE) {
#pragma unroll
                    for (int x = 0; x < 32; ++x) r[x] = __float_as_uint(gemm_epilogue<EPI>(__uint_as_float(r[x]), scale));
                }
                const int col = tn * BN + cb;
                if (HasCellEpilogue<CellEpilogue>::value && row < shape.m) {
#pragma unroll
                    for (int x = 0; x < 32; ++x)
                        if (col + x < shape.n) r[x] = __float_as_uint(cell(__uint_as_float(r[x]), row, col + x));
                }
                if (row < shape.m) {
                    out_t* dst = c + static_cast<size_t>(row) * shape.n + col;
                    if (vec_ok && col + 32 <= shape.n) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint4 v;
                            v.x = pack2<BF16>(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1]));
                            v.y = pack2<BF16>(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
                            v.z = pack2<BF16>(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
                            v.w = pack2<BF16>(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                            *reinterpret_cast<uint4*>(dst + 8 * q) = v;
                        }
                    } else {
                        for (int j = 0; j < 32; ++j)
                            if (col + j < shape.n) {
                                uint32_t p = pack2<BF16>(__uint_as_float(r[j]), 0.0f);
                                dst[j] = *reinterpret_cast<out_t*>(&p);
                            }
                    }
                }
            }
            tc::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive_cluster(tc::smem_of_cta(&tmem_empty[buf], 0));
        }
    }

    // teardown: both CTAs meet (neither may leave while the other can still read its shared memory or arrive
    // on its barriers), then the allocating warp of each frees the tensor memory
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::cluster_sync();
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

}  // namespace emb
