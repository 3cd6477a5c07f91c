// Block-reduction template: a per-thread strided fold over global memory, a butterfly over the
// lanes, one shared slab entry per warp, and a tree over the warps behind ONE barrier.
//
// It is the sm_100a form of the reference's reduction lowering: the cooperative idiom
// StridedLoop{Load; Accum} -> WarpShuffle -> Smem -> Cond(lane==0){Write} -> Sync -> TreeHalve
// (examples/r01_array_sum/k_sum_1_reduce.ir.txt:1-12), its butterfly (emmy_ptx/lower.py:1268-1305),
// its one-barrier tree in which every thread folds all the warps' partials in the tree's own order
// (emmy_ptx/lower.py:1334-1350), and its 16-byte global loads (emmy_ptx/regroup.py:235-246).
// With STRICT every result is bit for bit what the IR's order of operations gives
// (tests/oracle.py:150-166 the fold, :238-245 the butterfly, :247-268 the tree); without it the
// per-thread fold runs on independent accumulators that are merged at the end.
#pragma once
#include "emb_ops.cuh"

namespace emb {

template <int VEC> struct Vec;
template <> struct Vec<1> { float v[1]; };
template <> struct Vec<2> { float v[2]; };
template <> struct Vec<4> { float v[4]; };

// Read-only, streaming: the data is used once, so it does not take L1 lines from anything else.
template <int VEC> __device__ __forceinline__ Vec<VEC> load_stream(const float* p);
template <> __device__ __forceinline__ Vec<1> load_stream<1>(const float* p) {
    Vec<1> r;
    asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(r.v[0]) : "l"(p));
    return r;
}
template <> __device__ __forceinline__ Vec<2> load_stream<2>(const float* p) {
    Vec<2> r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.f32 {%0, %1}, [%2];" : "=f"(r.v[0]), "=f"(r.v[1]) : "l"(p));
    return r;
}
template <> __device__ __forceinline__ Vec<4> load_stream<4>(const float* p) {
    Vec<4> r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3])
                 : "l"(p));
    return r;
}

// Butterfly over aligned groups of LEN lanes: distance LEN/2, ..., 1; mine (+) partner's.
template <class Op, int LEN> __device__ __forceinline__ float warp_butterfly(float v) {
#pragma unroll
    for (int w = LEN / 2; w > 0; w >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, w));
    return v;
}

// The whole warp's maximum in one instruction. Order-free, so equal to the butterfly except
// for which of two zeros or NaNs survives; used where only the value matters.
__device__ __forceinline__ float warp_max_redux(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

// The tree over LEN slab entries, level by level as TreeHalve defines it (slot t takes
// slot t (+) slot t+half for t < half; half = LEN/2, ..., 1), computed by every thread in
// registers from one read of the slab: same operations in the same order, no further barrier.
template <class Op, int LEN> __device__ __forceinline__ float tree_fold(const float* slab) {
    float s[LEN];
#pragma unroll
    for (int i = 0; i < LEN; ++i) s[i] = slab[i];
#pragma unroll
    for (int half = LEN / 2; half > 0; half >>= 1) {
#pragma unroll
        for (int t = 0; t < half; ++t) s[t] = Op::apply(s[t], s[t + half]);
    }
    return s[0];
}

// What a fold does to a loaded value before folding it; the default folds the value itself.
struct MapIdentity {
    __device__ __forceinline__ float operator()(float v) const { return v; }
};

// Per-thread fold of map(x[i + j]), j < VEC, for i = start, start + step, ... < end.
//
// The trips are taken UNROLL at a time with every load of the round issued before the first
// add (a thread keeps UNROLL * VEC * 4 bytes in flight); trips past `end` are predicated off, so
// a ragged last round costs no serial tail. STRICT: one accumulator, the IR's order (a skipped
// trip adds nothing, not even a zero). Otherwise UNROLL * VEC independent accumulators, merged
// at the end.
template <int VEC, class Fold, int UNROLL, bool STRICT, class Map = MapIdentity>
__device__ __forceinline__ float strided_fold(const float* __restrict__ x, long long start, long long step, long long end,
                                              Map map = Map()) {
    float a[STRICT ? 1 : UNROLL][STRICT ? 1 : VEC];
#pragma unroll
    for (int u = 0; u < (STRICT ? 1 : UNROLL); ++u)
#pragma unroll
        for (int j = 0; j < (STRICT ? 1 : VEC); ++j) a[u][j] = Fold::identity();
    for (long long i = start; i < end; i += UNROLL * step) {
        Vec<VEC> v[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            ok[u] = i + u * step < end;
            if (ok[u]) v[u] = load_stream<VEC>(x + i + u * step);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
            if (ok[u]) {
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    float& acc = a[STRICT ? 0 : u][STRICT ? 0 : j];
                    acc = Fold::apply(acc, map(v[u].v[j]));
                }
            }
    }
    if (!STRICT) {
#pragma unroll
        for (int u = 1; u < UNROLL; ++u)
#pragma unroll
            for (int j = 0; j < VEC; ++j) a[0][j] = Fold::apply(a[0][j], a[u][j]);
#pragma unroll
        for (int j = 1; j < VEC; ++j) a[0][0] = Fold::apply(a[0][0], a[0][j]);
    }
    return a[0][0];
}

// Lanes, then warps. `slab` holds TREE_LEN floats of shared memory (unused when TREE_LEN == 0).
template <class Shuffle, int SHUFFLE_LEN, class Tree, int TREE_LEN>
__device__ __forceinline__ float block_combine(float acc, float* slab) {
    acc = warp_butterfly<Shuffle, SHUFFLE_LEN>(acc);
    if (TREE_LEN > 0) {
        if ((threadIdx.x & 31) == 0) slab[threadIdx.x >> 5] = acc;
        __syncthreads();
        acc = tree_fold<Tree, (TREE_LEN > 0 ? TREE_LEN : 1)>(slab);
    }
    return acc;
}

}  // namespace emb
