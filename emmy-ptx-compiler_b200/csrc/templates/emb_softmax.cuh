// Row-softmax template: one CTA per row, the row read from HBM once and held in registers
// across the three phases the IR spells (maximum, sum of exponentials, scaled write).
//
// The IR form it replaces is three cooperative loops over the same row, each re-loading it,
// with the block-reduction idiom after the first two. The order of every floating-point
// operation is the IR's: thread t owns elements t*VEC + k*BLOCK*VEC + j in increasing k, j;
// lanes combine by butterfly, warps by the tree (tests/oracle.py:150-166, :238-268); exp(x - m)
// of the second phase is the same expression as the third's, so it is computed once.
// HBM traffic is the algorithmic minimum: 4 bytes read and 4 bytes written per element.
#pragma once
#include "emb_reduce.cuh"

namespace emb {

template <int VEC> __device__ __forceinline__ void store_stream(float* p, const Vec<VEC>& r);
template <> __device__ __forceinline__ void store_stream<1>(float* p, const Vec<1>& r) {
    asm volatile("st.global.cs.f32 [%0], %1;" ::"l"(p), "f"(r.v[0]) : "memory");
}
template <> __device__ __forceinline__ void store_stream<2>(float* p, const Vec<2>& r) {
    asm volatile("st.global.cs.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(r.v[0]), "f"(r.v[1]) : "memory");
}
template <> __device__ __forceinline__ void store_stream<4>(float* p, const Vec<4>& r) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]),
                 "f"(r.v[3])
                 : "memory");
}

template <int BLOCK, int VEC, int COLS, bool STRICT>
__device__ __forceinline__ void softmax_row(const float* __restrict__ x, float* __restrict__ out, long long row) {
    constexpr int STEP = BLOCK * VEC;
    constexpr int TRIPS = (COLS + STEP - 1) / STEP;
    constexpr int WARPS = BLOCK / 32;
    constexpr int LANES = BLOCK < 32 ? BLOCK : 32;
    __shared__ float slab_m[WARPS > 0 ? WARPS : 1];
    __shared__ float slab_l[WARPS > 0 ? WARPS : 1];
    const float* xr = x + row * COLS;
    float* outr = out + row * COLS;
    const int c0 = threadIdx.x * VEC;

    Vec<VEC> v[TRIPS];
#pragma unroll
    for (int k = 0; k < TRIPS; ++k)
        if (c0 + k * STEP < COLS) v[k] = load_stream<VEC>(xr + c0 + k * STEP);

    float m = OpMax::identity();
#pragma unroll
    for (int k = 0; k < TRIPS; ++k)
        if (c0 + k * STEP < COLS)
#pragma unroll
            for (int j = 0; j < VEC; ++j) m = fmaxf(m, v[k].v[j]);
    if (!STRICT && LANES == 32) {
        m = warp_max_redux(m);
        if (WARPS > 1) {
            if ((threadIdx.x & 31) == 0) slab_m[threadIdx.x >> 5] = m;
            __syncthreads();
            m = tree_fold<OpMax, (WARPS > 1 ? WARPS : 1)>(slab_m);
        }
    } else {
        m = block_combine<OpMax, LANES, OpMax, (WARPS > 1 ? WARPS : 0)>(m, slab_m);
    }

    float l = 0.0f;
#pragma unroll
    for (int k = 0; k < TRIPS; ++k)
        if (c0 + k * STEP < COLS)
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                float e = exp_f32(sub(v[k].v[j], m));
                v[k].v[j] = e;
                l = add(l, e);
            }
    l = block_combine<OpAdd, LANES, OpAdd, (WARPS > 1 ? WARPS : 0)>(l, slab_l);
    const float inv = rcp(l);

#pragma unroll
    for (int k = 0; k < TRIPS; ++k)
        if (c0 + k * STEP < COLS) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[k].v[j] = mul(v[k].v[j], inv);
            store_stream<VEC>(outr + c0 + k * STEP, v[k]);
        }
}

}  // namespace emb
