// e4m3 weight decode for the MLP template: codes[R][C] (one byte each) -> bf16 values, TRANSPOSED to
// out[C][R], so that a weight matrix stored [k][n] (n contiguous) becomes the K-major [n][k] operand the
// matmul template loads. The decode is the reference's `from_f8e4m3` (emmy_ptx/elementwise.py:100-110):
// exact widening through f16 (every e4m3 value is a bf16 value too), the per-tensor scale stays outside.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace emb {

__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(unsigned short pair) {
    uint32_t halves;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(halves) : "h"(pair));
    const __half2 h2 = *reinterpret_cast<const __half2*>(&halves);
    const __nv_bfloat162 b2 = __floats2bfloat162_rn(__low2float(h2), __high2float(h2));
    return *reinterpret_cast<const uint32_t*>(&b2);
}

// The grid for `rows` x `cols` codes: one CTA of 256 threads per 64 x 128 tile when the shape divides (the streaming path),
// else per 64 x 64 tile (the general path below).
__host__ __device__ constexpr bool dequant_streams(int rows, int cols) { return rows % 64 == 0 && cols % 128 == 0; }

// Streaming path: a 64-row x 128-column tile per CTA. Every global access is a whole 128-byte line (a row segment of
// 128 codes in, 64 bf16 of an output row out); the tile is transposed through shared memory as 16-byte chunks whose
// position in a row is XORed with the 16-column group of that row, rows 144 bytes apart, so that neither the 2-byte
// transposing stores nor the 16-byte reads meet a bank conflict.
__device__ __forceinline__ void dequant_transpose_tile_64x128(const uint8_t* __restrict__ codes, __nv_bfloat16* __restrict__ out,
                                                              int rows, int cols) {
    constexpr int PITCH = 64 + 8;  // bf16 per shared row (an output row's 64 values + 16 bytes)
    __shared__ __align__(16) __nv_bfloat16 tile[128 * PITCH];
    const int tiles_c = cols / 128;
    const int r0 = (blockIdx.x / tiles_c) * 64, c0 = (blockIdx.x % tiles_c) * 128;
    const int seg = threadIdx.x & 7;  // 16 columns: c0 + 16 seg ..
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int r = (threadIdx.x >> 3) + 32 * pass;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(codes + static_cast<size_t>(r0 + r) * cols + c0 + 16 * seg));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        const int chunk = (r >> 3) ^ seg;  // (all 16 columns of this thread share the column group `seg`)
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t two = e4m3x2_to_bf16x2(static_cast<unsigned short>(w[q] >> (16 * h)));
                const int c = 16 * seg + 4 * q + 2 * h;
                unsigned short* at = reinterpret_cast<unsigned short*>(tile) + c * PITCH + chunk * 8 + (r & 7);
                at[0] = static_cast<unsigned short>(two);
                at[PITCH] = static_cast<unsigned short>(two >> 16);
            }
    }
    __syncthreads();
    const int c = threadIdx.x >> 1, half = threadIdx.x & 1;  // an output row and 32 of its 64 values
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(c0 + c) * rows + r0 + 32 * half);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int chunk = (4 * half + k) ^ ((c >> 4) & 7);
        dst[k] = *reinterpret_cast<const uint4*>(tile + c * PITCH + chunk * 8);
    }
}

// General path: 64 x 64 tile per CTA of 256 threads, through shared memory: 16-byte global reads along C where they are
// aligned, 16-byte global writes along R; any shape.
__device__ __forceinline__ void dequant_transpose_tile_64x64(const uint8_t* __restrict__ codes, __nv_bfloat16* __restrict__ out, int rows,
                                                             int cols) {
    __shared__ __nv_bfloat16 tile[64][64 + 8];
    const int tiles_c = (cols + 63) / 64;
    const int r0 = (blockIdx.x / tiles_c) * 64, c0 = (blockIdx.x % tiles_c) * 64;
    {
        const int r = threadIdx.x >> 2, cq = (threadIdx.x & 3) * 16;  // 64 rows x 4 sixteen-byte segments
        uint32_t w[4] = {0, 0, 0, 0};
        if (r0 + r < rows && c0 + cq + 16 <= cols && (cols & 15) == 0) {
            const uint4 v = *reinterpret_cast<const uint4*>(codes + static_cast<size_t>(r0 + r) * cols + c0 + cq);
            w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
        } else if (r0 + r < rows) {
            for (int j = 0; j < 16; ++j)
                if (c0 + cq + j < cols) w[j >> 2] |= static_cast<uint32_t>(codes[static_cast<size_t>(r0 + r) * cols + c0 + cq + j]) << (8 * (j & 3));
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t two = e4m3x2_to_bf16x2(static_cast<unsigned short>(w[q] >> (16 * h)));
                *reinterpret_cast<unsigned short*>(&tile[r][cq + 4 * q + 2 * h]) = static_cast<unsigned short>(two);
                *reinterpret_cast<unsigned short*>(&tile[r][cq + 4 * q + 2 * h + 1]) = static_cast<unsigned short>(two >> 16);
            }
    }
    __syncthreads();
    {
        const int c = threadIdx.x >> 2, rq = (threadIdx.x & 3) * 16;  // 64 output rows (= input columns) x 4 segments of 16
        if (c0 + c < cols) {
            __nv_bfloat16* dst = out + static_cast<size_t>(c0 + c) * rows + r0 + rq;
            if (r0 + rq + 16 <= rows && (rows & 7) == 0) {
                __align__(16) __nv_bfloat16 v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = tile[rq + j][c];
                reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(v)[0];
                reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(v)[1];
            } else {
                for (int j = 0; j < 16; ++j)
                    if (r0 + rq + j < rows) dst[j] = tile[rq + j][c];
            }
        }
    }
}

// WAIT_PRIOR: the kernel is launched programmatically dependent on the kernel before it in the stream, whose data it does
// not need: it runs beside that kernel, and ONE thread waits for it at the very end, so that this grid - and with it
// whatever the stream holds next - completes only after that kernel has.
// STREAM: the 64 x 128 streaming path (the host sizes the grid for it and asks for it only when dequant_streams(rows, cols)).
// A decode that runs BESIDE a matmul keeps the general path: its 9 KB of shared memory let three of its CTAs share an SM with
// the matmul's CTA, the streaming path's 18 KB only one.
template <bool WAIT_PRIOR = false, bool STREAM = false>
__device__ __forceinline__ void dequant_transpose_e4m3(const uint8_t* __restrict__ codes, __nv_bfloat16* __restrict__ out, int rows,
                                                       int cols) {
    if (STREAM)
        dequant_transpose_tile_64x128(codes, out, rows, cols);
    else
        dequant_transpose_tile_64x64(codes, out, rows, cols);
    if (WAIT_PRIOR && blockIdx.x == 0 && threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace emb
