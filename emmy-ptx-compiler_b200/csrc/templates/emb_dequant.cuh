// e4m3 weight decode for the MLP template: codes[R][C] (one byte each) -> bf16 values, TRANSPOSED to
// out[C][R], so that a weight matrix stored [k][n] (n contiguous) becomes the K-major [n][k] operand the
// matmul template loads. The decode is the reference's `from_f8e4m3` (emmy_ptx/elementwise.py:100-110):
// exact widening through f16 (every e4m3 value is a bf16 value too), the per-tensor scale stays outside.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace emb {

// 64 x 64 tile per CTA of 256 threads, through shared memory: 16-byte global reads along C, 16-byte global
// writes along R.
// WAIT_PRIOR: the kernel is launched programmatically dependent on the kernel before it in the stream, whose data it does
// not need: it runs beside that kernel, and ONE thread waits for it at the very end, so that this grid - and with it
// whatever the stream holds next - completes only after that kernel has.
template <bool WAIT_PRIOR = false>
__device__ __forceinline__ void dequant_transpose_e4m3(const uint8_t* __restrict__ codes, __nv_bfloat16* __restrict__ out, int rows,
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
                const unsigned short pair = static_cast<unsigned short>(w[q] >> (16 * h));
                uint32_t halves;
                asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(halves) : "h"(pair));
                const __half2 h2 = *reinterpret_cast<const __half2*>(&halves);
                tile[r][cq + 4 * q + 2 * h] = __float2bfloat16_rn(__low2float(h2));
                tile[r][cq + 4 * q + 2 * h + 1] = __float2bfloat16_rn(__high2float(h2));
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
    if (WAIT_PRIOR && blockIdx.x == 0 && threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace emb
