// emb_array_sum_f32_static: the two-kernel f32 array sum with its scratch (the per-block partials) in a
// fixed device array of this library instead of a buffer the caller allocates.
//
// Who needs it: hosts that hold device pointers but may not allocate device memory themselves - a
// plugin running inside another framework's memory pool, a real-time or capture-phase caller where
// cudaMalloc's implicit synchronisation is forbidden, an embedding with a fixed memory budget. The
// ordinary path (emb_launch of the compiled k_sum__partial / k_sum_1_reduce chain) needs a caller-owned
// `sum__partial` buffer of one float per block; here that buffer is `g_partials` below.
//
// The kernels instantiate the same reduction template in its in-order form, so for the same `blocks`
// the result is bit for bit the one of the compiled chain under --strict.

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdio>

#define EMB_STRICT 1
#include "emb_reduce.cuh"
#include "emmy_b200.h"

int emb_fail_text(int code, const char* text);  // shim.cpp

namespace {

constexpr int THREADS = 256;
constexpr int MAX_DEVICES = 64;

// The scratch: one partial per block of the first kernel. Every GPU that loads the library holds these
// EMB_STATIC_SUM_MAX_BLOCKS * 4 bytes until the process exits. In HOST code this name is only a stand-in
// for the symbol, not a device address: the address comes from cudaGetSymbolAddress, per device.
static __device__ __align__(256) float g_partials[EMB_STATIC_SUM_MAX_BLOCKS];

// (looked up once per device; host threads may race to do so, and all of them store the same address)
std::atomic<float*> g_partials_address[MAX_DEVICES] = {};

__global__ void __launch_bounds__(THREADS) sum_partials_static(const float* __restrict__ x, long long n, float* __restrict__ partials) {
    __shared__ float slab[THREADS / 32];
    const long long start = (static_cast<long long>(blockIdx.x) * THREADS + threadIdx.x) * 4;
    const long long step = static_cast<long long>(gridDim.x) * THREADS * 4;
    float acc = emb::strided_fold<4, emb::OpAdd, 8, true>(x, start, step, n);
    acc = emb::block_combine<emb::OpAdd, 32, emb::OpAdd, THREADS / 32>(acc, slab);
    if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

__global__ void __launch_bounds__(THREADS) sum_final_static(const float* __restrict__ partials, int count, float* __restrict__ out) {
    __shared__ float slab[THREADS / 32];
    float acc = emb::strided_fold<1, emb::OpAdd, 8, true>(partials, threadIdx.x, THREADS, count);
    acc = emb::block_combine<emb::OpAdd, 32, emb::OpAdd, THREADS / 32>(acc, slab);
    if (threadIdx.x == 0) out[0] = acc;
}

int cuda_fail(cudaError_t e, const char* what) {
    char text[256];
    snprintf(text, sizeof text, "%s: %s", what, cudaGetErrorString(e));
    return emb_fail_text(static_cast<int>(e) > 0 ? static_cast<int>(e) : EMB_E_ARGUMENT, text);
}

}  // namespace

extern "C" int emb_array_sum_f32_static(const float* x, uint64_t n, uint32_t blocks, float* sum_out, void* stream) {
    if (!x || !sum_out) return emb_fail_text(EMB_E_ARGUMENT, "array_sum_static: null input or output pointer");
    if (blocks == 0 || blocks > EMB_STATIC_SUM_MAX_BLOCKS) {
        char text[160];
        snprintf(text, sizeof text, "array_sum_static: %u blocks, but the built-in scratch holds at most %d partials", blocks,
                 EMB_STATIC_SUM_MAX_BLOCKS);
        return emb_fail_text(EMB_E_ARGUMENT, text);
    }
    if (n == 0 || n % 4 != 0 || n > (1ull << 40) || (reinterpret_cast<uintptr_t>(x) & 15))
        return emb_fail_text(EMB_E_ARGUMENT, "array_sum_static: n must be a positive multiple of 4 (at most 2^40) and x 16-byte aligned");
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (device < 0 || device >= MAX_DEVICES) return emb_fail_text(EMB_E_ARGUMENT, "array_sum_static: device index out of range");
    float* partials = g_partials_address[device].load(std::memory_order_relaxed);
    if (!partials) {
        // set-up, once per device, with that device current: the symbol's address on THIS device
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&partials), g_partials);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_partials)");
        g_partials_address[device].store(partials, std::memory_order_relaxed);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    sum_partials_static<<<blocks, THREADS, 0, s>>>(x, static_cast<long long>(n), partials);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch of sum_partials_static");
    sum_final_static<<<1, THREADS, 0, s>>>(partials, static_cast<int>(blocks), sum_out);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch of sum_final_static");
    return 0;
}
