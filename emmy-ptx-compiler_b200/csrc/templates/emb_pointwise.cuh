// Streaming pieces of the pointwise template: a thread moves RUNS of four consecutive elements
// between global memory and registers with one access per run (16 bytes for 32-bit elements),
// read-only data through the non-coherent path without taking L1 lines (ld.global.nc.L1::no_allocate),
// results with the evict-first hint (st.global.cs): every byte is used once.
//
// The arithmetic between the load and the store is NOT here: it is the statement lowering's, one C++
// expression per IR statement with the reference's semantics (emmy_ptx/elementwise.py:185-214: IEEE
// round-to-nearest basic operations, fmaxf/fminf for maximum/minimum, numpy's fixed-width integers),
// so a kernel on this template gives the same bits as the same kernel lowered statement by statement.
// What the template changes is only which thread owns which cells and how they travel.
#pragma once
#include <stdint.h>

namespace emb {

// Four elements of T as they lie in memory.
template <class T> struct alignas(sizeof(T) * 4 <= 16 ? sizeof(T) * 4 : 16) Run4 {
    T v[4];
};

template <int BYTES> struct RawRun;
template <> struct RawRun<4> { uint32_t w[1]; };
template <> struct RawRun<8> { uint32_t w[2]; };
template <> struct RawRun<16> { uint32_t w[4]; };
template <> struct RawRun<32> { uint32_t w[8]; };

__device__ __forceinline__ void load_raw(const void* p, RawRun<4>& r) {
    asm volatile("ld.global.nc.L1::no_allocate.b32 %0, [%1];" : "=r"(r.w[0]) : "l"(p));
}
__device__ __forceinline__ void load_raw(const void* p, RawRun<8>& r) {
    asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0, %1}, [%2];" : "=r"(r.w[0]), "=r"(r.w[1]) : "l"(p));
}
__device__ __forceinline__ void load_raw(const void* p, RawRun<16>& r) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3])
                 : "l"(p));
}
__device__ __forceinline__ void load_raw(const void* p, RawRun<32>& r) {
    const char* q = static_cast<const char*>(p);
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3])
                 : "l"(q));
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.w[4]), "=r"(r.w[5]), "=r"(r.w[6]), "=r"(r.w[7])
                 : "l"(q + 16));
}

__device__ __forceinline__ void store_raw(void* p, const RawRun<4>& r) {
    asm volatile("st.global.cs.b32 [%0], %1;" ::"l"(p), "r"(r.w[0]) : "memory");
}
__device__ __forceinline__ void store_raw(void* p, const RawRun<8>& r) {
    asm volatile("st.global.cs.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(r.w[0]), "r"(r.w[1]) : "memory");
}
__device__ __forceinline__ void store_raw(void* p, const RawRun<16>& r) {
    asm volatile("st.global.cs.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(r.w[0]), "r"(r.w[1]), "r"(r.w[2]), "r"(r.w[3])
                 : "memory");
}
__device__ __forceinline__ void store_raw(void* p, const RawRun<32>& r) {
    char* q = static_cast<char*>(p);
    asm volatile("st.global.cs.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(q), "r"(r.w[0]), "r"(r.w[1]), "r"(r.w[2]), "r"(r.w[3])
                 : "memory");
    asm volatile("st.global.cs.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(q + 16), "r"(r.w[4]), "r"(r.w[5]), "r"(r.w[6]), "r"(r.w[7])
                 : "memory");
}

// `p` must be aligned to the run (4 * sizeof(T) bytes, 16 for the 64-bit types).
template <class T> __device__ __forceinline__ Run4<T> load_run(const T* p) {
    RawRun<sizeof(T) * 4> raw;
    load_raw(p, raw);
    Run4<T> run;
    __builtin_memcpy(&run, &raw, sizeof(raw));
    return run;
}

template <class T> __device__ __forceinline__ void store_run(T* p, const Run4<T>& run) {
    RawRun<sizeof(T) * 4> raw;
    __builtin_memcpy(&raw, &run, sizeof(raw));
    store_raw(p, raw);
}

}  // namespace emb
