// libemmyb200.so: module loading, launching and timing over the CUDA driver API.
// The driver library is opened at run time (dlopen), so the shared object loads on a machine
// without a GPU driver; every call then returns EMB_E_NO_DRIVER.

#include "emmy_b200.h"

#include <cuda.h>
#include <dlfcn.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

// The driver entry points used, resolved once through cuGetProcAddress.
struct Driver {
    bool ok = false;
    CUresult (*Init)(unsigned) = nullptr;
    CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
    CUresult (*DevicePrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
    CUresult (*CtxSetCurrent)(CUcontext) = nullptr;
    CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*FuncGetAttribute)(int*, CUfunction_attribute, CUfunction) = nullptr;
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
    CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
    CUresult (*EventCreate)(CUevent*, unsigned) = nullptr;
    CUresult (*EventRecord)(CUevent, CUstream) = nullptr;
    CUresult (*EventSynchronize)(CUevent) = nullptr;
    CUresult (*EventElapsedTime)(float*, CUevent, CUevent) = nullptr;
    CUresult (*EventDestroy)(CUevent) = nullptr;
    CUresult (*StreamSynchronize)(CUstream) = nullptr;
    CUresult (*MemsetD32Async)(CUdeviceptr, unsigned, size_t, CUstream) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
};

Driver g_drv;
std::once_flag g_once;
std::mutex g_ctx_mutex;
CUcontext g_ctx[64] = {};

void load_driver() {
    void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return;
    using GetProc = CUresult (*)(const char*, void**, int, cuuint64_t, CUdriverProcAddressQueryResult*);
    auto get = reinterpret_cast<GetProc>(dlsym(lib, "cuGetProcAddress_v2"));
    if (!get) return;
    bool all = true;
    auto want = [&](const char* name, auto& slot) {
        void* p = nullptr;
        CUdriverProcAddressQueryResult st;
        if (get(name, &p, 12080, CU_GET_PROC_ADDRESS_DEFAULT, &st) != CUDA_SUCCESS || !p) all = false;
        slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(p);
    };
    want("cuInit", g_drv.Init);
    want("cuDeviceGet", g_drv.DeviceGet);
    want("cuDevicePrimaryCtxRetain", g_drv.DevicePrimaryCtxRetain);
    want("cuCtxSetCurrent", g_drv.CtxSetCurrent);
    want("cuModuleLoadData", g_drv.ModuleLoadData);
    want("cuModuleUnload", g_drv.ModuleUnload);
    want("cuModuleGetFunction", g_drv.ModuleGetFunction);
    want("cuFuncGetAttribute", g_drv.FuncGetAttribute);
    want("cuFuncSetAttribute", g_drv.FuncSetAttribute);
    want("cuLaunchKernelEx", g_drv.LaunchKernelEx);
    want("cuTensorMapEncodeTiled", g_drv.TensorMapEncodeTiled);
    want("cuEventCreate", g_drv.EventCreate);
    want("cuEventRecord", g_drv.EventRecord);
    want("cuEventSynchronize", g_drv.EventSynchronize);
    want("cuEventElapsedTime", g_drv.EventElapsedTime);
    want("cuEventDestroy", g_drv.EventDestroy);
    want("cuStreamSynchronize", g_drv.StreamSynchronize);
    want("cuMemsetD32Async", g_drv.MemsetD32Async);
    want("cuGetErrorString", g_drv.GetErrorString);
    g_drv.ok = all;
}

bool driver() {
    std::call_once(g_once, load_driver);
    return g_drv.ok;
}

int check(CUresult r, const char* what) {
    if (r == CUDA_SUCCESS) return 0;
    const char* text = nullptr;
    if (g_drv.GetErrorString) g_drv.GetErrorString(r, &text);
    return fail(static_cast<int>(r), "%s: %s (CUresult %d)", what, text ? text : "unknown error", static_cast<int>(r));
}

#define NEED_DRIVER() \
    if (!driver()) return fail(EMB_E_NO_DRIVER, "the CUDA driver library (libcuda.so.1) is not available")

int launch_one(const emb_launch_t& k, CUstream stream) {
    if (!k.fn) return fail(EMB_E_ARGUMENT, "launch: null function");
    if (k.nparams < 0 || (k.nparams > 0 && !k.params)) return fail(EMB_E_ARGUMENT, "launch: bad parameter list");
    for (int i = 0; i < 3; ++i)
        if (k.grid[i] == 0 || k.block[i] == 0) return fail(EMB_E_ARGUMENT, "launch: zero grid or block extent");
    CUfunction fn = static_cast<CUfunction>(k.fn);
    if (k.smem_bytes > 48u * 1024u) {
        int r = check(g_drv.FuncSetAttribute(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                             static_cast<int>(k.smem_bytes)), "cuFuncSetAttribute(max dynamic shared)");
        if (r) return r;
    }
    CUlaunchConfig cfg;
    std::memset(&cfg, 0, sizeof cfg);
    cfg.gridDimX = k.grid[0], cfg.gridDimY = k.grid[1], cfg.gridDimZ = k.grid[2];
    cfg.blockDimX = k.block[0], cfg.blockDimY = k.block[1], cfg.blockDimZ = k.block[2];
    cfg.sharedMemBytes = k.smem_bytes;
    cfg.hStream = stream;
    CUlaunchAttribute attr[2];
    unsigned nattr = 0;
    if (k.flags & EMB_LAUNCH_PDL) {
        attr[nattr].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr[nattr].value.programmaticStreamSerializationAllowed = 1;
        ++nattr;
    }
    if (k.cluster_x > 1) {
        if (k.grid[0] % k.cluster_x) return fail(EMB_E_ARGUMENT, "launch: grid %u is not a multiple of the cluster size %u",
                                                 k.grid[0], k.cluster_x);
        attr[nattr].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attr[nattr].value.clusterDim.x = k.cluster_x;
        attr[nattr].value.clusterDim.y = 1;
        attr[nattr].value.clusterDim.z = 1;
        ++nattr;
    }
    if (nattr) {
        cfg.attrs = attr;
        cfg.numAttrs = nattr;
    }
    return check(g_drv.LaunchKernelEx(&cfg, fn, k.params, nullptr), "cuLaunchKernelEx");
}

}  // namespace

// for the other translation units of the library: record an error text for the calling thread
int emb_fail_text(int code, const char* text) { return fail(code, "%s", text); }

extern "C" {

int emb_abi_version(void) { return 2; }

const char* emb_last_error(void) { return g_error; }

int emb_init(int device) {
    NEED_DRIVER();
    if (device < 0 || device >= 64) return fail(EMB_E_ARGUMENT, "device %d out of range", device);
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    if (!g_ctx[device]) {
        int r = check(g_drv.Init(0), "cuInit");
        if (r) return r;
        CUdevice dev;
        if ((r = check(g_drv.DeviceGet(&dev, device), "cuDeviceGet"))) return r;
        if ((r = check(g_drv.DevicePrimaryCtxRetain(&g_ctx[device], dev), "cuDevicePrimaryCtxRetain"))) return r;
    }
    return check(g_drv.CtxSetCurrent(g_ctx[device]), "cuCtxSetCurrent");
}

int emb_module_load(const void* image, size_t nbytes, void** module_out) {
    NEED_DRIVER();
    if (!image || !nbytes || !module_out) return fail(EMB_E_ARGUMENT, "module_load: null image or output");
    CUmodule mod = nullptr;
    int r = check(g_drv.ModuleLoadData(&mod, image), "cuModuleLoadData");
    if (r) return r;
    *module_out = mod;
    return 0;
}

int emb_module_unload(void* module) {
    NEED_DRIVER();
    if (!module) return 0;
    return check(g_drv.ModuleUnload(static_cast<CUmodule>(module)), "cuModuleUnload");
}

int emb_get_function(void* module, const char* entry, void** fn_out) {
    NEED_DRIVER();
    if (!module || !entry || !fn_out) return fail(EMB_E_ARGUMENT, "get_function: null argument");
    CUfunction fn = nullptr;
    int r = check(g_drv.ModuleGetFunction(&fn, static_cast<CUmodule>(module), entry), entry);
    if (r) return r;
    *fn_out = fn;
    return 0;
}

int emb_function_info(void* fn, int* registers, int* static_smem, int* local_bytes, int* max_threads) {
    NEED_DRIVER();
    if (!fn) return fail(EMB_E_ARGUMENT, "function_info: null function");
    CUfunction f = static_cast<CUfunction>(fn);
    struct { int* out; CUfunction_attribute attr; } q[] = {
        {registers, CU_FUNC_ATTRIBUTE_NUM_REGS}, {static_smem, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES},
        {local_bytes, CU_FUNC_ATTRIBUTE_LOCAL_SIZE_BYTES}, {max_threads, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK}};
    for (auto& e : q) {
        if (!e.out) continue;
        int r = check(g_drv.FuncGetAttribute(e.out, e.attr, f), "cuFuncGetAttribute");
        if (r) return r;
    }
    return 0;
}

int emb_launch(const emb_launch_t* launch, void* stream) {
    NEED_DRIVER();
    if (!launch) return fail(EMB_E_ARGUMENT, "launch: null descriptor");
    return launch_one(*launch, static_cast<CUstream>(stream));
}

int emb_launch_chain(const emb_launch_t* launches, int n, void* stream) {
    NEED_DRIVER();
    if (!launches || n <= 0) return fail(EMB_E_ARGUMENT, "launch_chain: empty chain");
    for (int i = 0; i < n; ++i) {
        int r = launch_one(launches[i], static_cast<CUstream>(stream));
        if (r) return r;
    }
    return 0;
}

int emb_time_chain(const emb_launch_t* launches, int n, void* stream, int warmup, int iters, void* flush_ptr,
                   size_t flush_bytes, float* us_out) {
    NEED_DRIVER();
    if (!launches || n <= 0 || iters <= 0 || warmup < 0 || !us_out)
        return fail(EMB_E_ARGUMENT, "time_chain: bad chain, counts or output");
    CUstream s = static_cast<CUstream>(stream);
    std::vector<CUevent> ev(2 * static_cast<size_t>(iters), nullptr);
    int r = 0;
    for (auto& e : ev)
        if ((r = check(g_drv.EventCreate(&e, CU_EVENT_DEFAULT), "cuEventCreate"))) break;
    for (int i = 0; !r && i < warmup; ++i) r = emb_launch_chain(launches, n, stream);
    for (int i = 0; !r && i < iters; ++i) {
        if (flush_ptr && flush_bytes >= 4)
            r = check(g_drv.MemsetD32Async(reinterpret_cast<CUdeviceptr>(flush_ptr), 0u, flush_bytes / 4, s),
                      "cuMemsetD32Async(flush)");
        if (!r) r = check(g_drv.EventRecord(ev[2 * i], s), "cuEventRecord");
        if (!r) r = emb_launch_chain(launches, n, stream);
        if (!r) r = check(g_drv.EventRecord(ev[2 * i + 1], s), "cuEventRecord");
    }
    if (!r) r = check(g_drv.StreamSynchronize(s), "cuStreamSynchronize");
    for (int i = 0; !r && i < iters; ++i) {
        float ms = 0.f;
        r = check(g_drv.EventElapsedTime(&ms, ev[2 * i], ev[2 * i + 1]), "cuEventElapsedTime");
        us_out[i] = ms * 1000.f;
    }
    for (auto& e : ev)
        if (e) g_drv.EventDestroy(e);
    return r;
}

int emb_time_rotating(const emb_launch_t* launches, int chain_len, int n_sets, void* stream, int warmup, int iters,
                      int batch, float* us_out) {
    NEED_DRIVER();
    if (!launches || chain_len <= 0 || n_sets <= 0 || iters <= 0 || warmup < 0 || batch <= 0 || !us_out)
        return fail(EMB_E_ARGUMENT, "time_rotating: bad chain, counts or output");
    CUstream s = static_cast<CUstream>(stream);
    std::vector<CUevent> ev(2 * static_cast<size_t>(iters), nullptr);
    int r = 0;
    for (auto& e : ev)
        if ((r = check(g_drv.EventCreate(&e, CU_EVENT_DEFAULT), "cuEventCreate"))) break;
    int run = 0;
    for (int i = 0; !r && i < warmup; ++i, ++run) r = emb_launch_chain(launches + (run % n_sets) * chain_len, chain_len, stream);
    for (int i = 0; !r && i < iters; ++i) {
        r = check(g_drv.EventRecord(ev[2 * i], s), "cuEventRecord");
        for (int b = 0; !r && b < batch; ++b, ++run)
            r = emb_launch_chain(launches + (run % n_sets) * chain_len, chain_len, stream);
        if (!r) r = check(g_drv.EventRecord(ev[2 * i + 1], s), "cuEventRecord");
    }
    if (!r) r = check(g_drv.StreamSynchronize(s), "cuStreamSynchronize");
    for (int i = 0; !r && i < iters; ++i) {
        float ms = 0.f;
        r = check(g_drv.EventElapsedTime(&ms, ev[2 * i], ev[2 * i + 1]), "cuEventElapsedTime");
        us_out[i] = ms * 1000.f / static_cast<float>(batch);
    }
    for (auto& e : ev)
        if (e) g_drv.EventDestroy(e);
    return r;
}

int emb_tensor_map(void* map_out, const void* base, int dtype, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
    NEED_DRIVER();
    if (!map_out || !base || !dims || !box || rank < 1 || rank > 5 || (rank > 1 && !strides_bytes))
        return fail(EMB_E_ARGUMENT, "tensor_map: null argument or rank outside 1..5");
    if (reinterpret_cast<uintptr_t>(map_out) % 64) return fail(EMB_E_ARGUMENT, "tensor_map: output must be 64-byte aligned");
    if (reinterpret_cast<uintptr_t>(base) % 16) return fail(EMB_E_ARGUMENT, "tensor_map: base must be 16-byte aligned");
    static const CUtensorMapDataType types[] = {CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                                CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                                CU_TENSOR_MAP_DATA_TYPE_UINT16, CU_TENSOR_MAP_DATA_TYPE_UINT32};
    static const unsigned width[] = {1, 2, 2, 4, 2, 4};
    static const CUtensorMapSwizzle swz[] = {CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                                             CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_SWIZZLE_128B};
    if (dtype < 0 || dtype > 5 || swizzle < 0 || swizzle > 3) return fail(EMB_E_ARGUMENT, "tensor_map: bad dtype or swizzle");
    cuuint64_t gdim[5], gstride[5];
    cuuint32_t bdim[5], estride[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estride[i] = 1;
        if (box[i] == 0 || box[i] > 256) return fail(EMB_E_ARGUMENT, "tensor_map: box[%d]=%u outside 1..256", i, box[i]);
        if (i + 1 < rank) {
            gstride[i] = strides_bytes[i];
            if (gstride[i] % 16) return fail(EMB_E_ARGUMENT, "tensor_map: stride %d is not a multiple of 16 bytes", i);
        }
    }
    if ((static_cast<uint64_t>(box[0]) * width[dtype]) % 16)
        return fail(EMB_E_ARGUMENT, "tensor_map: inner box extent is not a multiple of 16 bytes");
    return check(g_drv.TensorMapEncodeTiled(static_cast<CUtensorMap*>(map_out), types[dtype], static_cast<cuuint32_t>(rank),
                                            const_cast<void*>(base), gdim, gstride, bdim, estride,
                                            CU_TENSOR_MAP_INTERLEAVE_NONE, swz[swizzle],
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                 "cuTensorMapEncodeTiled");
}

}  // extern "C"
