/*
 * emmy_b200.h - C ABI of libemmyb200.so, the launch side of the B200 backend.
 *
 * What it replaces. The reference compiler writes PTX text to stdout and stops
 * there; assembling and launching happen in a remote HTTP service that is not
 * part of it (tools/run_suite.py:77-92: POST /compile {ptx} -> cubin id and
 * register counts; POST /run {entry, grid, block, smem_bytes, zero_outputs,
 * args, warmup, iters} -> median_us and outputs; the same two calls in
 * tests/test_gpu_lowering.py:70-80 and tests/test_oracle.py:236-253). This
 * library is the local stand-in for that service: it loads a module image
 * (PTX text or a cubin made by ptxas), resolves an entry point, launches it on
 * caller-owned device buffers with the geometry of meta.json, and times it
 * with CUDA events. It is a thin layer over the CUDA driver API
 * (cuModuleLoadData, cuLaunchKernelEx, cuTensorMapEncodeTiled).
 *
 * Conventions. Plain C types only. Every function returns 0 on success, a
 * CUresult value (> 0) when the driver refused, or a negative EMB_E_* code;
 * emb_last_error() then gives a text for the calling thread. The caller owns
 * all device memory (the Python host passes torch tensors' data pointers);
 * the library owns the modules it loaded until emb_module_unload. The library
 * uses the device's primary context, the one the CUDA runtime and torch use,
 * so pointers and streams are interchangeable. Calls are thread-safe as far
 * as the driver's are; there is no global state beyond the context, with one
 * exception: emb_array_sum_f32_static keeps a device array per GPU and a
 * process-wide table of its addresses, and, being written against the CUDA
 * runtime, returns cudaError_t values (> 0) where the others return CUresult.
 */
#ifndef EMMY_B200_H
#define EMMY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EMB_E_NO_DRIVER (-1)  /* libcuda could not be loaded (no GPU driver on this machine) */
#define EMB_E_ARGUMENT (-2)   /* an argument is out of range; see emb_last_error() */
#define EMB_E_DEVICE_STATUS (-3) /* a kernel reported a bounded wait that ran out (status word non-zero) */

/* Element types of a tensor map (values of CUtensorMapDataType are not exposed). */
enum { EMB_U8 = 0, EMB_F16 = 1, EMB_BF16 = 2, EMB_F32 = 3, EMB_U16 = 4, EMB_U32 = 5 };
/* Shared-memory swizzle of a tensor-map box. */
enum { EMB_SWIZZLE_NONE = 0, EMB_SWIZZLE_32B = 1, EMB_SWIZZLE_64B = 2, EMB_SWIZZLE_128B = 3 };

/* One kernel launch: what the runner's POST /run carries per kernel
 * (tools/run_suite.py:86-92: entry, grid, block, smem_bytes, args), with
 * `cluster_x` for modules that ask for thread-block clusters
 * (emmy_ptx/ptx.py:294-295 .reqnctapercluster). `params[i]` points at the
 * i-th kernel parameter's value: an 8-byte device pointer for a buffer
 * (the reference's only parameter kind, `.param .u64 p_<buffer>`,
 * emmy_ptx/ptx.py:288), or a 128-byte tensor map made by emb_tensor_map.
 * A module's `status` parameter is a caller-owned buffer of 8 zeroed 32-bit
 * words: [0..2] what a bounded wait that gave up recorded (code, CTA, step),
 * [4..5] work counters a persistent kernel uses and re-zeroes itself. */
typedef struct emb_launch_t {
    void* fn;
    uint32_t grid[3];
    uint32_t block[3];
    uint32_t cluster_x;  /* 0 or 1: no cluster attribute */
    uint32_t smem_bytes; /* dynamic shared memory */
    void** params;
    int32_t nparams;
    uint32_t flags; /* EMB_LAUNCH_* bits */
} emb_launch_t;

/* Programmatic dependent launch: the kernel may be scheduled while the kernel
 * before it in the stream is still running, and itself waits
 * (griddepcontrol.wait) before it touches that kernel's results. For a kernel
 * whose inputs are another kernel's `intermediate` outputs (meta.json,
 * tools/run_suite.py:81-85): hides the second launch's latency. */
#define EMB_LAUNCH_PDL 1u

/* Bind the calling thread to `device`'s primary context (retained once per
 * device). Must be called before the other functions; cheap to repeat. */
int emb_init(int device);

/* POST /compile's job after ptxas (tools/run_suite.py:77-80): make a module
 * from PTX text (NUL-terminated, JIT-compiled by the driver) or from a cubin
 * image. `nbytes` is the image size (for the record; the driver reads the
 * image's own length). */
int emb_module_load(const void* image, size_t nbytes, void** module_out);
int emb_module_unload(void* module);

/* The entry point named by meta.json's `entry` (tools/run_suite.py:88). */
int emb_get_function(void* module, const char* entry, void** fn_out);

/* Registers per thread, static shared bytes, local (spill) bytes per thread,
 * max threads per block: the `registers` figure POST /compile returns
 * (tools/run_suite.py:80,93) and its companions. Any out pointer may be NULL. */
int emb_function_info(void* fn, int* registers, int* static_smem, int* local_bytes, int* max_threads);

/* Launch one kernel / a chain of kernels in order on `stream` (a CUstream /
 * cudaStream_t; NULL is the legacy default stream). Raises the function's
 * dynamic shared memory limit when smem_bytes needs it. Asynchronous. */
int emb_launch(const emb_launch_t* launch, void* stream);
int emb_launch_chain(const emb_launch_t* launches, int n, void* stream);

/* POST /run's timing (tools/run_suite.py:91: warm-ups, then `iters` timed
 * launches; the reference reports their median): run the chain `warmup` times,
 * then `iters` times with a CUDA event pair around each run of the chain on
 * `stream`, and write the `iters` durations in microseconds to `us_out`.
 * If `flush_ptr` is non-NULL, `flush_bytes` of it are overwritten before every
 * timed run (outside the event pair) to evict the L2 cache. Synchronous. */
int emb_time_chain(const emb_launch_t* launches, int n, void* stream, int warmup, int iters,
                   void* flush_ptr, size_t flush_bytes, float* us_out);

/* The same, over `n_sets` copies of the chain bound to distinct buffers
 * (`launches` holds n_sets * chain_len descriptors, set after set): run i uses
 * set i % n_sets, so that with the sets together larger than the L2 cache
 * every timed run reads its inputs from HBM without a flush in between. One
 * event pair brackets `batch` consecutive runs (>= 1) and us_out[i] is that
 * duration divided by `batch`: with a batch of many runs the events' own cost
 * and the launch latency hidden behind the previous run drop out, which is how
 * a stream of launches behaves in production. `iters` counts batches. */
int emb_time_rotating(const emb_launch_t* launches, int chain_len, int n_sets, void* stream, int warmup, int iters,
                      int batch, float* us_out);

/* Build a tiled TMA descriptor (CUtensorMap, 128 bytes, 64-byte aligned
 * storage supplied by the caller) over a caller-owned tensor of `rank` (1..5)
 * dimensions. dims[0] is the innermost (contiguous) dimension;
 * strides_bytes[i] is the byte stride of dimension i+1 (rank-1 entries,
 * multiples of 16); box[i] is the tile extent per dimension. No counterpart
 * in the reference, whose runner protocol cannot pass a descriptor
 * (docs/DESIGN.md:860-863) and whose copy-engine path is therefore the
 * untiled cp.async.bulk (emmy_ptx/bulk.py:34-57); here the descriptor is an
 * extra kernel parameter listed in the module's launch header. */
int emb_tensor_map(void* map_out, const void* base, int dtype, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

/* The f32 array sum (block partials, then their fold) for callers that cannot
 * allocate device memory: a plugin inside another framework's memory pool, a
 * caller in a phase where cudaMalloc's implicit synchronisation is not allowed,
 * a host with a fixed device-memory budget. It has no counterpart in the
 * reference. The compiled chain k_sum__partial -> k_sum_1_reduce needs a
 * caller-owned scratch buffer `sum__partial` of one float per block; this entry
 * point keeps that scratch in a fixed array inside the library instead
 * (EMB_STATIC_SUM_MAX_BLOCKS floats = 8 KB, resident on every GPU that loads the
 * library until the process exits) and calls no allocator of any kind.
 *   x        n floats on the current device, 16-byte aligned; n a positive multiple of 4
 *   blocks   CTAs of the first kernel = number of partials; 1..EMB_STATIC_SUM_MAX_BLOCKS,
 *            anything larger is refused with EMB_E_ARGUMENT and a text
 *   sum_out  one float on the device
 * For equal `blocks` the result is bit for bit that of the chain compiled with
 * --strict (256 threads per block, 16-byte runs, the same butterfly and tree).
 * The first call on each device looks the array's device address up
 * (cudaGetSymbolAddress, with that device current): make that first call before
 * any stream capture begins. All calls on a device share the one array, which
 * keeps the last call's partials (nothing in it has to start at zero): two calls
 * whose kernels overlap on the GPU, e.g. on different streams, race on it.
 * Asynchronous on `stream`. */
#define EMB_STATIC_SUM_MAX_BLOCKS 2048
int emb_array_sum_f32_static(const float* x, uint64_t n, uint32_t blocks, float* sum_out, void* stream);

/* ---- the exchange record of a sharded sum ------------------------------------
 * No counterpart in the reference, whose problems run on one GPU. A module whose
 * launch header lists a parameter of kind "exchange" (the last kernel of a sum)
 * takes there a DEVICE pointer to this record, or NULL for no exchange. With a
 * record the kernel stores its f32 result, with the step number in the upper half
 * of one 8-byte word, into slot [step & 1][rank] of every rank's slot memory
 * (peer stores), waits at most wait_limit_us for every rank's word of the same
 * step in its own slot memory and returns the sum of all ranks' values in rank
 * order. slot[r] is rank r's slot memory as THIS rank addresses it: 2 x
 * EMB_MAX_PEERS 8-byte words, zeroed before the first launch and mapped into
 * every rank (CUDA IPC or fabric handles; torch's symmetric memory does it). All
 * ranks must run the same number of such launches. status != 0 after a launch:
 * rank status - 1 was waited for in vain, that result and all later ones are
 * invalid, and no later launch waits again. */
#define EMB_MAX_PEERS 8
typedef struct {
    uint64_t slot[EMB_MAX_PEERS]; /* device addresses, unused entries 0 */
    uint32_t rank, world;         /* this rank, number of ranks (1..EMB_MAX_PEERS) */
    uint32_t step;                /* steps completed; start at 0, the kernels count */
    uint32_t status;              /* start at 0 */
    uint32_t wait_limit_us;       /* e.g. 2000000 */
    uint32_t reserved;            /* 0 */
} emb_peer_exchange_t;

/* Text of the last error on the calling thread ("" if none). */
const char* emb_last_error(void);

/* ABI version of this header. */
int emb_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* EMMY_B200_H */
