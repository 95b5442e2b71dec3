/*
 * mtb200_rt.h — C ABI of the compile-and-launch runtime (libmtb200.so).
 *
 * This library is what the kernel compiler's Python side binds with ctypes in
 * place of CuPy.  Each entry point names the reference call it stands in for;
 * paths are relative to the reference project root.
 *
 * Conventions
 *   - every function returns int: 0 = ok; > 0 = a raw CUresult / nvrtcResult
 *     tagged by domain (see MTB_DOMAIN_*); < 0 = a runtime error (MTB_E_*).
 *   - no exceptions, no abort(), no exit(); mtb_last_error() gives a
 *     thread-local, human-readable description of the last failure.
 *   - the caller owns every device buffer it passes in; the library only frees
 *     what it allocated itself (mtb_mem_alloc, modules, streams, events).
 *   - libcuda and libnvrtc are dlopen'ed on first use, so loading this library
 *     and calling mtb_compile() works on a machine without a GPU driver.
 *   - handles are opaque pointers; the module table is mutex-protected and the
 *     device's primary context is made current inside each call that needs it.
 */
#ifndef MTB200_RT_H
#define MTB200_RT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* error domains: return value = domain + raw code */
#define MTB_DOMAIN_CUDA   100000   /* CUresult   */
#define MTB_DOMAIN_NVRTC  200000   /* nvrtcResult */

#define MTB_E_BAD_ARGUMENT     (-1)
#define MTB_E_NO_DRIVER        (-2)   /* libcuda.so.1 not loadable / cuInit failed */
#define MTB_E_NO_NVRTC         (-3)   /* libnvrtc not loadable */
#define MTB_E_BUFFER_TOO_SMALL (-4)
#define MTB_E_NOT_LOADED       (-5)   /* launch of a module that was never loaded on a device */
#define MTB_E_DEVICE_WAIT      (-6)   /* a kernel reported that one of its bounded waits ran out */
#define MTB_E_TOO_LARGE        (-7)   /* request exceeds a fixed capacity of the library */

typedef struct mtb_module mtb_module_t;   /* one compiled kernel (cubin + loaded function) */

typedef struct mtb_device_info {
    char     name[128];
    int      cc_major, cc_minor;
    int      sm_count;
    int      max_threads_per_block;
    int      max_smem_per_block_optin;   /* bytes */
    int      l2_bytes;
    int      sm_clock_khz, mem_clock_khz;
    uint64_t total_mem_bytes;
} mtb_device_info_t;

/* ---- library / device -------------------------------------------------------
 * Replaces the CuPy import-and-probe in src/mytriton/cuda_utils.py:23-48
 * (_cupy, _cuda_device_available, cuda_available, cuda_module). */
int         mtb_init(void);
int         mtb_device_count(int* count);
int         mtb_device_set(int device);            /* retain + bind the primary context */
int         mtb_device_get(int* device);
int         mtb_device_info(int device, mtb_device_info_t* out);
int         mtb_device_sync(void);
int         mtb_mem_info(uint64_t* free_bytes, uint64_t* total_bytes);
const char* mtb_last_error(void);
const char* mtb_version(void);

/* ---- compile ---------------------------------------------------------------
 * Replaces cp.RawKernel(src, name, options=("--std=c++14",)) in
 * src/mytriton/cuda_utils.py:105-111.  NVRTC -> cubin for `arch` (e.g.
 * "sm_100a"); needs no GPU.  The compile log (warnings or errors) is copied,
 * NUL-terminated and truncated if necessary, into log[0..log_cap). */
int mtb_compile(const char* src, const char* kernel_name, const char* arch,
                const char* const* options, int n_options,
                mtb_module_t** out_module, char* log, size_t log_cap);
int mtb_module_cubin(const mtb_module_t* module, const void** data, size_t* size);
/* Wraps an sm_100a cubin obtained earlier from mtb_module_cubin() (an on-disk kernel
 * cache; the reference keeps only in-memory dict caches, src/mytriton/compiler.py:74-79).
 * The bytes are copied. */
int mtb_module_from_cubin(const void* cubin, size_t size, const char* kernel_name,
                          mtb_module_t** out_module);
/* cuModuleLoadData + cuModuleGetFunction on the current device; raises the
 * function's dynamic shared-memory limit to dynamic_smem_bytes if non-zero. */
int mtb_module_load(mtb_module_t* module, int dynamic_smem_bytes);
int mtb_module_attr(const mtb_module_t* module, int* num_regs, int* static_smem_bytes,
                    int* local_bytes, int* max_threads);
int mtb_module_free(mtb_module_t* module);

/* ---- launch ----------------------------------------------------------------
 * Replaces kernel(launch_grid, (threads,), args) in
 * src/mytriton/cuda_utils.py:113-117: asynchronous on `stream` (NULL = the
 * legacy default stream), no synchronisation.  args[i] points at the i-th
 * kernel parameter's value (pointers, 32-bit scalars, 128-byte tensor maps).
 * cluster may be NULL or {1,1,1} for no cluster. */
int mtb_launch(mtb_module_t* module, const unsigned grid[3], const unsigned block[3],
               const unsigned cluster[3], unsigned dynamic_smem_bytes, void* stream,
               void** args);
/* The same launch with `device`'s primary context current for the duration of the
 * call (the caller's current context is restored afterwards).  A module is loaded
 * per device: MTB_E_NOT_LOADED means mtb_module_load has not run with that device
 * current.  For processes that drive several GPUs; the reference launches on CuPy's
 * current device only (src/mytriton/cuda_utils.py:113-117). */
int mtb_launch_on_device(mtb_module_t* module, int device, const unsigned grid[3],
                         const unsigned block[3], const unsigned cluster[3],
                         unsigned dynamic_smem_bytes, void* stream, void** args);

/* ---- TMA descriptors ---------------------------------------------------------
 * No counterpart in the reference (its kernels use plain global loads,
 * src/mytriton/cuda_codegen.py:349-365); needed by the tl.dot lowering.
 * Encodes a 2-D row-major tensor [dim_outer][dim_inner] of `elem_bytes`-wide
 * elements into a 128-byte CUtensorMap at out128 (64-byte aligned host memory).
 * swizzle: 0 none, 1 32B, 2 64B, 3 128B, 4 128B in 32-byte chunks (CUtensorMapSwizzle's
 * numbering).  Out-of-range box parts read as zero. */
int mtb_tensormap_encode_2d(void* out128, int elem_bytes, int is_float, int is_bf16,
                            uint64_t base, uint64_t dim_inner, uint64_t dim_outer,
                            uint64_t stride_outer_bytes, uint32_t box_inner,
                            uint32_t box_outer, int swizzle, int l2_promotion);

/* ---- streams / events / memory ------------------------------------------------
 * The reference leaves these to CuPy (cp.cuda.Stream.null.synchronize(),
 * cp.empty, cp.asarray in its tests, e.g. tests/test_add_kernel.py:238-254). */
int mtb_stream_create(void** stream);
int mtb_stream_destroy(void* stream);
int mtb_stream_sync(void* stream);
int mtb_event_create(void** event);
int mtb_event_destroy(void* event);
int mtb_event_record(void* event, void* stream);
int mtb_event_sync(void* event);
int mtb_event_elapsed_ms(void* start, void* stop, float* ms);
int mtb_mem_alloc(uint64_t* device_ptr, size_t bytes);
int mtb_mem_free(uint64_t device_ptr);
int mtb_memcpy_h2d(uint64_t dst, const void* src, size_t bytes, void* stream);
int mtb_memcpy_d2h(void* dst, uint64_t src, size_t bytes, void* stream);
int mtb_memcpy_d2d(uint64_t dst, uint64_t src, size_t bytes, void* stream);
int mtb_memset_u32(uint64_t dst, uint32_t value, size_t count, void* stream);
int mtb_host_alloc_pinned(void** host_ptr, size_t bytes);
int mtb_host_free_pinned(void* host_ptr);

/* ---- device status word --------------------------------------------------------
 * Kernels with bounded waits (mbarrier / TMEM allocation) write a non-zero code
 * into a caller-provided 32-bit status word instead of trapping or spinning for
 * ever.  Reads it back (synchronising `stream`) and maps non-zero to
 * MTB_E_DEVICE_WAIT with the code in *status. */
int mtb_status_check(uint64_t status_ptr, void* stream, uint32_t* status);

/* ---- split-row sum --------------------------------------------------------------
 * A row sum whose rows are split over several CTAs, for matrices with too few (or
 * too long) rows to fill the GPU with one program per row.  The reference computes
 * row sums with one block per row and names the missing piece itself ("no
 * multi-block reduction yet", README.md:380-384; kernel in
 * tests/test_long_row_sum_kernel.py:28-47).  x is [rows][cols] fp32 row-major,
 * out is [rows] fp32; `scratch` is caller-allocated device memory of at least
 * mtb_long_row_sum_scratch_bytes() bytes, 16-byte aligned.  Asynchronous on
 * `stream`.  Deterministic: the same input gives the same bits on every call. */
int mtb_long_row_sum_scratch_bytes(int rows, long long cols, size_t* bytes);
int mtb_long_row_sum(uint64_t x, uint64_t out, int rows, long long cols, uint64_t scratch,
                     size_t scratch_bytes, void* stream);

/* The same sum with no buffer to bring: the partial sums and counters live in a
 * fixed 80 KiB block inside the library image, and the call itself makes no
 * cudaMalloc, cudaFree or other allocating call.  (One thing outside its control:
 * the CUDA runtime loads a library's device code lazily, so the very first use of
 * this library's kernels on a device — this call included — makes the driver place
 * the library's image, the 80 KiB block with it, in device memory.  That happens
 * once per device; it is the reason for "first call during set-up" below.)
 * It has no counterpart in the reference.
 * Meant for callers that must not allocate once they are running: a service that
 * gave all device memory to its own pool at start-up (a later cudaMalloc would
 * fail or fragment it), a latency-sensitive loop that cannot afford the implicit
 * synchronisation of an allocation, or a host language binding where owning one
 * more device buffer across calls is a burden.
 * Limits: rows <= 4096 and rows * splits <= 16384 (splits is what
 * mtb_long_row_sum would choose: about 4 CTAs per SM in total, at most 64 per
 * row); beyond that it returns MTB_E_TOO_LARGE and says so in mtb_last_error().
 * The first call on each device looks up the block's device address (and may
 * trigger the one-time image load described above); make that first call during
 * set-up, before any stream capture begins and before memory is handed to a pool.
 * All calls on a device share the one block: two calls whose kernels may overlap
 * on the GPU (different streams, or different threads) race on it — serialise
 * them, or give one of them mtb_long_row_sum with its own scratch.  The block
 * keeps whatever the last call left; the counters are cleared at the start of
 * every call, the partial sums are always written before they are read. */
int mtb_long_row_sum_static(uint64_t x, uint64_t out, int rows, long long cols, void* stream);

/* Sets the calling thread's mtb_last_error() text (used by the library's own files). */
void mtb_set_last_error(const char* text);

#ifdef __cplusplus
}
#endif
#endif /* MTB200_RT_H */
