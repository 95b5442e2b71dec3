// libmtb200.so — compile-and-launch runtime behind include/mtb200_rt.h.
//
// A thin layer over NVRTC and the CUDA driver API.  Both libraries are opened
// with dlopen on first use, so this file links against neither and the library
// loads (and compiles kernels to cubins) on hosts without a GPU driver.
// Built with nvcc for sm_100a; see mytriton_b200/build.py.

#include "mtb200_rt.h"

#include <cuda.h>
#include <nvrtc.h>
#include <dlfcn.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#define MTB_XSTR(x) MTB_STR(x)
#define MTB_STR(x) #x

namespace {

thread_local char g_error[1024] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

// ---- dynamically resolved entry points -------------------------------------------
#define MTB_DRIVER_FUNCS(X)                                                         \
    X(cuInit) X(cuDeviceGetCount) X(cuDeviceGet) X(cuDeviceGetName)                 \
    X(cuDeviceGetAttribute) X(cuDeviceTotalMem) X(cuDevicePrimaryCtxRetain)         \
    X(cuCtxSetCurrent) X(cuCtxGetCurrent) X(cuCtxGetDevice) X(cuCtxSynchronize)     \
    X(cuCtxPushCurrent) X(cuCtxPopCurrent)                                          \
    X(cuMemGetInfo) X(cuModuleLoadData) X(cuModuleUnload) X(cuModuleGetFunction)    \
    X(cuFuncSetAttribute) X(cuFuncGetAttribute) X(cuLaunchKernelEx)                 \
    X(cuTensorMapEncodeTiled) X(cuStreamCreate) X(cuStreamDestroy)                  \
    X(cuStreamSynchronize) X(cuEventCreate) X(cuEventDestroy) X(cuEventRecord)      \
    X(cuEventSynchronize) X(cuEventElapsedTime) X(cuMemAlloc) X(cuMemFree)          \
    X(cuMemcpyHtoDAsync) X(cuMemcpyDtoHAsync) X(cuMemcpyDtoDAsync)                  \
    X(cuMemsetD32Async) X(cuMemAllocHost) X(cuMemFreeHost) X(cuGetErrorString)      \
    X(cuGetErrorName)

#define MTB_NVRTC_FUNCS(X)                                                          \
    X(nvrtcCreateProgram) X(nvrtcDestroyProgram) X(nvrtcCompileProgram)             \
    X(nvrtcGetProgramLogSize) X(nvrtcGetProgramLog) X(nvrtcGetCUBINSize)            \
    X(nvrtcGetCUBIN) X(nvrtcGetErrorString)

#define MTB_DECLARE(name) decltype(&name) p_##name = nullptr;
MTB_DRIVER_FUNCS(MTB_DECLARE)
MTB_NVRTC_FUNCS(MTB_DECLARE)
#undef MTB_DECLARE

std::mutex g_mutex;            // guards library loading, device table, module load/free
void* g_libcuda = nullptr;
void* g_libnvrtc = nullptr;
bool g_driver_ready = false;
constexpr int kMaxDevices = 64;
CUcontext g_primary[kMaxDevices] = {};

int load_nvrtc_locked() {
    if (g_libnvrtc) return 0;
    const char* names[] = {"libnvrtc.so.12", "libnvrtc.so",
                           "/usr/local/cuda/lib64/libnvrtc.so.12"};
    for (const char* n : names) {
        g_libnvrtc = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_libnvrtc) break;
    }
    if (!g_libnvrtc) return fail(MTB_E_NO_NVRTC, "cannot load libnvrtc: %s", dlerror());
#define MTB_LOAD(name)                                                              \
    p_##name = reinterpret_cast<decltype(&name)>(dlsym(g_libnvrtc, MTB_XSTR(name))); \
    if (!p_##name) return fail(MTB_E_NO_NVRTC, "libnvrtc lacks %s", MTB_XSTR(name));
    MTB_NVRTC_FUNCS(MTB_LOAD)
#undef MTB_LOAD
    return 0;
}

int load_driver_locked() {
    if (g_driver_ready) return 0;
    if (!g_libcuda) {
        g_libcuda = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (!g_libcuda) return fail(MTB_E_NO_DRIVER, "cannot load libcuda.so.1: %s", dlerror());
#define MTB_LOAD(name)                                                              \
    p_##name = reinterpret_cast<decltype(&name)>(dlsym(g_libcuda, MTB_XSTR(name)));  \
    if (!p_##name) return fail(MTB_E_NO_DRIVER, "libcuda lacks %s", MTB_XSTR(name));
        MTB_DRIVER_FUNCS(MTB_LOAD)
#undef MTB_LOAD
    }
    CUresult r = p_cuInit(0);
    if (r != CUDA_SUCCESS) return fail(MTB_E_NO_DRIVER, "cuInit failed with CUresult %d", (int)r);
    g_driver_ready = true;
    return 0;
}

int cu_fail(CUresult r, const char* what) {
    const char* name = nullptr;
    const char* text = nullptr;
    if (p_cuGetErrorName) p_cuGetErrorName(r, &name);
    if (p_cuGetErrorString) p_cuGetErrorString(r, &text);
    return fail(MTB_DOMAIN_CUDA + (int)r, "%s: %s (%s)", what, name ? name : "CUDA error",
                text ? text : "?");
}

#define CU_TRY(call)                                       \
    do {                                                   \
        CUresult _r = (call);                              \
        if (_r != CUDA_SUCCESS) return cu_fail(_r, #call); \
    } while (0)

int ensure_driver() {
    std::lock_guard<std::mutex> lock(g_mutex);
    return load_driver_locked();
}

// Make sure the calling thread has a current context; bind device 0 if none.
int ensure_context() {
    if (int rc = ensure_driver()) return rc;
    CUcontext ctx = nullptr;
    CU_TRY(p_cuCtxGetCurrent(&ctx));
    if (ctx) return 0;
    return mtb_device_set(0);
}

}  // namespace

// A compiled kernel.  The cubin is device-independent; what the driver makes of it (module,
// function handle, the dynamic shared-memory limit set on the function) belongs to one
// context, so there is one slot per device, indexed by the CUDA device ordinal of the context
// that is current when mtb_module_load / mtb_launch is called.
struct mtb_loaded_image {
    CUmodule module = nullptr;
    CUfunction function = nullptr;
    int dynamic_smem = 0;
};

struct mtb_module {
    std::string name;
    std::vector<char> cubin;
    mtb_loaded_image on[kMaxDevices];
};

namespace {

// The slot of the calling thread's current device, or NULL when no context is current.
mtb_loaded_image* current_image(mtb_module* module) {
    CUdevice dev = 0;
    if (!p_cuCtxGetDevice || p_cuCtxGetDevice(&dev) != CUDA_SUCCESS) return nullptr;
    if ((int)dev < 0 || (int)dev >= kMaxDevices) return nullptr;
    return &module->on[(int)dev];
}

}  // namespace

extern "C" {

const char* mtb_last_error(void) { return g_error; }
void mtb_set_last_error(const char* text) { snprintf(g_error, sizeof g_error, "%s", text ? text : ""); }
const char* mtb_version(void) { return "mtb200 0.1 (sm_100a)"; }

int mtb_init(void) { return ensure_driver(); }

int mtb_device_count(int* count) {
    if (!count) return fail(MTB_E_BAD_ARGUMENT, "count is NULL");
    if (int rc = ensure_driver()) return rc;
    CU_TRY(p_cuDeviceGetCount(count));
    return 0;
}

int mtb_device_set(int device) {
    if (device < 0 || device >= kMaxDevices) return fail(MTB_E_BAD_ARGUMENT, "bad device %d", device);
    if (int rc = ensure_driver()) return rc;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_primary[device]) {
        CUdevice dev;
        CU_TRY(p_cuDeviceGet(&dev, device));
        CU_TRY(p_cuDevicePrimaryCtxRetain(&g_primary[device], dev));
    }
    CU_TRY(p_cuCtxSetCurrent(g_primary[device]));
    return 0;
}

int mtb_device_get(int* device) {
    if (!device) return fail(MTB_E_BAD_ARGUMENT, "device is NULL");
    if (int rc = ensure_context()) return rc;
    CUdevice dev;
    CU_TRY(p_cuCtxGetDevice(&dev));
    *device = (int)dev;
    return 0;
}

int mtb_device_info(int device, mtb_device_info_t* out) {
    if (!out) return fail(MTB_E_BAD_ARGUMENT, "out is NULL");
    if (int rc = ensure_driver()) return rc;
    CUdevice dev;
    CU_TRY(p_cuDeviceGet(&dev, device));
    memset(out, 0, sizeof *out);
    CU_TRY(p_cuDeviceGetName(out->name, (int)sizeof out->name, dev));
    struct { int* dst; CUdevice_attribute attr; } wanted[] = {
        {&out->cc_major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR},
        {&out->cc_minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR},
        {&out->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT},
        {&out->max_threads_per_block, CU_DEVICE_ATTRIBUTE_MAX_THREADS_PER_BLOCK},
        {&out->max_smem_per_block_optin, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN},
        {&out->l2_bytes, CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE},
        {&out->sm_clock_khz, CU_DEVICE_ATTRIBUTE_CLOCK_RATE},
        {&out->mem_clock_khz, CU_DEVICE_ATTRIBUTE_MEMORY_CLOCK_RATE},
    };
    for (auto& w : wanted) CU_TRY(p_cuDeviceGetAttribute(w.dst, w.attr, dev));
    size_t total = 0;
    CU_TRY(p_cuDeviceTotalMem(&total, dev));
    out->total_mem_bytes = total;
    return 0;
}

int mtb_device_sync(void) {
    if (int rc = ensure_context()) return rc;
    CU_TRY(p_cuCtxSynchronize());
    return 0;
}

int mtb_mem_info(uint64_t* free_bytes, uint64_t* total_bytes) {
    if (int rc = ensure_context()) return rc;
    size_t f = 0, t = 0;
    CU_TRY(p_cuMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return 0;
}

// ---- compile ------------------------------------------------------------------------

int mtb_compile(const char* src, const char* kernel_name, const char* arch,
                const char* const* options, int n_options, mtb_module_t** out_module,
                char* log, size_t log_cap) {
    if (log && log_cap) log[0] = '\0';
    if (!src || !kernel_name || !out_module || n_options < 0)
        return fail(MTB_E_BAD_ARGUMENT, "mtb_compile: NULL source, name or output");
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (int rc = load_nvrtc_locked()) return rc;
    }
    nvrtcProgram prog = nullptr;
    nvrtcResult r = p_nvrtcCreateProgram(&prog, src, kernel_name, 0, nullptr, nullptr);
    if (r != NVRTC_SUCCESS)
        return fail(MTB_DOMAIN_NVRTC + (int)r, "nvrtcCreateProgram: %s", p_nvrtcGetErrorString(r));

    std::string arch_flag = std::string("--gpu-architecture=") + (arch ? arch : "sm_100a");
    std::vector<const char*> argv;
    argv.push_back(arch_flag.c_str());
    for (int i = 0; i < n_options; ++i) argv.push_back(options[i]);

    nvrtcResult compiled = p_nvrtcCompileProgram(prog, (int)argv.size(), argv.data());
    size_t log_size = 0;
    if (p_nvrtcGetProgramLogSize(prog, &log_size) == NVRTC_SUCCESS && log_size > 1) {
        std::vector<char> full(log_size);
        p_nvrtcGetProgramLog(prog, full.data());
        if (log && log_cap) {
            size_t n = log_size - 1 < log_cap - 1 ? log_size - 1 : log_cap - 1;
            memcpy(log, full.data(), n);
            log[n] = '\0';
        }
        if (compiled != NVRTC_SUCCESS) {
            fail(MTB_DOMAIN_NVRTC + (int)compiled, "NVRTC compile of %s failed: %.800s",
                 kernel_name, full.data());
        }
    } else if (compiled != NVRTC_SUCCESS) {
        fail(MTB_DOMAIN_NVRTC + (int)compiled, "NVRTC compile of %s failed: %s", kernel_name,
             p_nvrtcGetErrorString(compiled));
    }
    if (compiled != NVRTC_SUCCESS) {
        p_nvrtcDestroyProgram(&prog);
        return MTB_DOMAIN_NVRTC + (int)compiled;
    }
    size_t size = 0;
    r = p_nvrtcGetCUBINSize(prog, &size);
    if (r != NVRTC_SUCCESS || size == 0) {
        p_nvrtcDestroyProgram(&prog);
        return fail(MTB_DOMAIN_NVRTC + (int)r, "nvrtcGetCUBINSize: no cubin produced for %s",
                    arch_flag.c_str());
    }
    mtb_module* m = new mtb_module;
    m->name = kernel_name;
    m->cubin.resize(size);
    r = p_nvrtcGetCUBIN(prog, m->cubin.data());
    p_nvrtcDestroyProgram(&prog);
    if (r != NVRTC_SUCCESS) {
        delete m;
        return fail(MTB_DOMAIN_NVRTC + (int)r, "nvrtcGetCUBIN: %s", p_nvrtcGetErrorString(r));
    }
    *out_module = m;
    return 0;
}

int mtb_module_cubin(const mtb_module_t* module, const void** data, size_t* size) {
    if (!module || !data || !size) return fail(MTB_E_BAD_ARGUMENT, "mtb_module_cubin: NULL argument");
    *data = module->cubin.data();
    *size = module->cubin.size();
    return 0;
}

int mtb_module_from_cubin(const void* cubin, size_t size, const char* kernel_name,
                          mtb_module_t** out_module) {
    if (!cubin || size == 0 || !kernel_name || !out_module)
        return fail(MTB_E_BAD_ARGUMENT, "mtb_module_from_cubin: NULL or empty argument");
    mtb_module* m = new mtb_module;
    m->name = kernel_name;
    m->cubin.assign(static_cast<const char*>(cubin), static_cast<const char*>(cubin) + size);
    *out_module = m;
    return 0;
}

int mtb_module_load(mtb_module_t* module, int dynamic_smem_bytes) {
    if (!module || dynamic_smem_bytes < 0) return fail(MTB_E_BAD_ARGUMENT, "mtb_module_load: bad argument");
    if (int rc = ensure_context()) return rc;
    std::lock_guard<std::mutex> lock(g_mutex);
    mtb_loaded_image* image = current_image(module);
    if (!image) return fail(MTB_E_BAD_ARGUMENT, "mtb_module_load: no usable current device");
    if (!image->function) {
        CU_TRY(p_cuModuleLoadData(&image->module, module->cubin.data()));
        CUresult r = p_cuModuleGetFunction(&image->function, image->module, module->name.c_str());
        if (r != CUDA_SUCCESS) {
            p_cuModuleUnload(image->module);
            image->module = nullptr;
            image->function = nullptr;
            return cu_fail(r, "cuModuleGetFunction");
        }
    }
    if (dynamic_smem_bytes > image->dynamic_smem) {
        CU_TRY(p_cuFuncSetAttribute(image->function,
                                    CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                    dynamic_smem_bytes));
        image->dynamic_smem = dynamic_smem_bytes;
    }
    return 0;
}

int mtb_module_attr(const mtb_module_t* module, int* num_regs, int* static_smem_bytes,
                    int* local_bytes, int* max_threads) {
    if (!module) return fail(MTB_E_BAD_ARGUMENT, "module is NULL");
    const mtb_loaded_image* image = current_image(const_cast<mtb_module_t*>(module));
    if (!image || !image->function)
        return fail(MTB_E_NOT_LOADED, "module %s is not loaded on the current device", module->name.c_str());
    if (num_regs) CU_TRY(p_cuFuncGetAttribute(num_regs, CU_FUNC_ATTRIBUTE_NUM_REGS, image->function));
    if (static_smem_bytes)
        CU_TRY(p_cuFuncGetAttribute(static_smem_bytes, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, image->function));
    if (local_bytes)
        CU_TRY(p_cuFuncGetAttribute(local_bytes, CU_FUNC_ATTRIBUTE_LOCAL_SIZE_BYTES, image->function));
    if (max_threads)
        CU_TRY(p_cuFuncGetAttribute(max_threads, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, image->function));
    return 0;
}

int mtb_module_free(mtb_module_t* module) {
    if (!module) return 0;
    std::lock_guard<std::mutex> lock(g_mutex);
    for (int dev = 0; dev < kMaxDevices; ++dev) {
        if (!module->on[dev].module || !p_cuModuleUnload) continue;
        // a module is unloaded in the context it was loaded into
        const bool pushed = g_primary[dev] && p_cuCtxPushCurrent(g_primary[dev]) == CUDA_SUCCESS;
        p_cuModuleUnload(module->on[dev].module);
        if (pushed) { CUcontext ignored; p_cuCtxPopCurrent(&ignored); }
    }
    delete module;
    return 0;
}

// ---- launch -------------------------------------------------------------------------

int mtb_launch(mtb_module_t* module, const unsigned grid[3], const unsigned block[3],
               const unsigned cluster[3], unsigned dynamic_smem_bytes, void* stream, void** args) {
    if (!module || !grid || !block) return fail(MTB_E_BAD_ARGUMENT, "mtb_launch: NULL argument");
    const mtb_loaded_image* image = current_image(module);
    if (!image || !image->function)
        return fail(MTB_E_NOT_LOADED, "module %s is not loaded on the current device", module->name.c_str());
    if ((int)dynamic_smem_bytes > image->dynamic_smem && dynamic_smem_bytes > 48 * 1024)
        return fail(MTB_E_BAD_ARGUMENT, "launch asks for %u B dynamic smem but module was loaded for %d",
                    dynamic_smem_bytes, image->dynamic_smem);
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDimX = grid[0]; cfg.gridDimY = grid[1]; cfg.gridDimZ = grid[2];
    cfg.blockDimX = block[0]; cfg.blockDimY = block[1]; cfg.blockDimZ = block[2];
    cfg.sharedMemBytes = dynamic_smem_bytes;
    cfg.hStream = (CUstream)stream;
    CUlaunchAttribute attr[1];
    if (cluster && (cluster[0] > 1 || cluster[1] > 1 || cluster[2] > 1)) {
        attr[0].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attr[0].value.clusterDim.x = cluster[0];
        attr[0].value.clusterDim.y = cluster[1];
        attr[0].value.clusterDim.z = cluster[2];
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    CU_TRY(p_cuLaunchKernelEx(&cfg, image->function, args, nullptr));
    return 0;
}

int mtb_launch_on_device(mtb_module_t* module, int device, const unsigned grid[3], const unsigned block[3],
                         const unsigned cluster[3], unsigned dynamic_smem_bytes, void* stream, void** args) {
    if (device < 0 || device >= kMaxDevices) return fail(MTB_E_BAD_ARGUMENT, "bad device %d", device);
    CUdevice current = -1;
    if (p_cuCtxGetDevice && p_cuCtxGetDevice(&current) == CUDA_SUCCESS && (int)current == device)
        return mtb_launch(module, grid, block, cluster, dynamic_smem_bytes, stream, args);
    // another device (or none) is current: make this one current for the launch only
    if (int rc = ensure_driver()) return rc;
    CUcontext target = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_primary[device]) {
            CUdevice dev;
            CU_TRY(p_cuDeviceGet(&dev, device));
            CU_TRY(p_cuDevicePrimaryCtxRetain(&g_primary[device], dev));
        }
        target = g_primary[device];
    }
    CU_TRY(p_cuCtxPushCurrent(target));
    const int rc = mtb_launch(module, grid, block, cluster, dynamic_smem_bytes, stream, args);
    CUcontext ignored;
    p_cuCtxPopCurrent(&ignored);
    return rc;
}

// ---- tensor maps ----------------------------------------------------------------------

int mtb_tensormap_encode_2d(void* out128, int elem_bytes, int is_float, int is_bf16, uint64_t base,
                            uint64_t dim_inner, uint64_t dim_outer, uint64_t stride_outer_bytes,
                            uint32_t box_inner, uint32_t box_outer, int swizzle, int l2_promotion) {
    if (!out128) return fail(MTB_E_BAD_ARGUMENT, "out128 is NULL");
    if (int rc = ensure_driver()) return rc;
    CUtensorMapDataType dt;
    if (is_bf16 && elem_bytes == 2) dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    else if (is_float && elem_bytes == 4) dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    else if (is_float && elem_bytes == 2) dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    else if (elem_bytes == 4) dt = CU_TENSOR_MAP_DATA_TYPE_INT32;
    else if (elem_bytes == 1) dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
    else return fail(MTB_E_BAD_ARGUMENT, "unsupported element: %d bytes", elem_bytes);
    if (swizzle < 0 || swizzle > 6 || l2_promotion < 0 || l2_promotion > 3)
        return fail(MTB_E_BAD_ARGUMENT, "bad swizzle/l2 promotion");
    if (base % 16 || stride_outer_bytes % 16)
        return fail(MTB_E_BAD_ARGUMENT, "tensor map base and row stride must be 16-byte aligned");
    if (((uint64_t)box_inner * elem_bytes) % 16)
        return fail(MTB_E_BAD_ARGUMENT, "tensor map inner box extent must be a multiple of 16 bytes");
    cuuint64_t dims[2] = {dim_inner, dim_outer};
    cuuint64_t strides[1] = {stride_outer_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CU_TRY(p_cuTensorMapEncodeTiled(
        reinterpret_cast<CUtensorMap*>(out128), dt, 2, reinterpret_cast<void*>(base), dims, strides,
        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, (CUtensorMapSwizzle)swizzle,
        (CUtensorMapL2promotion)l2_promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return 0;
}

// ---- streams / events / memory ----------------------------------------------------------

int mtb_stream_create(void** stream) {
    if (!stream) return fail(MTB_E_BAD_ARGUMENT, "stream is NULL");
    if (int rc = ensure_context()) return rc;
    CUstream s;
    CU_TRY(p_cuStreamCreate(&s, CU_STREAM_NON_BLOCKING));
    *stream = s;
    return 0;
}
int mtb_stream_destroy(void* stream) {
    if (!stream) return 0;
    CU_TRY(p_cuStreamDestroy((CUstream)stream));
    return 0;
}
int mtb_stream_sync(void* stream) {
    if (int rc = ensure_context()) return rc;
    CU_TRY(p_cuStreamSynchronize((CUstream)stream));
    return 0;
}
int mtb_event_create(void** event) {
    if (!event) return fail(MTB_E_BAD_ARGUMENT, "event is NULL");
    if (int rc = ensure_context()) return rc;
    CUevent e;
    CU_TRY(p_cuEventCreate(&e, CU_EVENT_DEFAULT));
    *event = e;
    return 0;
}
int mtb_event_destroy(void* event) {
    if (!event) return 0;
    CU_TRY(p_cuEventDestroy((CUevent)event));
    return 0;
}
int mtb_event_record(void* event, void* stream) {
    CU_TRY(p_cuEventRecord((CUevent)event, (CUstream)stream));
    return 0;
}
int mtb_event_sync(void* event) {
    CU_TRY(p_cuEventSynchronize((CUevent)event));
    return 0;
}
int mtb_event_elapsed_ms(void* start, void* stop, float* ms) {
    if (!ms) return fail(MTB_E_BAD_ARGUMENT, "ms is NULL");
    CU_TRY(p_cuEventElapsedTime(ms, (CUevent)start, (CUevent)stop));
    return 0;
}
int mtb_mem_alloc(uint64_t* device_ptr, size_t bytes) {
    if (!device_ptr || bytes == 0) return fail(MTB_E_BAD_ARGUMENT, "mtb_mem_alloc: bad argument");
    if (int rc = ensure_context()) return rc;
    CUdeviceptr p = 0;
    CU_TRY(p_cuMemAlloc(&p, bytes));
    *device_ptr = (uint64_t)p;
    return 0;
}
int mtb_mem_free(uint64_t device_ptr) {
    if (!device_ptr) return 0;
    CU_TRY(p_cuMemFree((CUdeviceptr)device_ptr));
    return 0;
}
int mtb_memcpy_h2d(uint64_t dst, const void* src, size_t bytes, void* stream) {
    if (int rc = ensure_context()) return rc;
    CU_TRY(p_cuMemcpyHtoDAsync((CUdeviceptr)dst, src, bytes, (CUstream)stream));
    return 0;
}
int mtb_memcpy_d2h(void* dst, uint64_t src, size_t bytes, void* stream) {
    if (int rc = ensure_context()) return rc;
    CU_TRY(p_cuMemcpyDtoHAsync(dst, (CUdeviceptr)src, bytes, (CUstream)stream));
    return 0;
}
int mtb_memcpy_d2d(uint64_t dst, uint64_t src, size_t bytes, void* stream) {
    if (int rc = ensure_context()) return rc;
    CU_TRY(p_cuMemcpyDtoDAsync((CUdeviceptr)dst, (CUdeviceptr)src, bytes, (CUstream)stream));
    return 0;
}
int mtb_memset_u32(uint64_t dst, uint32_t value, size_t count, void* stream) {
    if (int rc = ensure_context()) return rc;
    CU_TRY(p_cuMemsetD32Async((CUdeviceptr)dst, value, count, (CUstream)stream));
    return 0;
}
int mtb_host_alloc_pinned(void** host_ptr, size_t bytes) {
    if (!host_ptr || bytes == 0) return fail(MTB_E_BAD_ARGUMENT, "mtb_host_alloc_pinned: bad argument");
    if (int rc = ensure_context()) return rc;
    CU_TRY(p_cuMemAllocHost(host_ptr, bytes));
    return 0;
}
int mtb_host_free_pinned(void* host_ptr) {
    if (!host_ptr) return 0;
    CU_TRY(p_cuMemFreeHost(host_ptr));
    return 0;
}

int mtb_status_check(uint64_t status_ptr, void* stream, uint32_t* status) {
    if (!status_ptr || !status) return fail(MTB_E_BAD_ARGUMENT, "mtb_status_check: NULL argument");
    if (int rc = ensure_context()) return rc;
    uint32_t word = 0;
    CU_TRY(p_cuMemcpyDtoHAsync(&word, (CUdeviceptr)status_ptr, sizeof word, (CUstream)stream));
    CU_TRY(p_cuStreamSynchronize((CUstream)stream));
    *status = word;
    if (word != 0)
        return fail(MTB_E_DEVICE_WAIT, "kernel reported status 0x%08x (a bounded device wait ran out)", word);
    return 0;
}

}  // extern "C"
