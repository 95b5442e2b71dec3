// Split-row sum: rows that are too few (or too long) for "one program per row".
//
// The kernel language runs one program per row, so a row sum over R rows keeps at
// most R SMs busy; the reference states the same limit ("no multi-block reduction
// yet", README.md:380-384).  This kernel splits every row over several CTAs:
//   stage 1  CTA (s, r) sums columns [s*chunk, (s+1)*chunk) of row r (128-bit
//            loads, four in flight per thread, fixed-order CTA combine) and writes
//            one partial to scratch;
//   stage 2  the CTA that finishes a row last (a ticket counter in scratch) adds
//            that row's partials in index order and writes out[r].
// The result does not depend on which CTA finishes last: partials are combined in
// a fixed order, so repeated calls are bit-identical.
//
// Scratch layout: `rows * splits` floats of partials followed by `rows` 32-bit
// ticket counters.  Counters must be zero when the kernel starts; the kernel
// leaves them at zero again.

#include "mtb200_rt.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float cta_sum(float value, float* slots) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) value += __shfl_xor_sync(0xffffffffu, value, o);
    if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = value;
    __syncthreads();
    float total = slots[0];
    #pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) total += slots[w];
    return total;
}

__global__ __launch_bounds__(kThreads)
void split_row_sum_kernel(const float* __restrict__ x, float* __restrict__ out, int rows,
                          long long cols, int splits, long long chunk,
                          float* partials, unsigned* tickets) {
    __shared__ float slots[kThreads / 32];
    __shared__ bool last;
    const int split = blockIdx.x, row = blockIdx.y;
    const long long begin = (long long)split * chunk;
    const long long end = begin + chunk < cols ? begin + chunk : cols;
    const float* base = x + (long long)row * cols;

    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    const bool vector_ok = ((reinterpret_cast<unsigned long long>(base + begin) & 15ull) == 0ull);
    long long i = begin + (long long)threadIdx.x * 4;
    if (vector_ok) {
        const long long stride = (long long)kThreads * 4;
        for (; i + 3 * stride + 3 < end; i += 4 * stride) {      // four 128-bit loads in flight
            const float4 a = __ldcs(reinterpret_cast<const float4*>(base + i));
            const float4 b = __ldcs(reinterpret_cast<const float4*>(base + i + stride));
            const float4 c = __ldcs(reinterpret_cast<const float4*>(base + i + 2 * stride));
            const float4 d = __ldcs(reinterpret_cast<const float4*>(base + i + 3 * stride));
            acc0 += (a.x + a.y) + (a.z + a.w);
            acc1 += (b.x + b.y) + (b.z + b.w);
            acc2 += (c.x + c.y) + (c.z + c.w);
            acc3 += (d.x + d.y) + (d.z + d.w);
        }
        for (; i + 3 < end; i += stride) {
            const float4 a = __ldcs(reinterpret_cast<const float4*>(base + i));
            acc0 += (a.x + a.y) + (a.z + a.w);
        }
        for (long long j = i; j < end && j < i + 4; ++j) acc1 += base[j];   // ragged tail of this thread
    } else {
        for (long long j = begin + threadIdx.x; j < end; j += kThreads) acc0 += base[j];
    }
    const float partial = cta_sum((acc0 + acc1) + (acc2 + acc3), slots);

    if (threadIdx.x == 0) {
        partials[(long long)row * splits + split] = partial;
        __threadfence();
        const unsigned ticket = atomicAdd(&tickets[row], 1u);
        last = (ticket == (unsigned)splits - 1u);
    }
    __syncthreads();
    if (last && threadIdx.x < 32) {
        __threadfence();
        float total = 0.f;
        const volatile float* mine = partials + (long long)row * splits;
        for (int s = threadIdx.x; s < splits; s += 32) total += mine[s];      // fixed order per lane
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (threadIdx.x == 0) {
            out[row] = total;
            tickets[row] = 0u;                                   // ready for the next call
        }
    }
}

int fail_with(int code, const char* text) {
    mtb_set_last_error(text);
    return code;
}

int plan_splits(int rows, long long cols, int* splits, long long* chunk) {
    if (rows <= 0 || cols <= 0) return fail_with(MTB_E_BAD_ARGUMENT, "mtb_long_row_sum: rows and cols must be positive");
    if (rows > 65535) return fail_with(MTB_E_TOO_LARGE, "mtb_long_row_sum: at most 65535 rows per call");
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    long long want = (4LL * sms + rows - 1) / rows;              // ~4 CTAs per SM in total
    const long long most = (cols + 4095) / 4096;                 // at least 4096 columns per CTA
    if (want > most) want = most;
    if (want > 64) want = 64;
    if (want < 1) want = 1;
    long long per = (cols + want - 1) / want;
    per = (per + 1023) / 1024 * 1024;                            // keeps 16-byte alignment of chunks
    *splits = (int)((cols + per - 1) / per);
    *chunk = per;
    return 0;
}

int launch_split_row_sum(const float* x, float* out, int rows, long long cols, int splits,
                         long long chunk, float* partials, unsigned* tickets, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(tickets, 0, sizeof(unsigned) * (size_t)rows, stream);
    if (e != cudaSuccess) return fail_with(MTB_DOMAIN_CUDA + (int)e, cudaGetErrorString(e));
    split_row_sum_kernel<<<dim3((unsigned)splits, (unsigned)rows), kThreads, 0, stream>>>(
        x, out, rows, cols, splits, chunk, partials, tickets);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail_with(MTB_DOMAIN_CUDA + (int)e, cudaGetErrorString(e));
    return 0;
}

}  // namespace

// ---- built-in scratch for mtb_long_row_sum_static ------------------------------------
// One fixed block of device memory that lives in the library image: every GPU that
// loads libmtb200.so carries these 80 KiB until the process exits.  Layout is the same
// as the caller-provided scratch: partial sums first, then the per-row ticket counters.
constexpr size_t kStaticPartialSlots = 16384;                 // floats: rows * splits may not exceed this
constexpr size_t kStaticTicketSlots = 4096;                   // rows may not exceed this
static __device__ __align__(256) unsigned char g_builtin_scratch[
    kStaticPartialSlots * sizeof(float) + kStaticTicketSlots * sizeof(unsigned)];

namespace {                                                   // nothing below is exported

constexpr int kStaticMaxDevices = 64;
std::mutex g_builtin_mutex;
void* g_builtin_address[kStaticMaxDevices] = {};              // device address, per device

// `g_builtin_scratch` named in host code is only the host-side handle of the symbol, not
// something a kernel can dereference; the device address has to be asked for, once per
// device, while that device is current.
int builtin_scratch_address(void** address) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail_with(MTB_DOMAIN_CUDA + (int)e, cudaGetErrorString(e));
    if (device < 0 || device >= kStaticMaxDevices)
        return fail_with(MTB_E_BAD_ARGUMENT, "mtb_long_row_sum_static: device index out of range");
    std::lock_guard<std::mutex> lock(g_builtin_mutex);
    if (!g_builtin_address[device]) {
        void* found = nullptr;
        e = cudaGetSymbolAddress(&found, g_builtin_scratch);
        if (e != cudaSuccess) return fail_with(MTB_DOMAIN_CUDA + (int)e, cudaGetErrorString(e));
        g_builtin_address[device] = found;
    }
    *address = g_builtin_address[device];
    return 0;
}

}  // namespace

extern "C" {

int mtb_long_row_sum_static(uint64_t x, uint64_t out, int rows, long long cols, void* stream) {
    if (!x || !out) return fail_with(MTB_E_BAD_ARGUMENT, "mtb_long_row_sum_static: NULL buffer");
    int splits = 0;
    long long chunk = 0;
    if (int rc = plan_splits(rows, cols, &splits, &chunk)) return rc;
    if ((size_t)rows > kStaticTicketSlots || (size_t)rows * (size_t)splits > kStaticPartialSlots) {
        char text[200];
        snprintf(text, sizeof text,
                 "mtb_long_row_sum_static: %d rows x %d splits exceeds the built-in scratch "
                 "(%zu rows, %zu partial sums); use mtb_long_row_sum with your own scratch",
                 rows, splits, kStaticTicketSlots, kStaticPartialSlots);
        return fail_with(MTB_E_TOO_LARGE, text);
    }
    void* scratch = nullptr;
    if (int rc = builtin_scratch_address(&scratch)) return rc;
    float* partials = static_cast<float*>(scratch);
    unsigned* tickets = reinterpret_cast<unsigned*>(partials + kStaticPartialSlots);
    return launch_split_row_sum(reinterpret_cast<const float*>(x), reinterpret_cast<float*>(out), rows,
                                cols, splits, chunk, partials, tickets, (cudaStream_t)stream);
}

int mtb_long_row_sum_scratch_bytes(int rows, long long cols, size_t* bytes) {
    if (!bytes) return fail_with(MTB_E_BAD_ARGUMENT, "bytes is NULL");
    int splits = 0;
    long long chunk = 0;
    if (int rc = plan_splits(rows, cols, &splits, &chunk)) return rc;
    *bytes = sizeof(float) * (size_t)rows * (size_t)splits + sizeof(unsigned) * (size_t)rows;
    return 0;
}

int mtb_long_row_sum(uint64_t x, uint64_t out, int rows, long long cols, uint64_t scratch,
                     size_t scratch_bytes, void* stream) {
    if (!x || !out || !scratch) return fail_with(MTB_E_BAD_ARGUMENT, "mtb_long_row_sum: NULL buffer");
    int splits = 0;
    long long chunk = 0;
    if (int rc = plan_splits(rows, cols, &splits, &chunk)) return rc;
    const size_t need = sizeof(float) * (size_t)rows * (size_t)splits + sizeof(unsigned) * (size_t)rows;
    if (scratch_bytes < need) return fail_with(MTB_E_BUFFER_TOO_SMALL, "mtb_long_row_sum: scratch too small");
    if (scratch % 16) return fail_with(MTB_E_BAD_ARGUMENT, "mtb_long_row_sum: scratch must be 16-byte aligned");
    float* partials = reinterpret_cast<float*>(scratch);
    unsigned* tickets = reinterpret_cast<unsigned*>(partials + (size_t)rows * (size_t)splits);
    return launch_split_row_sum(reinterpret_cast<const float*>(x), reinterpret_cast<float*>(out), rows,
                                cols, splits, chunk, partials, tickets, (cudaStream_t)stream);
}

}  // extern "C"
