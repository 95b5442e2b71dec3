// Fan-out copy: one contiguous block of device memory written to several destinations.
//
// The row-panel schedule of the sharded GEMM pushes every finished panel of C to the same
// rows of each peer's C.  Copy engines do that well for one peer and poorly for several at
// once; this kernel reads the panel once (from L2, where the GEMM has just written it) and
// stores it to every destination with 128-bit stores — ordinary peer stores over NVLink, no
// multicast, no loads from peer memory.  It needs no shared memory and few registers, so its
// CTAs run beside the persistent GEMM's CTAs on the same SMs.  The reference has no
// multi-device path; this belongs to the M-sharded benchmark configuration.

#include "mtb200_rt.h"

#include <cuda_runtime.h>

#include <cstdint>

namespace {

struct Destinations { unsigned long long p[8]; };

int fail_fanout(int code, const char* text) {
    mtb_set_last_error(text);
    return code;
}

__global__ __launch_bounds__(256)
void fanout_copy_kernel(const float4* __restrict__ src, Destinations dst, int n_dst, long long n_vec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_vec; i += stride * 4) {
        float4 v[4];
        #pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long index = i + u * stride;
            if (index < n_vec) v[u] = __ldcg(src + index);          // L2 only: the data is not re-read here
        }
        for (int d = 0; d < n_dst; ++d) {
            float4* out = reinterpret_cast<float4*>(dst.p[d]);
            #pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long index = i + u * stride;
                if (index < n_vec) out[index] = v[u];
            }
        }
    }
}

}  // namespace

extern "C" int mtb_fanout_copy(uint64_t src, const uint64_t* destinations, int n_destinations,
                               size_t bytes, int ctas, void* stream) {
    if (!src || !destinations) return fail_fanout(MTB_E_BAD_ARGUMENT, "mtb_fanout_copy: NULL argument");
    if (n_destinations < 1 || n_destinations > 8)
        return fail_fanout(MTB_E_BAD_ARGUMENT, "mtb_fanout_copy: 1 to 8 destinations");
    if (bytes % 16 || src % 16) return fail_fanout(MTB_E_BAD_ARGUMENT, "mtb_fanout_copy: size and addresses must be multiples of 16 bytes");
    Destinations dst = {};
    for (int d = 0; d < n_destinations; ++d) {
        if (!destinations[d] || destinations[d] % 16)
            return fail_fanout(MTB_E_BAD_ARGUMENT, "mtb_fanout_copy: size and addresses must be multiples of 16 bytes");
        dst.p[d] = destinations[d];
    }
    if (bytes == 0) return 0;
    if (ctas <= 0) ctas = 296;                       // two per SM of a B200
    const long long n_vec = (long long)(bytes / 16);
    fanout_copy_kernel<<<ctas, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4*>(src), dst, n_destinations, n_vec);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail_fanout(MTB_DOMAIN_CUDA + (int)e, cudaGetErrorString(e));
    return 0;
}
