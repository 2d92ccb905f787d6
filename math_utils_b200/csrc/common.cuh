// Shared device helpers for the sm_100a kernels of this library.
//
// Every launcher is an extern "C" function that takes raw device pointers,
// sizes and a stream, checks what it can on the host, and returns 0 or one of
// the MU_ERR_* codes below (the Python side turns a code into an exception).
// No launcher allocates, synchronises or reads device memory on the host.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_set>

#define MU_OK 0
#define MU_ERR_BAD_ARGUMENT 1      // a size or pointer the kernel cannot take
#define MU_ERR_UNSUPPORTED_SIZE 2  // a size outside what this kernel was written for
#define MU_ERR_LAUNCH 3            // the CUDA runtime refused the launch
#define MU_ERR_ALIGNMENT 4         // a pointer or stride that breaks an alignment rule

#define MU_EXPORT extern "C" __attribute__((visibility("default")))

#define MU_CHECK_LAUNCH()                                   \
    do {                                                    \
        cudaError_t e__ = cudaGetLastError();               \
        if (e__ != cudaSuccess) return MU_ERR_LAUNCH;       \
    } while (0)

namespace mu {

constexpr int ACT_NONE = 0;
constexpr int ACT_GELU_NEW = 1;   // tanh form
constexpr int ACT_GELU_ERF = 2;   // exact form

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float gelu_new(float x) {
    const float k = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_erf(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
}
// 0.5 (1 + tanh y) = 1 / (1 + exp(-2 y)), so gelu_new(x) = x / (1 + exp(-2 y)): no tanh, no
// cancellation for negative x, a fast exponential and a fast division (errors of a few 2^-22).
// For results that are rounded to bfloat16 right after; the float32 path keeps the tanhf form.
__device__ __forceinline__ float gelu_new_fast(float x) {
    const float k = 0.7978845608028654f;
    const float y = k * (x + 0.044715f * x * x * x);
    return __fdividef(x, 1.0f + __expf(-2.0f * y));
}
// The activation for an output that is stored as bfloat16.
__device__ __forceinline__ float apply_act_bf16(float x, int act) {
    if (act == ACT_GELU_NEW) return gelu_new_fast(x);
    if (act == ACT_GELU_ERF) return gelu_erf(x);
    return x;
}
__device__ __forceinline__ float apply_act(float x, int act) {
    if (act == ACT_GELU_NEW) return gelu_new(x);
    if (act == ACT_GELU_ERF) return gelu_erf(x);
    return x;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; every thread gets the result.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    r = warp_sum(r);
    return r;
}

// --- programmatic dependent launch -------------------------------------------------------
// Kernels of the single-token step are launched so that the next one may start while the
// previous one drains: it runs its prologue (index arithmetic, prefetch of weights, which
// no kernel ever writes) and then waits, at pdl_wait(), until every kernel before it has
// finished and its results are visible.  Nothing that another kernel produces is read, and
// nothing at all is written, before that wait.  pdl_trigger() lets the next kernel in.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// SMs of the current device (asked once: this library drives one device per process); 0 on failure.
inline int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
            sms = 0;
    }
    return sms;
}

inline int& pdl_enabled() {
    static int enabled = 1;
    return enabled;
}

// Launches with the programmatic-serialization attribute (if enabled) and, when cluster_y > 1,
// as thread-block clusters of (1, cluster_y, 1).
// The kernels of a prompt step ask for the largest shared-memory share of the SM's on-chip memory, whether
// they use it or not: the large products and the attention need it, and an SM that has to change the split
// between shared memory and L1 from one kernel to the next first runs empty.  (The kernels of single-token
// steps are better off with the L1 they get by default.)
inline void prefer_shared_memory(const void* kernel) {
    static std::mutex mutex;
    static std::unordered_set<const void*> seen;
    std::lock_guard<std::mutex> lock(mutex);
    if (seen.insert(kernel).second) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaGetLastError();
    }
}

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      int cluster_y, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_y > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = (unsigned)cluster_y;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) == cudaSuccess ? MU_OK : MU_ERR_LAUNCH;
}

}  // namespace mu
