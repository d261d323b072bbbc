// Shared helpers of the sm_100a kernels: element types, status reporting, reductions.
//
// Every exported function has C linkage, takes raw device pointers plus the stream to
// launch on, and returns 0 on success.  On failure it returns a non-zero code and leaves
// a message that `jk_last_error` hands out; nothing calls exit().  (The reference's
// RUN_INFINI macro prints and exits the process: src/utils.hpp:10-34.)
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define JK_EXPORT extern "C" __attribute__((visibility("default")))

enum JkDtype : int { JK_F32 = 0, JK_BF16 = 1 };

enum JkStatus : int {
    JK_OK = 0,
    JK_BAD_ARGUMENT = 1,
    JK_UNSUPPORTED = 2,
    JK_CUDA_ERROR = 3,
};

// One per shared object, defined by JK_DEFINE_ERROR_BUFFER; hidden, so that a module loaded into a program
// that already has another module's symbols keeps writing to its own.
__attribute__((visibility("hidden"))) char *jk_error_buffer();

#define JK_DEFINE_ERROR_BUFFER(prefix)                                              \
    static thread_local char g_error[512] = "";                                    \
    __attribute__((visibility("hidden"))) char *jk_error_buffer() { return g_error; }                                  \
    JK_EXPORT const char *prefix##_last_error() { return g_error; }

#define JK_FAIL(code, ...)                                                          \
    do {                                                                            \
        snprintf(jk_error_buffer(), 512, __VA_ARGS__);                              \
        return (code);                                                              \
    } while (0)

#define JK_REQUIRE(cond, ...)                                                       \
    do {                                                                            \
        if (!(cond)) JK_FAIL(JK_BAD_ARGUMENT, __VA_ARGS__);                         \
    } while (0)

#define JK_CHECK_LAUNCH(name)                                                       \
    do {                                                                            \
        cudaError_t e_ = cudaGetLastError();                                        \
        if (e_ != cudaSuccess)                                                      \
            JK_FAIL(JK_CUDA_ERROR, "%s: %s", name, cudaGetErrorString(e_));         \
    } while (0)

// ---- programmatic dependent launch ---------------------------------------------------------
// Every kernel of this package is launched with the attribute that lets it start while the kernel
// before it in the stream is still running.  A kernel calls pdl_trigger() first (the kernel after
// it may then be scheduled as soon as all blocks of this one have started) and pdl_wait() before it
// reads anything an earlier kernel wrote and before its own first global write; what it does in
// between (setting up shared memory, prefetching weights) overlaps the earlier kernel's tail.
// Both are no-ops in a launch without the attribute.  JK_NO_PDL=1 in the environment turns it off.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

#ifndef __CUDA_ARCH__
#include <cstdlib>
#include <mutex>
#include <set>
#include <utility>
static inline bool jk_pdl_enabled() {
    static const bool on = [] { const char *e = std::getenv("JK_NO_PDL"); return !(e && e[0] == '1'); }();
    return on;
}
// Every kernel asks for the same split of the SM's on-chip memory (all of it shared memory): a step is
// a chain of short kernels, and an SM that has to change the split between two of them drains first.
static inline void jk_prefer_shared(const void *kernel) {
    static const bool on = [] { const char *e = std::getenv("JK_NO_CARVEOUT"); return !(e && e[0] == '1'); }();
    if (!on) return;
    static std::mutex mu;
    static std::set<const void *> seen;
    std::lock_guard<std::mutex> lock(mu);
    if (seen.insert(kernel).second)
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}
#endif

// `cluster` > 1 launches thread-block clusters of that many blocks along x (the grid is a multiple of it).
template <typename... KArgs, typename... Args>
static inline cudaError_t jk_launch_clusters(void (*kernel)(KArgs...), int cluster, dim3 grid, dim3 block, size_t smem,
                                             cudaStream_t stream, Args &&...args) {
#ifndef __CUDA_ARCH__
    jk_prefer_shared(reinterpret_cast<const void *>(kernel));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (jk_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
#else
    return cudaSuccess;
#endif
}

template <typename... KArgs, typename... Args>
static inline cudaError_t jk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args &&...args) {
    return jk_launch_clusters(kernel, 1, grid, block, smem, stream, std::forward<Args>(args)...);
}

// ---- element access: storage type T (float or __nv_bfloat16), arithmetic in float ----
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// ---- reductions ------------------------------------------------------------------------
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

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds
// 33 floats of shared memory.  The order of the additions depends on the block size only.
__device__ __forceinline__ float block_sum(float v, float *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
