// Shared helpers for the sm_100a kernels of this library.
//
// Every exported entry point is `extern "C"`, takes raw device pointers, sizes and a
// CUDA stream, launches on that stream without synchronising, and returns 0 or an
// error code from the table below.  Nothing here allocates.  The reference launches
// its kernels the same stream-ordered way (src/compute/ComputeOps.hpp:39-41) and
// range-checks kernel arguments on the host before launch
// (src/compute/cuda/GpuOps.cpp:40-47).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MM_OK 0
#define MM_ERR_BAD_ARG 1       // a size or combination the kernel refuses
#define MM_ERR_UNSUPPORTED 2   // valid in principle, not built for this shape/dtype
#define MM_ERR_LAUNCH 3        // cudaGetLastError() after the launch was not success
#define MM_ERR_DRIVER 4        // a driver entry point (tensor map encode) failed

// dtype codes shared with the Python binding
#define MM_F32 0
#define MM_BF16 1

#define MM_EXPORT extern "C" __attribute__((visibility("default")))

#define MM_CHECK_LAUNCH()                                  \
    do {                                                   \
        cudaError_t e__ = cudaGetLastError();              \
        if (e__ != cudaSuccess) {                          \
            mm_set_last_error(cudaGetErrorString(e__));    \
            return MM_ERR_LAUNCH;                          \
        }                                                  \
        ++g_mm_launch_count;                               \
    } while (0)

extern long long g_mm_launch_count;   // kernels of this library launched (or captured) so far
extern int g_mm_pdl;                  // host.cu: dependent launches where they pay (0 off, 1 on)
extern long long g_mm_dep_count;      // the launch count right after the last launch that a dependent launch may follow
extern void* g_mm_dep_stream;

#define MM_REQUIRE(cond, msg)          \
    do {                               \
        if (!(cond)) {                 \
            mm_set_last_error(msg);    \
            return MM_ERR_BAD_ARG;     \
        }                              \
    } while (0)

void mm_set_last_error(const char* msg);

// ---- element conversion ------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- reductions --------------------------------------------------------------
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

// Block-wide sum in a fixed order (lane tree, then warp 0 over the warp partials), so a
// row's result never depends on what else is in the batch.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// ---- launching ------------------------------------------------------------------------------------------------------
// A plain stream-ordered launch with the kernel's parameter types enforced.
template <typename... KArgs, typename... Args>
static inline void mm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- programmatic dependent launch --------------------------------------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may have its blocks scheduled while the kernel before
// it in the stream still runs: they do what does not depend on it (a weight-streaming kernel issues its first weight
// loads), then block in pdl_wait() until that kernel has completed and its writes are visible.  Such a kernel calls
// pdl_wait() before its first read of activations and before any write, and pdl_trigger() once its own weights are
// through, so never more than one kernel is ahead (triggering before the wait let a whole chain of future kernels pile
// up on the SMs and measured 2.5 times slower).  Without the attribute both calls do nothing.
// What decides whether this pays (B200, 7B shapes, batch 8): where the early blocks land.  With room for a third block
// per SM they go wherever the running kernel's blocks leave first (the gate/up product's 296 blocks: three on five SMs and
// one on five others instead of two everywhere), the kernel ends with its fullest SM, and the step is slower (3.35
// against 3.17 ms).  Compiled for two blocks per SM (128 registers a thread, so a third block never fits) a block of the
// next kernel can only take the place of one that left, every SM ends up with its two again, and the step is faster
// (2.98 against 3.05 ms).  Reserving shared memory to the same end does not work: kernels whose shared-memory
// carve-out differs from their neighbours' do not share an SM at all, and the change of carve-out costs more than the
// boundary.  One thread waits, the others stand at the CTA barrier: waiting blocks share their SMs with the running kernel.
__device__ __forceinline__ void pdl_wait() {
    if (threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();
}
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline void mm_launch_dependent(bool dependent, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
