// Shared declarations of the kernel library: C ABI, error reporting, dtype codes, reductions.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and a stream, allocates
// nothing, and returns 0 or a non-zero code after storing a message that mrun_last_error()
// returns.  Sizes that a kernel cannot take are refused here, never computed wrongly.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MRUN_API extern "C" __attribute__((visibility("default")))

// dtype codes of the C ABI
enum : int { MRUN_F32 = 0, MRUN_BF16 = 1 };

// Stores a printf-style message for the calling thread and returns a non-zero code.
int mrun_set_error(const char* fmt, ...);

#define MRUN_REQUIRE(cond, ...)                       \
    do {                                              \
        if (!(cond)) return mrun_set_error(__VA_ARGS__); \
    } while (0)

#define MRUN_CHECK_LAUNCH(name)                                                         \
    do {                                                                                \
        cudaError_t err__ = cudaGetLastError();                                         \
        if (err__ != cudaSuccess)                                                       \
            return mrun_set_error("%s: launch failed: %s", name, cudaGetErrorString(err__)); \
    } while (0)

#define MRUN_CHECK_CUDA(call, name)                                                     \
    do {                                                                                \
        cudaError_t err__ = (call);                                                     \
        if (err__ != cudaSuccess)                                                       \
            return mrun_set_error("%s: %s", name, cudaGetErrorString(err__));           \
    } while (0)

// Which kernel classes are launched so that their blocks may start while the kernel before them
// in the stream is still running: a bit mask from the environment variable MRUN_PDL
// (1 = norm/rotary/activation kernels, 2 = the decode GEMM, 4 = the decode attention).
enum : int { MRUN_PDL_ELEMENTWISE = 1, MRUN_PDL_GEMM = 2, MRUN_PDL_ATTENTION = 4 };
bool mrun_pdl_enabled(int kernel_class);

namespace mrun {

// Programmatic dependent launch.  A kernel launched with launch_pdl() may begin before the
// previous kernel in its stream has finished; it must call pdl_wait() before it reads anything
// that kernel wrote and before it writes anything at all.  What it does before the wait (index
// arithmetic, loads of weights and of other data that no kernel of the step writes) overlaps the
// previous kernel's tail.  pdl_launch_dependents() lets the *next* kernel's blocks be scheduled
// once every block of this one has reached it.  It is called after pdl_wait(), never before: a
// kernel that released its successor before waiting itself would let a whole chain of kernels
// pile up on the SMs, each holding block slots while it waits for the one before it.  Both are
// no-ops in a kernel launched normally.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(int kernel_class, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = mrun_pdl_enabled(kernel_class) ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, KArgs(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Sum over a warp in a fixed butterfly order: every lane gets the same bits.
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

// Block-wide sum / max for blockDim.x a multiple of 32 (at most 1024).  `scratch` holds 33
// floats.  The order of additions depends on blockDim.x only, so a row's result does not depend
// on what else the launch computes.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// SiLU(gate) * up.  The 32-bit path divides and takes the exponential exactly; the bfloat16
// kernels (the stand-alone SwiGLU and the GEMM epilogues alike, so that a decode step and a prompt
// step give the same number) use the special-function unit for both: a relative error near
// 2^-21, far inside bfloat16's rounding, and a sixth of the instructions.
template <bool EXACT>
__device__ __forceinline__ float silu_mul(float gate, float up) {
    if constexpr (EXACT) return gate / (1.f + expf(-gate)) * up;
    else return __fdividef(gate, 1.f + __expf(-gate)) * up;
}

}  // namespace mrun
