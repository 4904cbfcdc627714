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
// gate functions of a gated feed-forward (0 = the product has no gated epilogue)
enum : int { MRUN_GATE_NONE = 0, MRUN_GATE_SILU = 1, MRUN_GATE_GELU_TANH = 2 };
#define MRUN_REQUIRE_GATE(act, name) \
    MRUN_REQUIRE((act) == MRUN_GATE_SILU || (act) == MRUN_GATE_GELU_TANH, "%s: unknown gate function code %d", name, act)

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

namespace mrun {

// Launches a kernel whose arguments are given with the caller's types (they are converted to the
// kernel's parameter types) and returns the launch's error code.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    return cudaLaunchKernelEx(&config, kernel, KArgs(args)...);
}

// Programmatic dependent launch.  A kernel launched with launch_kernel_overlapped() may begin
// while the kernel before it in the stream is still running, once that kernel has let it
// (dependents_may_start(), or its end).  Until wait_for_kernel_before() returns it may only read
// memory that no kernel of the step writes (weights, the step's index arrays) and may write
// nothing: the memory of its outputs may still be in use by the kernel before.  A kernel lets its
// own successor start only after its own wait, so that never more than two kernels share the
// device.  Both calls do nothing in a kernel that was launched the plain way.
__device__ __forceinline__ void wait_for_kernel_before() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dependents_may_start() { asm volatile("griddepcontrol.launch_dependents;"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
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
    config.numAttrs = 1;
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

// act(gate) * up, the gate's function named by a code of the C ABI.  The 32-bit path divides and
// takes the exponential exactly; the bfloat16 kernels (the stand-alone kernel and the GEMM
// epilogues alike, so that a decode step and a prompt step give the same number) use the
// special-function unit: a relative error near 2^-21 for SiLU, far inside bfloat16's rounding,
// and a sixth of the instructions.  Another gate function is one more case here and one more
// name in the Python table; no kernel changes.
template <bool EXACT>
__device__ __forceinline__ float gated_mul(int act, float gate, float up) {
    if (act == MRUN_GATE_GELU_TANH) {
        const float inner = 0.7978845608028654f * (gate + 0.044715f * gate * gate * gate);
        float th;
        if constexpr (EXACT) th = tanhf(inner);
        else asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(inner));
        return 0.5f * gate * (1.f + th) * up;
    }
    if constexpr (EXACT) return gate / (1.f + expf(-gate)) * up;
    else return __fdividef(gate, 1.f + __expf(-gate)) * up;
}

}  // namespace mrun
