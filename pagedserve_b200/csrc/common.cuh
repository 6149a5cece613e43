// Shared helpers for the sm_100a kernels of pagedserve_b200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PS_OK 0
#define PS_ERR_BAD_ARGUMENT 1
#define PS_ERR_UNSUPPORTED 2
#define PS_ERR_LAUNCH 3

// dtype codes shared with the Python side
#define PS_F32 0
#define PS_BF16 1

// activation codes
#define PS_ACT_NONE 0
#define PS_ACT_GELU_TANH 1
#define PS_ACT_GELU_ERF 2

#define PS_EXPORT extern "C" __attribute__((visibility("default")))

namespace ps {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
__device__ __forceinline__ float gelu_tanh(float x) {
    const float k = 0.7978845608028654f;
    float inner = k * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(inner));
}
// 0.5 x (1 + erf(x / sqrt 2))
__device__ __forceinline__ float gelu_erf(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
}
__device__ __forceinline__ float apply_act(float x, int act) {
    if (act == PS_ACT_GELU_TANH) return gelu_tanh(x);
    if (act == PS_ACT_GELU_ERF) return gelu_erf(x);
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

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? PS_OK : PS_ERR_LAUNCH;
}

}  // namespace ps
