// Storage-type access for kernels that run in bfloat16 or float32 storage: loads widen to fp32, stores round once.
#pragma once
#include <cuda_bf16.h>

namespace kge {
template <typename E> __device__ __forceinline__ float ldf(const E* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename E> __device__ __forceinline__ void stf(E* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
// the value after one rounding to the storage type
template <typename E> __device__ __forceinline__ float rnd(float v);
template <> __device__ __forceinline__ float rnd<float>(float v) { return v; }
template <> __device__ __forceinline__ float rnd<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
}  // namespace kge
