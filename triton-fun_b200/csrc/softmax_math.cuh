// Register-level arithmetic shared by the tensor-core attention kernels: exp2 on the special
// function unit, packed fp32x2 operations, 3-input max, 16-bit packing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace splat {
namespace sm {

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// packed fp32x2 arithmetic: one issue slot for two lanes of work
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    uint64_t ua = *reinterpret_cast<uint64_t*>(&a), ub = *reinterpret_cast<uint64_t*>(&b),
             uc = *reinterpret_cast<uint64_t*>(&c), ud;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(ud) : "l"(ua), "l"(ub), "l"(uc));
    return *reinterpret_cast<float2*>(&ud);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    uint64_t ua = *reinterpret_cast<uint64_t*>(&a), ub = *reinterpret_cast<uint64_t*>(&b), ud;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(ud) : "l"(ua), "l"(ub));
    return *reinterpret_cast<float2*>(&ud);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    uint64_t ua = *reinterpret_cast<uint64_t*>(&a), ub = *reinterpret_cast<uint64_t*>(&b), ud;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(ud) : "l"(ua), "l"(ub));
    return *reinterpret_cast<float2*>(&ud);
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace sm
}  // namespace splat
