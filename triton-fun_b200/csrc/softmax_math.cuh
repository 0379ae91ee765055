// Register-level arithmetic shared by the tensor-core attention kernels: exp2 on the special
// function unit and on the FMA pipes, packed fp32x2 operations, 3-input max, 16-bit packing.
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

// 2^x for -125 <= x < 128 without the special function unit, two values at a time on the packed
// fp32x2 pipes: split x into floor(x) + f with the round-down magic-number addition, evaluate 2^f
// on [0, 1) with a cubic that is exact at both ends (maximum relative error 1.04e-4, a quarter of
// the rounding step of a 16-bit-float probability and a twentieth of a bfloat16 one), then add
// floor(x) into the exponent field.  Inputs below -125 are clamped: the result is then 2^-125
// instead of something smaller, which no sum of probabilities can see.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
    const float kMagic = 12582912.f;   // 1.5 * 2^23: x + kMagic holds floor(x) in its low mantissa bits
    const float2 xc = make_float2(fmaxf(x.x, -125.f), fmaxf(x.y, -125.f));
    float2 sh;
    asm("add.rm.f32 %0, %1, %2;" : "=f"(sh.x) : "f"(xc.x), "f"(kMagic));
    asm("add.rm.f32 %0, %1, %2;" : "=f"(sh.y) : "f"(xc.y), "f"(kMagic));
    const float2 fl = add2(sh, make_float2(-kMagic, -kMagic));          // floor(x), exact
    const float2 f = add2(xc, make_float2(-fl.x, -fl.y));              // x - floor(x) in [0, 1)
    const float c1 = 0.6954243779182434f, c2 = 0.226307675242424f, c3 = 0.07826796919107437f;
    float2 p = fma2(f, make_float2(c3, c3), make_float2(c2, c2));
    p = fma2(p, f, make_float2(c1, c1));
    p = fma2(p, f, make_float2(1.f, 1.f));                             // 2^f in [1, 2]
    float2 y;
    y.x = __uint_as_float(__float_as_uint(p.x) + (__float_as_uint(sh.x) << 23));
    y.y = __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(sh.y) << 23));
    return y;
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
