// Shared device/host helpers for the splat_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "splat_b200.h"

namespace splat {

// ---------------------------------------------------------------------------------------------
// dtype traits: load/store as float, 16-byte vector widths.
// ---------------------------------------------------------------------------------------------
template <typename T> struct DT;
template <> struct DT<float> {
    static constexpr int kVec = 4;  // elements per 16 bytes
    __device__ static __forceinline__ float to_f(float x) { return x; }
    __device__ static __forceinline__ float from_f(float x) { return x; }
};
template <> struct DT<__half> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ float to_f(__half x) { return __half2float(x); }
    __device__ static __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};
template <> struct DT<__nv_bfloat16> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
    __device__ static __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};

// 16 bytes of T, unpacked to floats.
template <typename T>
__device__ __forceinline__ void load16_as_float(const T* p, float* out) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < DT<T>::kVec; ++i) out[i] = DT<T>::to_f(e[i]);
}

template <typename T>
__device__ __forceinline__ void store16_from_float(T* p, const float* in) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < DT<T>::kVec; ++i) e[i] = DT<T>::from_f(in[i]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// ---------------------------------------------------------------------------------------------
// Row metadata: float32 triple of the reference -> integers.
// stride = sTod_lin, start = rint(sTod_tr * sTod_lin) (sTod_tr holds start/stride), nnz = nnzs.
// ---------------------------------------------------------------------------------------------
struct RowAffine {
    int start;
    int stride;
    int nnz;
};

__device__ __forceinline__ RowAffine row_affine(const float* __restrict__ sTod_lin,
                                                const float* __restrict__ sTod_tr,
                                                const float* __restrict__ nnzs, int64_t row) {
    RowAffine r;
    float lin = __ldg(sTod_lin + row);
    float tr = __ldg(sTod_tr + row);
    r.stride = (int)rintf(lin);
    if (r.stride < 1) r.stride = 1;
    r.start = (int)rint((double)tr * (double)r.stride);
    r.nnz = (int)rintf(__ldg(nnzs + row));
    if (r.nnz < 0) r.nnz = 0;
    return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_min_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_max_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------------------------
// Host-side helpers.
// ---------------------------------------------------------------------------------------------
inline int32_t launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SPLAT_OK : SPLAT_ERR_LAUNCH;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int elem_size(int32_t dtype) { return dtype == SPLAT_F32 ? 4 : 2; }

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Natural-log log-sum-exp of a row from its running maximum m and sum l = sum_j 2^(s_j - m), both in
// the log2 domain (scores already multiplied by scale * log2 e); -inf for a row without non-zeros.
__device__ __forceinline__ float lse_from_log2(float m, float l) {
    return l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;
}
// dot(a[0..d), b[0], b[stride], ...) in fp32: the single score of a row with one non-zero.
template <typename T>
__device__ __forceinline__ float dot_strided(const T* a, const T* b, int64_t b_stride, int d) {
    float acc = 0.f;
    for (int c = 0; c < d; ++c) acc = fmaf(DT<T>::to_f(a[c]), DT<T>::to_f(b[(int64_t)c * b_stride]), acc);
    return acc;
}

}  // namespace splat
