// ACSR metadata construction on the GPU.
//
// Reference semantics (SPLAT/acsr_helpers.py:99-160): per row, nnz and -- when nnz > 1 -- the
// first two set columns a < b give the affine map (stride s = b - a, start a); rows with nnz <= 1
// are described as (stride 1, start 0).  The reference solves a 2x2 system in float64 and later
// rounds to float32; the closed form x = 1/s, y = -a/s evaluated in float64 and rounded once to
// float32 reproduces its tensors bit for bit (checked against fixtures made by the reference).
#include <limits.h>

#include "common.cuh"

namespace splat {

constexpr int kScanThreads = 128;

struct ScanAcc {
    int count, f1, f2, last;
    __device__ __forceinline__ void hit(int idx) {
        if (count == 0) f1 = idx;
        else if (count == 1) f2 = idx;
        last = idx;
        ++count;
    }
};

// One block per row.  Every thread walks its chunks in ascending column order, so the first two
// hits it sees are its two smallest columns.
__global__ void __launch_bounds__(kScanThreads)
mask_row_summary_kernel(const uint8_t* __restrict__ mask, int64_t n_rows, int64_t n_cols,
                        int64_t ld, int vec_ok, int32_t* __restrict__ out) {
    const int64_t row = blockIdx.x;
    const uint8_t* p = mask + row * ld;
    ScanAcc acc{0, INT_MAX, INT_MAX, -1};
    const int tid = threadIdx.x;
    if (vec_ok) {
        const int64_t n_vec = n_cols / 16;
        const uint4* pv = reinterpret_cast<const uint4*>(p);
        for (int64_t c = tid; c < n_vec; c += kScanThreads) {
            uint4 w = __ldg(pv + c);
            if ((w.x | w.y | w.z | w.w) == 0u) continue;
            const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t x = words[k];
                if (x == 0u) continue;
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    if ((x >> (8 * b)) & 0xffu) acc.hit((int)(c * 16 + k * 4 + b));
            }
        }
        // scalar tail: columns [n_vec*16, n_cols) are larger than every vector column, and only
        // thread 0..15 touch them after finishing their vector chunks.
        for (int64_t c = n_vec * 16 + tid; c < n_cols; c += kScanThreads)
            if (p[c]) acc.hit((int)c);
    } else {
        // byte-strided walk: thread t sees columns t, t+128, ... in ascending order
        for (int64_t c = tid; c < n_cols; c += kScanThreads)
            if (p[c]) acc.hit((int)c);
    }

    __shared__ int s_count[kScanThreads / 32], s_f1[kScanThreads / 32], s_last[kScanThreads / 32];
    __shared__ int s_f2[kScanThreads / 32];
    __shared__ int s_gfirst;
    const int lane = tid & 31, warp = tid >> 5;
    int count = warp_sum_i(acc.count);
    int f1 = warp_min_i(acc.f1);
    int last = warp_max_i(acc.last);
    if (lane == 0) { s_count[warp] = count; s_f1[warp] = f1; s_last[warp] = last; }
    __syncthreads();
    if (tid == 0) {
        int g = INT_MAX;
        for (int w = 0; w < kScanThreads / 32; ++w) g = min(g, s_f1[w]);
        s_gfirst = g;
    }
    __syncthreads();
    const int gfirst = s_gfirst;
    // second smallest overall: each thread offers its smallest column that is not the global first
    int cand = (acc.f1 == gfirst) ? acc.f2 : acc.f1;
    cand = warp_min_i(cand);
    if (lane == 0) s_f2[warp] = cand;
    __syncthreads();
    if (tid == 0) {
        int total = 0, glast = -1, gsecond = INT_MAX;
        for (int w = 0; w < kScanThreads / 32; ++w) {
            total += s_count[w];
            glast = max(glast, s_last[w]);
            gsecond = min(gsecond, s_f2[w]);
        }
        out[row] = total > 0 ? gfirst : -1;
        out[n_rows + row] = total > 1 ? gsecond : -1;
        out[2 * n_rows + row] = total > 0 ? glast : -1;
        out[3 * n_rows + row] = total;
    }
}

// Closed-form (start, step, count) of one row of a pattern.
__device__ __forceinline__ void pattern_row(int kind, int64_t n, int64_t p0, int64_t p1, int64_t i,
                                            int64_t& start, int64_t& step, int64_t& count) {
    int64_t end;
    step = 1;
    switch (kind) {
        case SPLAT_PATTERN_BLOCKED:
            if (i < p0) { start = 0; end = p0; }
            else { start = (i / p0 - 1) * p0; end = start + 2 * p0; }
            if (end > n) end = n;
            break;
        case SPLAT_PATTERN_WINDOWED:
            start = i - p0 > 0 ? i - p0 : 0;
            end = i + p0 + 1 < n ? i + p0 + 1 : n;
            break;
        case SPLAT_PATTERN_CAUSAL_WINDOWED:
            start = i - p0 > 0 ? i - p0 : 0;
            end = i + 1;
            break;
        case SPLAT_PATTERN_STRIDED:
            start = i % p0; end = i + 1; step = p0;
            break;
        default: {  // SPLAT_PATTERN_DILATED
            int64_t cnt = i / p1 + 1;
            if (cnt > p0) cnt = p0;
            start = i - p1 * (cnt - 1); end = i + 1; step = p1;
            break;
        }
    }
    count = end > start ? (end - start + step - 1) / step : 0;
}

__global__ void pattern_row_summary_kernel(int kind, int64_t n, int64_t p0, int64_t p1,
                                           int32_t* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int64_t start, step, count;
    pattern_row(kind, n, p0, p1, i, start, step, count);
    out[i] = count > 0 ? (int32_t)start : -1;
    out[n + i] = count > 1 ? (int32_t)(start + step) : -1;
    out[2 * n + i] = count > 0 ? (int32_t)(start + (count - 1) * step) : -1;
    out[3 * n + i] = (int32_t)count;
}

// Each thread writes up to 16 consecutive bytes of one mask row.
__global__ void pattern_mask_kernel(int kind, int64_t n, int64_t p0, int64_t p1,
                                    uint8_t* __restrict__ mask, int64_t ld, int vec_ok) {
    const int64_t c0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 16;
    if (c0 >= n) return;
    for (int64_t row = blockIdx.y; row < n; row += gridDim.y) {
        int64_t start, step, count;
        pattern_row(kind, n, p0, p1, row, start, step, count);
        __align__(16) uint8_t bytes[16];
#pragma unroll
        for (int b = 0; b < 16; ++b) {
            int64_t off = c0 + b - start;
            bytes[b] = (off >= 0 && off % step == 0 && off / step < count) ? 1 : 0;
        }
        uint8_t* dst = mask + row * ld + c0;
        if (vec_ok && c0 + 16 <= n) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(bytes);
        } else {
            for (int b = 0; b < 16 && c0 + b < n; ++b) dst[b] = bytes[b];
        }
    }
}

__global__ void acsr_finalize_kernel(const int32_t* __restrict__ rows, int64_t n_rows,
                                     float* __restrict__ dTos_lin, float* __restrict__ dTos_tr,
                                     float* __restrict__ sTod_lin, float* __restrict__ sTod_tr,
                                     float* __restrict__ nnzs, int32_t* __restrict__ trailing_dim) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int cnt = 0;
    if (i < n_rows) {
        const int a0 = rows[i], b0 = rows[n_rows + i];
        cnt = rows[3 * n_rows + i];
        const bool multi = cnt > 1;
        const double s = multi ? (double)(b0 - a0) : 1.0;
        const double a = multi ? (double)a0 : 0.0;
        const double tr = a / s;           // IEEE division, float64 as in the reference
        dTos_lin[i] = (float)(1.0 / s);
        dTos_tr[i] = (float)(0.0 - tr);    // +0.0 when a == 0
        sTod_lin[i] = (float)s;
        sTod_tr[i] = (float)tr;
        nnzs[i] = (float)cnt;
    }
    cnt = warp_max_i(cnt);
    if ((threadIdx.x & 31) == 0 && cnt > 0) atomicMax(trailing_dim, cnt);
}

// One thread per row block: span = (min start/stride, max nnz*stride + start/stride), initial
// values (n_cols, -1) as in SPLAT/acsr_helpers.py:103,135-140.
__global__ void acsr_span_kernel(const int32_t* __restrict__ rows, int64_t n_rows, int64_t n_cols,
                                 int block_height, int64_t n_blocks,
                                 float* __restrict__ span_start, float* __restrict__ span_end) {
    int64_t blk = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (blk >= n_blocks) return;
    double lo = (double)n_cols, hi = -1.0;
    int64_t r1 = (blk + 1) * block_height;
    if (r1 > n_rows) r1 = n_rows;
    for (int64_t i = blk * block_height; i < r1; ++i) {
        const int a0 = rows[i], b0 = rows[n_rows + i], cnt = rows[3 * n_rows + i];
        const bool multi = cnt > 1;
        const double s = multi ? (double)(b0 - a0) : 1.0;
        const double tr = (multi ? (double)a0 : 0.0) / s;
        lo = fmin(lo, tr);
        hi = fmax(hi, (double)cnt * s + tr);
    }
    span_start[blk] = (float)lo;
    span_end[blk] = (float)hi;
}

__global__ void classify_init_kernel(int32_t* plan) {
    plan[0] = 0;        // max_nnz
    plan[1] = INT_MAX;  // stride_min over rows with nnz > 1
    plan[2] = 0;        // stride_max over rows with nnz > 1
    plan[3] = 0;        // rows with nnz > 1 whose start mod stride != row mod stride
    plan[4] = 0;        // rows with nnz == 1
    plan[5] = 0;        // max column + 1
    plan[6] = 0;        // rows with nnz == 0
    plan[7] = 0;        // rows with nnz > 1
}

__global__ void classify_kernel(const float* __restrict__ sTod_lin,
                                const float* __restrict__ sTod_tr,
                                const float* __restrict__ nnzs, int64_t n_rows,
                                int32_t* __restrict__ plan) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int nnz = 0, smin = INT_MAX, smax = 0, mis = 0, single = 0, maxcol = 0, empty = 0, multi = 0;
    if (i < n_rows) {
        RowAffine r = row_affine(sTod_lin, sTod_tr, nnzs, i);
        nnz = r.nnz;
        if (r.nnz > 1) {
            smin = smax = r.stride;
            mis = (r.start % r.stride) != (int)(i % r.stride);
            multi = 1;
        } else if (r.nnz == 1) single = 1;
        else empty = 1;
        if (r.nnz > 0) maxcol = r.start + (r.nnz - 1) * r.stride + 1;
    }
    nnz = warp_max_i(nnz); smin = warp_min_i(smin); smax = warp_max_i(smax);
    mis = warp_sum_i(mis); single = warp_sum_i(single); maxcol = warp_max_i(maxcol);
    empty = warp_sum_i(empty); multi = warp_sum_i(multi);
    if ((threadIdx.x & 31) == 0) {
        atomicMax(plan + 0, nnz);
        if (multi) { atomicMin(plan + 1, smin); atomicMax(plan + 2, smax); }
        if (mis) atomicAdd(plan + 3, mis);
        if (single) atomicAdd(plan + 4, single);
        atomicMax(plan + 5, maxcol);
        if (empty) atomicAdd(plan + 6, empty);
        if (multi) atomicAdd(plan + 7, multi);
    }
}

}  // namespace splat

using namespace splat;

extern "C" int32_t splat_mask_row_summary_u8(const uint8_t* mask, int64_t n_rows, int64_t n_cols,
                                             int64_t ld, int32_t* rows_i32, void* stream) {
    if (!mask || !rows_i32 || n_rows < 0 || n_cols < 0 || ld < n_cols) return SPLAT_ERR_BAD_ARG;
    if (n_rows > INT_MAX || n_cols > INT_MAX) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (n_rows == 0) return SPLAT_OK;
    const int vec_ok = aligned16(mask) && (ld % 16 == 0);
    mask_row_summary_kernel<<<(unsigned)n_rows, kScanThreads, 0, (cudaStream_t)stream>>>(
        mask, n_rows, n_cols, ld, vec_ok, rows_i32);
    return launch_status();
}

static bool pattern_args_ok(int32_t kind, int64_t n, int64_t p0, int64_t p1) {
    if (n < 0 || n > INT_MAX) return false;
    switch (kind) {
        case SPLAT_PATTERN_BLOCKED: return p0 >= 1;
        case SPLAT_PATTERN_WINDOWED:
        case SPLAT_PATTERN_CAUSAL_WINDOWED: return p0 >= 0;
        case SPLAT_PATTERN_STRIDED: return p0 >= 1;
        case SPLAT_PATTERN_DILATED: return p0 >= 1 && p1 >= 1;
        default: return false;
    }
}

extern "C" int32_t splat_pattern_row_summary(int32_t kind, int64_t n, int64_t p0, int64_t p1,
                                             int32_t* rows_i32, void* stream) {
    if (!rows_i32 || !pattern_args_ok(kind, n, p0, p1)) return SPLAT_ERR_BAD_ARG;
    if (n == 0) return SPLAT_OK;
    pattern_row_summary_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        kind, n, p0, p1, rows_i32);
    return launch_status();
}

extern "C" int32_t splat_pattern_mask_u8(int32_t kind, int64_t n, int64_t p0, int64_t p1,
                                         uint8_t* mask, int64_t ld, void* stream) {
    if (!mask || !pattern_args_ok(kind, n, p0, p1) || ld < n) return SPLAT_ERR_BAD_ARG;
    if (n == 0) return SPLAT_OK;
    const int vec_ok = aligned16(mask) && (ld % 16 == 0);
    const int64_t chunks = (n + 15) / 16;
    dim3 grid((unsigned)((chunks + 127) / 128), (unsigned)(n < 65535 ? n : 65535));
    pattern_mask_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(kind, n, p0, p1, mask, ld, vec_ok);
    return launch_status();
}

extern "C" int32_t splat_acsr_from_row_summary(const int32_t* rows_i32, int64_t n_rows,
                                               int64_t n_cols, int32_t block_height,
                                               float* dTos_lin, float* dTos_tr, float* sTod_lin,
                                               float* sTod_tr, float* nnzs, float* span_start,
                                               float* span_end, int32_t* trailing_dim_dev,
                                               void* stream) {
    if (!rows_i32 || !dTos_lin || !dTos_tr || !sTod_lin || !sTod_tr || !nnzs || !span_start ||
        !span_end || !trailing_dim_dev || n_rows < 0 || n_cols < 0 || block_height < 1)
        return SPLAT_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(trailing_dim_dev, 0, sizeof(int32_t), st) != cudaSuccess)
        return SPLAT_ERR_LAUNCH;
    if (n_rows == 0) return SPLAT_OK;
    acsr_finalize_kernel<<<(unsigned)((n_rows + 255) / 256), 256, 0, st>>>(
        rows_i32, n_rows, dTos_lin, dTos_tr, sTod_lin, sTod_tr, nnzs, trailing_dim_dev);
    const int64_t n_blocks = (n_rows + block_height - 1) / block_height;
    acsr_span_kernel<<<(unsigned)((n_blocks + 127) / 128), 128, 0, st>>>(
        rows_i32, n_rows, n_cols, block_height, n_blocks, span_start, span_end);
    return launch_status();
}

extern "C" int32_t splat_acsr_classify(const float* sTod_lin, const float* sTod_tr,
                                       const float* nnzs, int64_t n_rows, int32_t* plan_i32,
                                       void* stream) {
    if (!sTod_lin || !sTod_tr || !nnzs || !plan_i32 || n_rows < 0) return SPLAT_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    classify_init_kernel<<<1, 1, 0, st>>>(plan_i32);
    if (n_rows > 0)
        classify_kernel<<<(unsigned)((n_rows + 255) / 256), 256, 0, st>>>(sTod_lin, sTod_tr, nnzs,
                                                                          n_rows, plan_i32);
    return launch_status();
}
