// CUDA-core kernels for SDDMM, row softmax, SpMM and a fused chain over ACSR.  They consume only
// the per-row affine metadata, so they are correct for every metadata the builder can produce
// (any stride, ragged rows, empty rows) and for fp32 inputs with true fp32 FMA.  The tensor-core
// band kernel covers the regular, 16-bit cases; these kernels are the general path.
//
// Work decomposition: one warp per sparse row.
//   SDDMM  : lanes own slots (slot j -> dense column start + j*stride); the Q row sits in shared
//            memory as fp32 and is broadcast; a lane streams its K row with 16-byte loads when K is
//            row-contiguous, or walks a contiguous K^T with lane-coalesced scalar loads.
//   SpMM   : the warp is split into G groups of d/vec lanes; group g handles slots j == g (mod G)
//            and each lane accumulates one 16-byte chunk of the output row; groups are reduced
//            with shuffles at the end.
//   fused  : 32 slots at a time -- scores as in SDDMM, online max/sum with exp2 and the softmax
//            scale folded into the exponent, then the SpMM accumulation with the probabilities
//            broadcast by shuffle.
#include "common.cuh"

namespace splat {

constexpr int kWarpsPerBlock = 4;

// Checked-index mode (splat_debug_check_indices): while a word is registered, every dense column
// these kernels derive from the row metadata is compared with [0, n_cols); a column outside it is
// clamped to the nearest valid one before it is dereferenced and the kernel's code is recorded in
// the word (the first code stays).  Off (null) the comparison is skipped.
static int32_t* g_index_check = nullptr;
enum : int32_t { kIndexSddmm = 71, kIndexSpmm = 72, kIndexFused = 73 };

__device__ __forceinline__ int64_t slot_col(const RowAffine& ra, int j, int64_t n_cols, int32_t* check,
                                            int32_t code) {
    int64_t col = (int64_t)ra.start + (int64_t)j * ra.stride;
    if (check != nullptr && (col < 0 || col >= n_cols)) {
        atomicCAS(check, 0, code);
        col = col < 0 ? 0 : n_cols - 1;
    }
    return col;
}

// ---------------------------------------------------------------------------------------------
// dot(Q row in shared memory, K[col, :])
// ---------------------------------------------------------------------------------------------
template <typename T, bool kRowContig>
__device__ __forceinline__ float dot_qk(const float* __restrict__ qs, const T* __restrict__ kbh,
                                        int64_t col, int d, int64_t ksc, int64_t ksk) {
    float acc = 0.f;
    if constexpr (kRowContig) {
        const T* kr = kbh + col * ksc;
        constexpr int V = DT<T>::kVec;
        float tmp[V];
        for (int k0 = 0; k0 < d; k0 += V) {
            load16_as_float(kr + k0, tmp);
#pragma unroll
            for (int t = 0; t < V; ++t) acc = fmaf(qs[k0 + t], tmp[t], acc);
        }
    } else {
        const T* kc = kbh + col * ksc;
        for (int k0 = 0; k0 < d; ++k0) acc = fmaf(qs[k0], DT<T>::to_f(kc[(int64_t)k0 * ksk]), acc);
    }
    return acc;
}

template <typename T>
__device__ __forceinline__ void stage_q_row(float* qs, const T* __restrict__ qrow, int d, int lane) {
    for (int k0 = lane; k0 < d; k0 += 32) qs[k0] = DT<T>::to_f(qrow[k0]);
    __syncwarp();
}

// ---------------------------------------------------------------------------------------------
// SDDMM
// ---------------------------------------------------------------------------------------------
template <typename T, bool kRowContig>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
sddmm_rows_kernel(const T* __restrict__ q, const T* __restrict__ k, int64_t ksb, int64_t ksc,
                  int64_t ksk, T* __restrict__ out, const float* __restrict__ lin,
                  const float* __restrict__ tr, const float* __restrict__ nnzs, int64_t total_rows,
                  int64_t n_rows, int64_t n_cols, int d, int trailing, int32_t* check) {
    extern __shared__ float smem_q[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t grow = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
    if (grow >= total_rows) return;
    const int64_t bh = grow / n_rows, row = grow % n_rows;
    float* qs = smem_q + (size_t)warp * d;
    stage_q_row(qs, q + grow * d, d, lane);
    const RowAffine ra = row_affine(lin, tr, nnzs, row);
    const T* kbh = k + bh * ksb;
    T* orow = out + grow * trailing;
    for (int j = lane; j < trailing; j += 32) {
        float v = 0.f;
        if (j < ra.nnz) v = dot_qk<T, kRowContig>(qs, kbh, slot_col(ra, j, n_cols, check, kIndexSddmm),
                                                  d, ksc, ksk);
        orow[j] = DT<T>::from_f(v);
    }
}

// ---------------------------------------------------------------------------------------------
// Row softmax.  Variant A keeps the row in registers (16-byte loads, up to kMaxVec vectors per
// lane); variant B re-reads the row (any trailing dimension or alignment).
// ---------------------------------------------------------------------------------------------
constexpr int kSoftmaxMaxVec = 4;

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
softmax_rows_vec_kernel(const T* s, T* p, const float* __restrict__ nnzs,
                        int64_t total_rows, int64_t n_rows, int trailing, float scale_log2e) {
    constexpr int V = DT<T>::kVec;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t grow = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
    if (grow >= total_rows) return;
    int nnz = (int)rintf(__ldg(nnzs + grow % n_rows));
    nnz = nnz < 0 ? 0 : (nnz > trailing ? trailing : nnz);
    const T* srow = s + grow * trailing;
    T* prow = p + grow * trailing;
    float vals[kSoftmaxMaxVec][V];
    float m = -INFINITY;
#pragma unroll
    for (int v = 0; v < kSoftmaxMaxVec; ++v) {
        const int e0 = (v * 32 + lane) * V;
        if (e0 < nnz) {
            load16_as_float(srow + e0, vals[v]);
#pragma unroll
            for (int t = 0; t < V; ++t) {
                vals[v][t] = (e0 + t < nnz) ? vals[v][t] * scale_log2e : -INFINITY;
                m = fmaxf(m, vals[v][t]);
            }
        } else {
#pragma unroll
            for (int t = 0; t < V; ++t) vals[v][t] = -INFINITY;
        }
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < kSoftmaxMaxVec; ++v)
#pragma unroll
        for (int t = 0; t < V; ++t) {
            const float e = (vals[v][t] == -INFINITY) ? 0.f : exp2f(vals[v][t] - m);
            vals[v][t] = e;
            sum += e;
        }
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
    for (int v = 0; v < kSoftmaxMaxVec; ++v) {
        const int e0 = (v * 32 + lane) * V;
        if (e0 < trailing) {
#pragma unroll
            for (int t = 0; t < V; ++t) vals[v][t] *= inv;
            store16_from_float(prow + e0, vals[v]);
        }
    }
}

// Rows of at most one 16-byte vector per lane (trailing_dim <= 32 * V): a warp takes R rows at a
// time and issues all their loads before the first reduction, so that enough bytes are in flight to
// keep HBM busy (one row per warp leaves the warp waiting on a single 512-byte request).
template <typename T, int R>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
softmax_rows_short_kernel(const T* s, T* p, const float* __restrict__ nnzs,
                          int64_t total_rows, int64_t n_rows, int trailing, float scale_log2e) {
    constexpr int V = DT<T>::kVec;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t grow0 = ((int64_t)blockIdx.x * kWarpsPerBlock + warp) * R;
    if (grow0 >= total_rows) return;
    const int e0 = lane * V;
    float vals[R][V];
    int nnz[R];
    const int64_t in_head0 = grow0 % n_rows;   // one 64-bit division per warp
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int64_t grow = grow0 + r;
        nnz[r] = 0;
        if (grow < total_rows) {
            int64_t in_head = in_head0 + r;
            while (in_head >= n_rows) in_head -= n_rows;
            int n = (int)rintf(__ldg(nnzs + in_head));
            nnz[r] = n < 0 ? 0 : (n > trailing ? trailing : n);
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (e0 < nnz[r]) {
            load16_as_float(s + (grow0 + r) * trailing + e0, vals[r]);
        } else {
#pragma unroll
            for (int t = 0; t < V; ++t) vals[r][t] = 0.f;
        }
    }
    float m[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m[r] = -INFINITY;
#pragma unroll
        for (int t = 0; t < V; ++t) {
            vals[r][t] = (e0 + t < nnz[r]) ? vals[r][t] * scale_log2e : -INFINITY;
            m[r] = fmaxf(m[r], vals[r][t]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int r = 0; r < R; ++r) m[r] = fmaxf(m[r], __shfl_xor_sync(0xffffffffu, m[r], o));
    float sum[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        sum[r] = 0.f;
#pragma unroll
        for (int t = 0; t < V; ++t) {
            const float e = (vals[r][t] == -INFINITY) ? 0.f : exp2f(vals[r][t] - m[r]);
            vals[r][t] = e;
            sum[r] += e;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int r = 0; r < R; ++r) sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], o);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (grow0 + r < total_rows && e0 < trailing) {
            const float inv = sum[r] > 0.f ? 1.f / sum[r] : 0.f;
#pragma unroll
            for (int t = 0; t < V; ++t) vals[r][t] *= inv;
            store16_from_float(p + (grow0 + r) * trailing + e0, vals[r]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
softmax_rows_loop_kernel(const T* s, T* p,
                         const float* __restrict__ nnzs, int64_t total_rows, int64_t n_rows,
                         int trailing, float scale_log2e) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t grow = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
    if (grow >= total_rows) return;
    int nnz = (int)rintf(__ldg(nnzs + grow % n_rows));
    nnz = nnz < 0 ? 0 : (nnz > trailing ? trailing : nnz);
    const T* srow = s + grow * trailing;
    T* prow = p + grow * trailing;
    float m = -INFINITY;
    for (int j = lane; j < nnz; j += 32) m = fmaxf(m, DT<T>::to_f(srow[j]) * scale_log2e);
    m = warp_max(m);
    float sum = 0.f;
    for (int j = lane; j < nnz; j += 32) sum += exp2f(DT<T>::to_f(srow[j]) * scale_log2e - m);
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    // s and p may alias: every element is read by the lane that overwrites it
    for (int j = lane; j < trailing; j += 32) {
        float v = 0.f;
        if (j < nnz) v = exp2f(DT<T>::to_f(srow[j]) * scale_log2e - m) * inv;
        prow[j] = DT<T>::from_f(v);
    }
}

// ---------------------------------------------------------------------------------------------
// SpMM accumulation helpers: the warp is G groups of LPG lanes; lane owns one 16-byte chunk.
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void accum_v(float* acc, float pv, const T* __restrict__ vrow_chunk) {
    constexpr int V = DT<T>::kVec;
    float tmp[V];
    load16_as_float(vrow_chunk, tmp);
#pragma unroll
    for (int t = 0; t < V; ++t) acc[t] = fmaf(pv, tmp[t], acc[t]);
}

template <int V>
__device__ __forceinline__ void reduce_groups(float* acc, int lpg) {
    for (int o = lpg; o < 32; o <<= 1)
#pragma unroll
        for (int t = 0; t < V; ++t) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
}

// lanes-per-group = d / vec must be a power of two <= 32 (host checks).
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
spmm_rows_kernel(const T* __restrict__ p, const T* __restrict__ v, T* __restrict__ o,
                 const float* __restrict__ lin, const float* __restrict__ tr,
                 const float* __restrict__ nnzs, int64_t total_rows, int64_t n_rows,
                 int64_t n_cols, int d, int trailing, int32_t* check) {
    constexpr int V = DT<T>::kVec;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t grow = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
    if (grow >= total_rows) return;
    const int64_t bh = grow / n_rows, row = grow % n_rows;
    const RowAffine ra = row_affine(lin, tr, nnzs, row);
    const int nnz = ra.nnz > trailing ? trailing : ra.nnz;
    const int lpg = d / V, G = 32 / lpg, g = lane / lpg, c0 = (lane % lpg) * V;
    const T* prow = p + grow * trailing;
    const T* vbh = v + bh * n_cols * d;
    float acc[V];
#pragma unroll
    for (int t = 0; t < V; ++t) acc[t] = 0.f;
    for (int j0 = 0; j0 < nnz; j0 += 32) {
        const int j = j0 + lane;
        const float pj = j < nnz ? DT<T>::to_f(prow[j]) : 0.f;
        const int lim = min(32, nnz - j0);
        // uniform trip count: every lane takes part in every shuffle
        for (int t0 = 0; t0 < lim; t0 += G) {
            const int t = t0 + g;
            const float pv = __shfl_sync(0xffffffffu, pj, t & 31);
            if (t < lim) {
                const int64_t col = slot_col(ra, j0 + t, n_cols, check, kIndexSpmm);
                accum_v<T>(acc, pv, vbh + col * d + c0);
            }
        }
    }
    reduce_groups<V>(acc, lpg);
    if (g == 0) store16_from_float(o + grow * d + c0, acc);
}

// Scalar SpMM for head dimensions the grouped kernel does not take.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
spmm_rows_scalar_kernel(const T* __restrict__ p, const T* __restrict__ v, T* __restrict__ o,
                        const float* __restrict__ lin, const float* __restrict__ tr,
                        const float* __restrict__ nnzs, int64_t total_rows, int64_t n_rows,
                        int64_t n_cols, int d, int trailing, int32_t* check) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t grow = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
    if (grow >= total_rows) return;
    const int64_t bh = grow / n_rows, row = grow % n_rows;
    const RowAffine ra = row_affine(lin, tr, nnzs, row);
    const int nnz = ra.nnz > trailing ? trailing : ra.nnz;
    const T* prow = p + grow * trailing;
    const T* vbh = v + bh * n_cols * d;
    for (int c = lane; c < d; c += 32) {
        float acc = 0.f;
        for (int j = 0; j < nnz; ++j) {
            const int64_t col = slot_col(ra, j, n_cols, check, kIndexSpmm);
            acc = fmaf(DT<T>::to_f(prow[j]), DT<T>::to_f(vbh[col * d + c]), acc);
        }
        o[grow * d + c] = DT<T>::from_f(acc);
    }
}

// ---------------------------------------------------------------------------------------------
// Fused SDDMM -> softmax -> SpMM, one warp per row, scores stay in registers.
// ---------------------------------------------------------------------------------------------
template <typename T, bool kRowContig>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attention_rows_kernel(const T* __restrict__ q, const T* __restrict__ k, int64_t ksb, int64_t ksc,
                      int64_t ksk, const T* __restrict__ v, T* __restrict__ o,
                      const float* __restrict__ lin, const float* __restrict__ tr,
                      const float* __restrict__ nnzs, int64_t total_rows, int64_t n_rows,
                      int64_t n_cols, int d, float scale_log2e, int32_t* check, float* lse) {
    constexpr int V = DT<T>::kVec;
    extern __shared__ float smem_q[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t grow = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
    if (grow >= total_rows) return;
    const int64_t bh = grow / n_rows, row = grow % n_rows;
    float* qs = smem_q + (size_t)warp * d;
    stage_q_row(qs, q + grow * d, d, lane);
    const RowAffine ra = row_affine(lin, tr, nnzs, row);
    const T* kbh = k + bh * ksb;
    const T* vbh = v + bh * n_cols * d;
    const int lpg = d / V, G = 32 / lpg, g = lane / lpg, c0 = (lane % lpg) * V;
    float acc[V];
#pragma unroll
    for (int t = 0; t < V; ++t) acc[t] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int j0 = 0; j0 < ra.nnz; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j < ra.nnz;
        float sc = -INFINITY;
        const int64_t col = valid ? slot_col(ra, j, n_cols, check, kIndexFused) : 0;
        if (valid) sc = dot_qk<T, kRowContig>(qs, kbh, col, d, ksc, ksk) * scale_log2e;
        const float m_new = fmaxf(m, warp_max(sc));      // finite: lane 0 of every chunk is valid
        const float corr = exp2f(m - m_new);              // 0 on the first chunk
        const float pj = valid ? exp2f(sc - m_new) : 0.f;
        l = l * corr + warp_sum(pj);
        m = m_new;
#pragma unroll
        for (int t = 0; t < V; ++t) acc[t] *= corr;
        const int lim = min(32, ra.nnz - j0);
        for (int t0 = 0; t0 < lim; t0 += G) {
            const int t = t0 + g;
            const float pv = __shfl_sync(0xffffffffu, pj, t & 31);
            if (t < lim) {
                const int64_t ct = slot_col(ra, j0 + t, n_cols, check, kIndexFused);
                accum_v<T>(acc, pv, vbh + ct * d + c0);
            }
        }
    }
    reduce_groups<V>(acc, lpg);
    if (lse != nullptr && lane == 0) lse[grow] = lse_from_log2(m, l);
    if (g == 0) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int t = 0; t < V; ++t) acc[t] *= inv;
        store16_from_float(o + grow * d + c0, acc);
    }
}

// ---------------------------------------------------------------------------------------------
// Host dispatch
// ---------------------------------------------------------------------------------------------
static bool grouped_d_ok(int64_t d, int vec) {
    if (d % vec) return false;
    int64_t lpg = d / vec;
    return lpg >= 1 && lpg <= 32 && (lpg & (lpg - 1)) == 0;
}

template <typename T>
static int32_t sddmm_t(const void* q, const void* k, int64_t ksb, int64_t ksc, int64_t ksk,
                       void* out, const float* lin, const float* tr, const float* nnzs, int64_t bh,
                       int64_t n_rows, int64_t n_cols, int64_t d, int64_t trailing, cudaStream_t st) {
    const int64_t total = bh * n_rows;
    const unsigned grid = (unsigned)((total + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const size_t smem = (size_t)kWarpsPerBlock * d * sizeof(float);
    const bool contig = ksk == 1 && (d % DT<T>::kVec == 0) && aligned16(k) &&
                        (ksc % DT<T>::kVec == 0) && (ksb % DT<T>::kVec == 0);
    if (contig)
        sddmm_rows_kernel<T, true><<<grid, kWarpsPerBlock * 32, smem, st>>>(
            (const T*)q, (const T*)k, ksb, ksc, ksk, (T*)out, lin, tr, nnzs, total, n_rows, n_cols, (int)d,
            (int)trailing, g_index_check);
    else
        sddmm_rows_kernel<T, false><<<grid, kWarpsPerBlock * 32, smem, st>>>(
            (const T*)q, (const T*)k, ksb, ksc, ksk, (T*)out, lin, tr, nnzs, total, n_rows, n_cols, (int)d,
            (int)trailing, g_index_check);
    return launch_status();
}

template <typename T>
static int32_t softmax_t(const void* s, void* p, const float* nnzs, int64_t bh, int64_t n_rows,
                         int64_t trailing, float scale, cudaStream_t st) {
    const int64_t total = bh * n_rows;
    const unsigned grid = (unsigned)((total + kWarpsPerBlock - 1) / kWarpsPerBlock);
    constexpr int V = DT<T>::kVec;
    const bool vec = (trailing % V == 0) && trailing <= 32 * V * kSoftmaxMaxVec && aligned16(s) &&
                     aligned16(p);
    if (vec && trailing <= 32 * V) {
        constexpr int R = 2;
        const unsigned grid_r = (unsigned)((total + (int64_t)kWarpsPerBlock * R - 1) / (kWarpsPerBlock * R));
        softmax_rows_short_kernel<T, R><<<grid_r, kWarpsPerBlock * 32, 0, st>>>(
            (const T*)s, (T*)p, nnzs, total, n_rows, (int)trailing, scale * kLog2e);
    } else if (vec)
        softmax_rows_vec_kernel<T><<<grid, kWarpsPerBlock * 32, 0, st>>>(
            (const T*)s, (T*)p, nnzs, total, n_rows, (int)trailing, scale * kLog2e);
    else
        softmax_rows_loop_kernel<T><<<grid, kWarpsPerBlock * 32, 0, st>>>(
            (const T*)s, (T*)p, nnzs, total, n_rows, (int)trailing, scale * kLog2e);
    return launch_status();
}

template <typename T>
static int32_t spmm_t(const void* p, const void* v, void* o, const float* lin, const float* tr,
                      const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                      int64_t trailing, cudaStream_t st) {
    const int64_t total = bh * n_rows;
    const unsigned grid = (unsigned)((total + kWarpsPerBlock - 1) / kWarpsPerBlock);
    if (grouped_d_ok(d, DT<T>::kVec) && aligned16(v) && aligned16(o))
        spmm_rows_kernel<T><<<grid, kWarpsPerBlock * 32, 0, st>>>(
            (const T*)p, (const T*)v, (T*)o, lin, tr, nnzs, total, n_rows, n_cols, (int)d,
            (int)trailing, g_index_check);
    else
        spmm_rows_scalar_kernel<T><<<grid, kWarpsPerBlock * 32, 0, st>>>(
            (const T*)p, (const T*)v, (T*)o, lin, tr, nnzs, total, n_rows, n_cols, (int)d,
            (int)trailing, g_index_check);
    return launch_status();
}

template <typename T>
static int32_t attention_t(const void* q, const void* k, int64_t ksb, int64_t ksc, int64_t ksk,
                           const void* v, void* o, const float* lin, const float* tr,
                           const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                           float scale, float* lse, cudaStream_t st) {
    if (!grouped_d_ok(d, DT<T>::kVec) || !aligned16(v) || !aligned16(o))
        return SPLAT_ERR_UNSUPPORTED_SHAPE;
    const int64_t total = bh * n_rows;
    const unsigned grid = (unsigned)((total + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const size_t smem = (size_t)kWarpsPerBlock * d * sizeof(float);
    const bool contig = ksk == 1 && aligned16(k) && (ksc % DT<T>::kVec == 0) &&
                        (ksb % DT<T>::kVec == 0);
    if (contig)
        attention_rows_kernel<T, true><<<grid, kWarpsPerBlock * 32, smem, st>>>(
            (const T*)q, (const T*)k, ksb, ksc, ksk, (const T*)v, (T*)o, lin, tr, nnzs, total,
            n_rows, n_cols, (int)d, scale * kLog2e, g_index_check, lse);
    else
        attention_rows_kernel<T, false><<<grid, kWarpsPerBlock * 32, smem, st>>>(
            (const T*)q, (const T*)k, ksb, ksc, ksk, (const T*)v, (T*)o, lin, tr, nnzs, total,
            n_rows, n_cols, (int)d, scale * kLog2e, g_index_check, lse);
    return launch_status();
}

static bool sizes_ok(int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d, int64_t trailing) {
    return bh >= 0 && n_rows >= 0 && n_cols >= 0 && d >= 1 && trailing >= 0 && d <= 2048 &&
           n_rows <= INT32_MAX && n_cols <= INT32_MAX && trailing <= INT32_MAX &&
           bh * n_rows / kWarpsPerBlock < (int64_t)INT32_MAX;
}

int32_t attention_generic(const void* q, const void* k, int64_t ksb, int64_t ksc, int64_t ksk,
                          const void* v, void* o, const float* lin, const float* tr,
                          const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                          float scale, int32_t dtype, float* lse, cudaStream_t st) {
    if (!sizes_ok(bh, n_rows, n_cols, d, 0)) return SPLAT_ERR_BAD_ARG;
    if (bh * n_rows == 0) return SPLAT_OK;   // empty batch: nothing to read or write, pointers may be null
    if (!q || !k || !v || !o || !lin || !tr || !nnzs) return SPLAT_ERR_BAD_ARG;
    switch (dtype) {
        case SPLAT_F32: return attention_t<float>(q, k, ksb, ksc, ksk, v, o, lin, tr, nnzs, bh, n_rows, n_cols, d, scale, lse, st);
        case SPLAT_F16: return attention_t<__half>(q, k, ksb, ksc, ksk, v, o, lin, tr, nnzs, bh, n_rows, n_cols, d, scale, lse, st);
        case SPLAT_BF16: return attention_t<__nv_bfloat16>(q, k, ksb, ksc, ksk, v, o, lin, tr, nnzs, bh, n_rows, n_cols, d, scale, lse, st);
        default: return SPLAT_ERR_UNSUPPORTED_DTYPE;
    }
}

}  // namespace splat

using namespace splat;

extern "C" int32_t splat_debug_check_indices(int32_t* status_word) {
    g_index_check = status_word;
    return SPLAT_OK;
}

extern "C" int32_t splat_sddmm(const void* q, const void* k, int64_t k_stride_bh,
                               int64_t k_stride_col, int64_t k_stride_k, void* s_out,
                               const float* sTod_lin, const float* sTod_tr, const float* nnzs,
                               int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                               int64_t trailing_dim, int32_t dtype, void* stream) {
    if (!sizes_ok(bh, n_rows, n_cols, d, trailing_dim)) return SPLAT_ERR_BAD_ARG;
    if (bh * n_rows * trailing_dim == 0) return SPLAT_OK;   // empty: pointers may be null
    if (!q || !k || !s_out || !sTod_lin || !sTod_tr || !nnzs) return SPLAT_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case SPLAT_F32: return sddmm_t<float>(q, k, k_stride_bh, k_stride_col, k_stride_k, s_out, sTod_lin, sTod_tr, nnzs, bh, n_rows, n_cols, d, trailing_dim, st);
        case SPLAT_F16: return sddmm_t<__half>(q, k, k_stride_bh, k_stride_col, k_stride_k, s_out, sTod_lin, sTod_tr, nnzs, bh, n_rows, n_cols, d, trailing_dim, st);
        case SPLAT_BF16: return sddmm_t<__nv_bfloat16>(q, k, k_stride_bh, k_stride_col, k_stride_k, s_out, sTod_lin, sTod_tr, nnzs, bh, n_rows, n_cols, d, trailing_dim, st);
        default: return SPLAT_ERR_UNSUPPORTED_DTYPE;
    }
}

extern "C" int32_t splat_softmax(const void* s_in, void* p_out, const float* nnzs, int64_t bh,
                                 int64_t n_rows, int64_t trailing_dim, float scale, int32_t dtype,
                                 void* stream) {
    if (!sizes_ok(bh, n_rows, 0, 1, trailing_dim)) return SPLAT_ERR_BAD_ARG;
    if (bh * n_rows * trailing_dim == 0) return SPLAT_OK;   // empty: pointers may be null
    if (!s_in || !p_out || !nnzs) return SPLAT_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case SPLAT_F32: return softmax_t<float>(s_in, p_out, nnzs, bh, n_rows, trailing_dim, scale, st);
        case SPLAT_F16: return softmax_t<__half>(s_in, p_out, nnzs, bh, n_rows, trailing_dim, scale, st);
        case SPLAT_BF16: return softmax_t<__nv_bfloat16>(s_in, p_out, nnzs, bh, n_rows, trailing_dim, scale, st);
        default: return SPLAT_ERR_UNSUPPORTED_DTYPE;
    }
}

extern "C" int32_t splat_spmm(const void* p, const void* v, void* o, const float* sTod_lin,
                              const float* sTod_tr, const float* nnzs, int64_t bh, int64_t n_rows,
                              int64_t n_cols, int64_t d, int64_t trailing_dim, int32_t dtype,
                              void* stream) {
    if (!sizes_ok(bh, n_rows, n_cols, d, trailing_dim)) return SPLAT_ERR_BAD_ARG;
    if (bh * n_rows == 0) return SPLAT_OK;   // empty: pointers may be null
    if (!p || !v || !o || !sTod_lin || !sTod_tr || !nnzs) return SPLAT_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case SPLAT_F32: return spmm_t<float>(p, v, o, sTod_lin, sTod_tr, nnzs, bh, n_rows, n_cols, d, trailing_dim, st);
        case SPLAT_F16: return spmm_t<__half>(p, v, o, sTod_lin, sTod_tr, nnzs, bh, n_rows, n_cols, d, trailing_dim, st);
        case SPLAT_BF16: return spmm_t<__nv_bfloat16>(p, v, o, sTod_lin, sTod_tr, nnzs, bh, n_rows, n_cols, d, trailing_dim, st);
        default: return SPLAT_ERR_UNSUPPORTED_DTYPE;
    }
}
