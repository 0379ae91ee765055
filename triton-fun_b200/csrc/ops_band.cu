// SDDMM and SpMM over ACSR for patterns whose rows are contiguous bands after regrouping by residue
// class (the same condition and the same (d, stride, L/stride, BH) tensor-map view as the fused
// kernel in attention_band.cu): TMA-staged tiles, tcgen05 MMAs with the accumulator in tensor
// memory.  Both kernels are bound by the (BH, L, trailing_dim) sparse operand they write or read;
// the tensor cores only have to keep up with that stream.
//
//   sddmm_band_kernel   S[i, j'] = Q[i] . K[start_i + j' stride]   (SPLAT/r_sddmm.py:16-114)
//       one CTA = one 128-row Q tile of one (bh, residue class), eight row warps; K travels in 64-key ring items;
//       S(k) = Q K(k)^T (8 x tcgen05.mma 128x64x16) lands in one of two 64-column buffers; the
//       store warps read their row's 64 scores, convert, transpose through shared memory and write
//       each row's run of the band into the sparse layout with coalesced stores.
//   spmm_band_kernel    O[i] = sum_j' P[i, j'] V[start_i + j' stride]   (SPLAT/r_spmm.py:14-164)
//       the loader warps gather each row's run of P for a 64-key step (coalesced), zero outside
//       the band, into a 128-byte-swizzled K-major tile in shared memory; O += P(k) V(k) is
//       4 x tcgen05.mma 128xdx16 with both operands in shared memory; O leaves through a TMA store.
// Rows with one non-zero (described by the metadata as column `start`, outside the band) and rows
// with none are fixed up by plain loads, padding slots of S are written as zero like the
// CUDA-core kernels do.
#include <limits.h>
#include <type_traits>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace splat {
namespace band {

using namespace tc;

// defined in attention_band.cu
bool allow_dynamic_smem(const void* kernel, int bytes);
bool make_map(CUtensorMap* map, const void* base, int32_t dtype, int64_t bh, int64_t n_rows,
              int64_t d, int64_t stride, int box_rows);
bool make_map_kt(CUtensorMap* map, const void* base, int32_t dtype, int64_t bh, int64_t n_cols,
                 int64_t d);

namespace ops {

constexpr int kTile = 128;
constexpr int kStep = 64;
constexpr int kSubBytes = kTile * 128;          // 128 rows x 128 bytes
constexpr int kStepBytesPerSub = kStep * 128;   // 64 keys x 128 bytes
constexpr int kRowWarps = 8;                    // row warp (q, h) = (warp & 3, warp >> 2): rows 32q .. 32q+31, half h of the work
constexpr int kThreads = 320;                   // warps 0-7 rows, 8 TMA producer, 9 MMA issuer
constexpr int kTmaWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kStages = 3;                     // ring depth that lets two CTAs share an SM at d = 128
constexpr int kStagePitch = 144;                // bytes per staged row: 128 + 16, conflict-free 16-byte stores
enum : int { kErrQ = 11, kErrFull = 12, kErrEmpty = 13, kErrReady = 14, kErrFree = 15 };

struct Params {
#ifdef SPLAT_OPS_TRACE
    long long* trace;
#endif
    const float* lin;
    const float* tr;
    const float* nnzs;
    const void* q;       // sddmm: (BH, L, d), for rows with one non-zero
    const void* kv;      // sddmm: K, spmm: V, (BH, L, d)
    void* sparse;        // sddmm: S out, spmm: P in, (BH, L, trailing_dim)
    int32_t* status;
    int64_t n_rows;      // L
    int rows_v;          // L / stride
    int stride;
    int trailing_dim;
    int direct;          // sddmm: S is 16-byte aligned, full runs may be stored straight from registers
    int kt_major;        // sddmm: K is a contiguous (BH, d, L) array (keys innermost), stride 1 only
};

#ifdef SPLAT_OPS_TRACE
#define OPS_TRACE(tag)                                                                    \
    do {                                                                                  \
        if (trace_on && lane == 0 && trace_n < 256) p.trace[trace_role * 256 + trace_n++] = ((long long)(tag) << 48) | (clock64() & 0xffffffffffffLL); \
    } while (0)
#else
#define OPS_TRACE(tag) do { } while (0)
#endif

__device__ __forceinline__ void wait_quiet(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > 200000000LL) break;
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
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

struct Control {
    uint64_t q_full;
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t ready[2];   // sddmm: scores of a step in tensor memory; spmm: P tile of a step in shared memory
    uint64_t freed[2];   // the consumer is through with that buffer
    uint64_t drain;
    uint32_t tmem_base;
    int32_t abort_at_entry;
    int32_t red_lo[4];
    int32_t red_hi[4];
    // per row and step: where its run of the sparse operand starts in global memory and which of
    // the step's 64 columns it covers; written by the row's own lane, read by the whole warp
    struct RowRun { unsigned long long ptr; int lo; int hi; } run[kRowWarps][32];   // one copy per row warp
};

// Per-row band metadata of the 128 rows of a tile, and the tile's step range [klo, khi).
struct RowInfo {
    int a;       // first band column in class coordinates (rows with more than one non-zero)
    int n;       // non-zeros of such a row, else 0
    int nnz;     // non-zeros of the row as the metadata has it
    int start;   // first column as the metadata has it
};

__device__ __forceinline__ RowInfo load_row(const Params& p, int u, int res) {
    RowInfo r{0, 0, 0, 0};
    if (u < p.rows_v) {
        const RowAffine ra = row_affine(p.lin, p.tr, p.nnzs, (int64_t)u * p.stride + res);
        r.nnz = ra.nnz;
        r.start = ra.start;
        if (ra.nnz > 1) {
            r.a = (ra.start - res) / p.stride;
            r.n = ra.nnz;
        }
    }
    return r;
}

// Stores 32 consecutive 16-bit elements (w[j] = elements 2j, 2j+1) at element offset g0 of a
// 16-byte-aligned array, from one thread, with the widest aligned stores the offset allows: the
// data is shifted in registers by g0 mod 8 elements (a 16-bit funnel shift for the odd part, two
// rounds of selects for the word part, no divergence), the three middle 16-byte chunks go out
// whole, the partial first and last chunks in 8/4/2-byte pieces.  Ten store instructions per warp
// for 2 KB instead of one shared-memory load and one 2-byte store per element.
__device__ __forceinline__ void store_run_shifted(uint16_t* base, long long g0, const uint32_t (&w)[16]) {
    const int sft = (int)(g0 & 7);
    uint16_t* gp = base + (g0 - sft);   // 16-byte aligned
    const bool odd = sft & 1;
    uint32_t v[20];
#pragma unroll
    for (int j = 0; j < 17; ++j) {
        const uint32_t lo = j > 0 ? w[j - 1] : 0u, hi = j < 16 ? w[j] : 0u;
        v[j] = odd ? __funnelshift_l(lo, hi, 16) : hi;
    }
    v[17] = v[18] = v[19] = 0u;
    if (sft & 2) {
#pragma unroll
        for (int j = 19; j >= 1; --j) v[j] = v[j - 1];
        v[0] = 0u;
    }
    if (sft & 4) {
#pragma unroll
        for (int j = 19; j >= 2; --j) v[j] = v[j - 2];
        v[0] = v[1] = 0u;
    }
    // whole chunks 1..3 (relative elements 8..31 are always inside [sft, sft + 32))
#pragma unroll
    for (int c = 1; c < 4; ++c)
        *reinterpret_cast<uint4*>(gp + 8 * c) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    // first chunk: relative elements [sft, 8)
    if (sft == 0) {
        *reinterpret_cast<uint4*>(gp) = make_uint4(v[0], v[1], v[2], v[3]);
    } else {
        if (odd) {   // element sft: upper half of word sft >> 1
            const uint32_t wv = sft < 4 ? (sft < 2 ? v[0] : v[1]) : (sft < 6 ? v[2] : v[3]);
            gp[sft] = (uint16_t)(wv >> 16);
        }
        const int t1 = sft + (sft & 1);           // even, 2..8
        if (t1 & 2) *reinterpret_cast<uint32_t*>(gp + t1) = t1 == 2 ? v[1] : v[3];
        const int t2 = t1 + (t1 & 2);             // 4 or 8
        if (t2 == 4) *reinterpret_cast<uint2*>(gp + 4) = make_uint2(v[2], v[3]);
    }
    // last chunk: relative elements [32, 32 + sft)
    if (sft & 4) *reinterpret_cast<uint2*>(gp + 32) = make_uint2(v[16], v[17]);
    if (sft & 2) *reinterpret_cast<uint32_t*>(gp + 32 + (sft & 4)) = (sft & 4) ? v[18] : v[16];
    if (odd) {
        const int e = sft & 6;                    // 0, 2, 4, 6: lower half of word 16 + e / 2
        const uint32_t wv = e < 4 ? (e < 2 ? v[16] : v[17]) : (e < 6 ? v[18] : v[19]);
        gp[32 + e] = (uint16_t)(wv & 0xffffu);
    }
}

// ---------------------------------------------------------------------------------------------
// SDDMM
// ---------------------------------------------------------------------------------------------
template <int D> struct SddmmLayout {
    static constexpr int kSub = D / 64;
    static constexpr int kQBytes = kSub * kSubBytes;
    static constexpr int kItemBytes = kSub * kStepBytesPerSub;
    static constexpr int kRingOff = kQBytes;
    static constexpr int kStageOff = kRingOff + kStages * kItemBytes;
    static constexpr int kCtrlOff = kStageOff + kTile * kStagePitch;
    static constexpr int kSmemBytes = kCtrlOff + (int)sizeof(Control) + 1024;
};

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 3)
sddmm_band_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const Params p) {
    using L = SddmmLayout<D>;
    constexpr int kTmemCols = 128;   // two 64-column score buffers
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* s_q = smem;
    uint8_t* s_ring = smem + L::kRingOff;
    uint8_t* s_stage = smem + L::kStageOff;
    Control* ctrl = reinterpret_cast<Control*>(smem + L::kCtrlOff);
    volatile int32_t* status = p.status;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int res = blockIdx.y;
    const int64_t bh = blockIdx.z;
    const int u0 = blockIdx.x * kTile;
#ifdef SPLAT_OPS_TRACE
    const bool trace_on = p.trace != nullptr && blockIdx.x == gridDim.x / 2 && blockIdx.z == gridDim.z / 2 && (warp == 0 || warp == kMmaWarp);
    const int trace_role = warp == 0 ? 0 : 1;
    int trace_n = 0;
    OPS_TRACE(1);
#endif

    if (warp == kMmaWarp) {
        tmem_alloc(&ctrl->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    if (threadIdx.x == 0) {
        mbar_init(&ctrl->q_full, 1);
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&ctrl->full[i], 1);
            mbar_init(&ctrl->empty[i], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctrl->ready[b], 1);
            mbar_init(&ctrl->freed[b], kRowWarps);
        }
        mbar_init(&ctrl->drain, 1);
        mbar_fence_init();
        ctrl->abort_at_entry = *status;
    }
    RowInfo me{0, 0, 0, 0};
    if (warp < kRowWarps) {
        me = load_row(p, u0 + (warp & 3) * 32 + lane, res);
        int lo = me.n > 0 ? me.a / kStep : INT_MAX;
        int hi = me.n > 0 ? (me.a + me.n + kStep - 1) / kStep : 0;
        lo = warp_min_i(lo);
        hi = warp_max_i(hi);
        if (lane == 0 && warp < 4) { ctrl->red_lo[warp] = lo; ctrl->red_hi[warp] = hi; }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;
    if (ctrl->abort_at_entry != 0) {
        if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
        return;
    }
    int klo = INT_MAX, khi = 0;
    for (int w = 0; w < 4; ++w) {
        klo = min(klo, ctrl->red_lo[w]);
        khi = max(khi, ctrl->red_hi[w]);
    }
    khi = min(khi, (p.rows_v + kStep - 1) / kStep);
    if (klo >= khi) { klo = 0; khi = 0; }
    const int steps = khi - klo;

    if (warp == kTmaWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && steps > 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            mbar_arrive_expect_tx(&ctrl->q_full, L::kQBytes);
            for (int sub = 0; sub < L::kSub; ++sub)
                tma_load_4d(s_q + sub * kSubBytes, &tm_q, &ctrl->q_full, sub * 64, res, u0, (int)bh);
            int item = 0;
            bool ok = true;
            for (int k = klo; k < khi; ++k, ++item) {
                const int stage = item % kStages;
                const uint32_t parity = ((uint32_t)(item / kStages) & 1u) ^ 1u;
                if (!mbar_wait(&ctrl->empty[stage], parity, status, kErrEmpty)) { ok = false; break; }
                mbar_arrive_expect_tx(&ctrl->full[stage], L::kItemBytes);
                if (p.kt_major)      // one [d][64 keys] block (K layouts: see attention_band.cu)
                    tma_load_4d(s_ring + stage * L::kItemBytes, &tm_k, &ctrl->full[stage], k * kStep, 0,
                                (int)bh, 0);
                else
                    for (int sub = 0; sub < L::kSub; ++sub)
                        tma_load_4d(s_ring + stage * L::kItemBytes + sub * kStepBytesPerSub, &tm_k,
                                    &ctrl->full[stage], sub * 64, res, k * kStep, (int)bh);
            }
            if (!ok) {   // leave only after the copies already issued have landed
                wait_quiet(&ctrl->q_full, 0);
                for (int i = max(0, item - kStages); i < item; ++i)
                    wait_quiet(&ctrl->full[i % kStages], (uint32_t)(i / kStages) & 1u);
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        // (the whole warp walks the loop on warp-uniform values and one elected lane issues: a
        // single lane in a divergent branch is issue-bound on tcgen05.mma)
        if (steps > 0) {
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            const uint32_t idesc = instr_desc_f16(fmt, kTile, kStep, p.kt_major ? 1u : 0u);
            const bool lead = elect_one();
            auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
                const bool r = mbar_wait(bar, parity, status, code);
                return __all_sync(0xffffffffu, r) != 0;
            };
            const uint32_t ring_addr = smem_u32(s_ring), q_base = smem_u32(s_q);
            bool ok = wait_all(&ctrl->q_full, 0, kErrQ);
            uint32_t free_phase[2] = {0, 0};
            for (int k = klo; k < khi && ok; ++k) {
                const int item = k - klo, b = k & 1;
                ok = wait_all(&ctrl->full[item % kStages], (uint32_t)(item / kStages) & 1u, kErrFull);
                if (ok && item >= 2) {   // the store warps have read the scores that were in this buffer
                    ok = wait_all(&ctrl->freed[b], free_phase[b], kErrFree);
                    free_phase[b] ^= 1u;
                }
                if (!ok) break;
                tc_fence_after_sync();
                OPS_TRACE(20);
                const uint32_t b_base = ring_addr + (item % kStages) * L::kItemBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t da = smem_desc_sw128(q_base + (kk >> 2) * kSubBytes + (kk & 3) * 32, 16, 1024);
                    const uint64_t db = p.kt_major
                        ? smem_desc_sw128(b_base + kk * 2048, D * 128, 1024)
                        : smem_desc_sw128(b_base + (kk >> 2) * kStepBytesPerSub + (kk & 3) * 32, 16, 1024);
                    if (lead) mma_ss(tmem_base + b * kStep, da, db, idesc, kk > 0);
                }
                if (lead) {
                    mma_commit(&ctrl->empty[item % kStages]);
                    mma_commit(&ctrl->ready[b]);
                }
                OPS_TRACE(21);
            }
            // let the tensor pipe drain before tensor memory is released
            if (lead) mma_commit(&ctrl->drain);
            wait_quiet(&ctrl->drain, 0);
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------------ store warps
        // Warp (q, h): rows 32q .. 32q+31 (its tensor-memory lanes), columns [32h, 32h + 32) of
        // every 64-column step.  Each warp stages and writes out only what its own lanes read.
        const int q = warp & 3, h = warp >> 2;
        const uint32_t s_addr = tmem_base + ((uint32_t)(q * 32) << 16) + h * 32;
        T* out = reinterpret_cast<T*>(p.sparse);
        uint8_t* my_stage = s_stage + (q * 32) * kStagePitch + h * 64;   // this warp's half of the 128-byte rows
        const int64_t row0 = bh * p.n_rows;   // + real row
        uint32_t phase[2] = {0, 0};
        bool ok = true;
        for (int k = klo; k < khi; ++k) {
            const int b = k & 1;
            OPS_TRACE(4);
            ok = mbar_wait(&ctrl->ready[b], phase[b], status, kErrReady);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            phase[b] ^= 1u;
            tc_fence_after_sync();
            OPS_TRACE(5);
            uint32_t r[32];
            tmem_ld32(s_addr + b * kStep, r);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->freed[b]);   // the buffer may take the scores of step k + 2
            OPS_TRACE(6);
            const int c0 = k * kStep + h * 32;   // first column of this warp's half
            // Fast path, every row of the warp has all 32 columns of this half inside its band:
            // each thread writes its own run straight from registers.
            if (p.direct && __all_sync(0xffffffffu, me.n > 0 && me.a <= c0 && me.a + me.n >= c0 + 32)) {
                uint32_t w[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    w[j] = pack2<T>(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                const int64_t real = (int64_t)(u0 + q * 32 + lane) * p.stride + res;
                store_run_shifted(reinterpret_cast<uint16_t*>(out),
                                  (long long)((row0 + real) * p.trailing_dim + (c0 - me.a)), w);
                continue;
            }
            // own row -> staging (16-bit), then row by row out of staging with coalesced stores
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint4 v4;
                v4.x = pack2<T>(__uint_as_float(r[8 * c + 0]), __uint_as_float(r[8 * c + 1]));
                v4.y = pack2<T>(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3]));
                v4.z = pack2<T>(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5]));
                v4.w = pack2<T>(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7]));
                *reinterpret_cast<uint4*>(my_stage + lane * kStagePitch + c * 16) = v4;
            }
            {   // this lane's row: destination of column c0 and the valid columns of the half
                const int64_t real = (int64_t)(u0 + q * 32 + lane) * p.stride + res;
                Control::RowRun rrn;
                rrn.ptr = reinterpret_cast<unsigned long long>(out + (row0 + real) * p.trailing_dim + (c0 - me.a));
                rrn.lo = me.n > 0 ? max(me.a - c0, 0) : 0;
                rrn.hi = me.n > 0 ? min(me.a + me.n - c0, 32) : 0;
                ctrl->run[warp][lane] = rrn;
            }
            __syncwarp();
            OPS_TRACE(7);
            // eight rows at a time, loads first: the compiler cannot move a shared-memory load above
            // a store through a pointer it knows nothing about, and one row per round trip is slow
            for (int rr0 = 0; rr0 < 32; rr0 += 8) {
                Control::RowRun d[8];
                T vals[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) d[i] = ctrl->run[warp][rr0 + i];   // broadcast loads
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    vals[i] = reinterpret_cast<const T*>(my_stage + (rr0 + i) * kStagePitch)[lane];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (lane >= d[i].lo && lane < d[i].hi) reinterpret_cast<T*>(d[i].ptr)[lane] = vals[i];
            }
            __syncwarp();   // staging and run[] are rewritten in the next step
            OPS_TRACE(8);
        }
        OPS_TRACE(9);
        // padding slots, rows with one non-zero (a dot product by hand) and rows with none:
        // even rows by the h = 0 warp, odd rows by the h = 1 warp
        {
            const T* qg = reinterpret_cast<const T*>(p.q);
            const T* kg = reinterpret_cast<const T*>(p.kv);
            // most rows are full (nnz == trailing_dim, no padding): visit only the others
            const bool mine = (lane & 1) == h && u0 + q * 32 + lane < p.rows_v;
            unsigned todo = __ballot_sync(0xffffffffu, mine && (me.nnz < p.trailing_dim || me.nnz == 1));
            while (todo) {
                const int rr = __ffs(todo) - 1;
                todo &= todo - 1;
                const int u = u0 + q * 32 + rr;
                const int nnz = __shfl_sync(0xffffffffu, me.nnz, rr);
                const int start = __shfl_sync(0xffffffffu, me.start, rr);
                const int64_t real = (int64_t)u * p.stride + res;
                T* dst = out + (row0 + real) * p.trailing_dim;
                for (int j = nnz + lane; j < p.trailing_dim; j += 32) dst[j] = from_f<T>(0.f);
                if (nnz == 1) {
                    float acc = 0.f;
                    const T* qr = qg + (row0 + real) * D;
                    // K[bh][start][c]: rows of d elements, or column `start` of the (d, L) array
                    const int64_t k0 = p.kt_major ? row0 * D + start : (row0 + start) * D;
                    const int64_t kc = p.kt_major ? p.n_rows : 1;
                    for (int c = lane; c < D; c += 32) acc += to_f<T>(qr[c]) * to_f<T>(kg[k0 + c * kc]);
                    acc = warp_sum(acc);
                    if (lane == 0) dst[0] = from_f<T>(acc);
                }
            }
        }
        (void)ok;
        OPS_TRACE(10);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// SpMM
// ---------------------------------------------------------------------------------------------
template <int D> struct SpmmLayout {
    static constexpr int kSub = D / 64;
    static constexpr int kPBytes = kSubBytes;                     // 128 rows x 64 keys, 16 bit
    static constexpr int kItemBytes = kSub * kStepBytesPerSub;    // 64 keys of V
    static constexpr int kOBytes = kSub * kSubBytes;              // output staging
    static constexpr int kPOff = 0;                               // two P tiles ...
    static constexpr int kFront = 2 * kPBytes > kOBytes ? 2 * kPBytes : kOBytes;   // ... reused as O staging
    static constexpr int kRingOff = kFront;
    static constexpr int kCtrlOff = kRingOff + kStages * kItemBytes;
    static constexpr int kSmemBytes = kCtrlOff + (int)sizeof(Control) + 1024;
};

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 3)
spmm_band_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                 const Params p) {
    using L = SpmmLayout<D>;
    constexpr int kTmemCols = D < 32 ? 32 : D;   // the output accumulator
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* s_p = smem + L::kPOff;
    uint8_t* s_ring = smem + L::kRingOff;
    Control* ctrl = reinterpret_cast<Control*>(smem + L::kCtrlOff);
    volatile int32_t* status = p.status;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int res = blockIdx.y;
    const int64_t bh = blockIdx.z;
    const int u0 = blockIdx.x * kTile;

    if (warp == kMmaWarp) {
        tmem_alloc(&ctrl->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&ctrl->full[i], 1);
            mbar_init(&ctrl->empty[i], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctrl->ready[b], kRowWarps);
            mbar_init(&ctrl->freed[b], 1);
        }
        mbar_init(&ctrl->drain, 1);
        mbar_fence_init();
        ctrl->abort_at_entry = *status;
    }
    RowInfo me{0, 0, 0, 0};
    if (warp < kRowWarps) {
        me = load_row(p, u0 + (warp & 3) * 32 + lane, res);
        int lo = me.n > 0 ? me.a / kStep : INT_MAX;
        int hi = me.n > 0 ? (me.a + me.n + kStep - 1) / kStep : 0;
        lo = warp_min_i(lo);
        hi = warp_max_i(hi);
        if (lane == 0 && warp < 4) { ctrl->red_lo[warp] = lo; ctrl->red_hi[warp] = hi; }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;
    if (ctrl->abort_at_entry != 0) {
        if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
        return;
    }
    int klo = INT_MAX, khi = 0;
    for (int w = 0; w < 4; ++w) {
        klo = min(klo, ctrl->red_lo[w]);
        khi = max(khi, ctrl->red_hi[w]);
    }
    khi = min(khi, (p.rows_v + kStep - 1) / kStep);
    if (klo >= khi) { klo = 0; khi = 0; }
    const int steps = khi - klo;

    if (warp == kTmaWarp) {
        // ------------------------------------------------------------------ TMA producer (V)
        if (lane == 0 && steps > 0) {
            tma_prefetch_desc(&tm_v);
            int item = 0;
            bool ok = true;
            for (int k = klo; k < khi; ++k, ++item) {
                const int stage = item % kStages;
                const uint32_t parity = ((uint32_t)(item / kStages) & 1u) ^ 1u;
                if (!mbar_wait(&ctrl->empty[stage], parity, status, kErrEmpty)) { ok = false; break; }
                mbar_arrive_expect_tx(&ctrl->full[stage], L::kItemBytes);
                for (int sub = 0; sub < L::kSub; ++sub)
                    tma_load_4d(s_ring + stage * L::kItemBytes + sub * kStepBytesPerSub, &tm_v,
                                &ctrl->full[stage], sub * 64, res, k * kStep, (int)bh);
            }
            if (!ok)
                for (int i = max(0, item - kStages); i < item; ++i)
                    wait_quiet(&ctrl->full[i % kStages], (uint32_t)(i / kStages) & 1u);
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        // (whole warp on warp-uniform values, one elected lane issues)
        if (steps > 0) {
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t idesc = instr_desc_f16(fmt, kTile, D, 1);   // A K-major, B (V) MN-major
            const bool lead = elect_one();
            auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
                const bool r = mbar_wait(bar, parity, status, code);
                return __all_sync(0xffffffffu, r) != 0;
            };
            const uint32_t ring_addr = smem_u32(s_ring), p_base = smem_u32(s_p);
            bool ok = true;
            uint32_t ready_phase[2] = {0, 0};
            for (int k = klo; k < khi && ok; ++k) {
                const int item = k - klo, b = k & 1;
                ok = wait_all(&ctrl->full[item % kStages], (uint32_t)(item / kStages) & 1u, kErrFull);
                if (ok) ok = wait_all(&ctrl->ready[b], ready_phase[b], kErrReady);
                if (!ok) break;
                ready_phase[b] ^= 1u;
                tc_fence_after_sync();
                const uint32_t a_base = p_base + b * L::kPBytes;
                const uint32_t b_base = ring_addr + (item % kStages) * L::kItemBytes;
#pragma unroll
                for (int kk = 0; kk < kStep / 16; ++kk) {
                    const uint64_t da = smem_desc_sw128(a_base + kk * 32, 16, 1024);
                    const uint64_t db = smem_desc_sw128(b_base + kk * 2048, kStepBytesPerSub, 1024);
                    if (lead) mma_ss(tmem_base, da, db, idesc, (k > klo || kk > 0) ? 1u : 0u);
                }
                if (lead) {
                    mma_commit(&ctrl->empty[item % kStages]);
                    mma_commit(&ctrl->freed[b]);
                }
            }
            if (lead) mma_commit(&ctrl->drain);   // every MMA complete: O final, P tiles free for the staging
            wait_quiet(&ctrl->drain, 0);
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------------ P loaders + epilogue
        // Warp (q, h): the loader of rows 32q + 16h .. + 15 (all 64 columns of a step), and in the
        // epilogue the 32-column chunks ch with ch mod 2 == h of rows 32q .. 32q+31.
        const int q = warp & 3, h = warp >> 2;
        const T* pin = reinterpret_cast<const T*>(p.sparse);
        const int64_t row0 = bh * p.n_rows;
        uint32_t free_phase[2] = {0, 0};
        bool ok = true;
        for (int k = klo; k < khi; ++k) {
            const int b = k & 1;
            if (k - klo >= 2) {   // the MMAs that read this tile two steps ago are complete
                ok = mbar_wait(&ctrl->freed[b], free_phase[b], status, kErrFree);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                free_phase[b] ^= 1u;
            }
            uint8_t* tile = s_p + b * L::kPBytes;
            const int c0 = k * kStep;
            {   // this lane's row: source of column c0 and the valid columns of the step
                const int64_t real = (int64_t)(u0 + q * 32 + lane) * p.stride + res;
                Control::RowRun rrn;
                rrn.ptr = reinterpret_cast<unsigned long long>(pin + (row0 + real) * p.trailing_dim + (c0 - me.a));
                rrn.lo = me.n > 0 ? max(me.a - c0, 0) : 0;
                rrn.hi = me.n > 0 ? min(me.a + me.n - c0, kStep) : 0;
                __syncwarp();   // the previous step's reads of run[] are done
                ctrl->run[warp][lane] = rrn;
            }
            __syncwarp();
            // eight rows at a time: all their loads are issued before the first store
            for (int rr0 = h * 16; rr0 < h * 16 + 16; rr0 += 8) {
                T vals[8][2];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const Control::RowRun rrn = ctrl->run[warp][rr0 + i];   // broadcast load
                    const T* src = reinterpret_cast<const T*>(rrn.ptr);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int e = lane + 32 * j;
                        vals[i][j] = (e >= rrn.lo && e < rrn.hi) ? src[e] : from_f<T>(0.f);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = q * 32 + rr0 + i;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int e = lane + 32 * j;
                        // 128-byte-swizzled K-major tile: 16-byte chunk index XOR row mod 8
                        *reinterpret_cast<T*>(tile + r * 128 + ((((e >> 3) ^ (r & 7))) << 4) + (e & 7) * 2) = vals[i][j];
                    }
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->ready[b]);
        }
        const bool have_o = ok && steps > 0;
        if (have_o) {
            ok = mbar_wait(&ctrl->drain, 0, status, kErrReady);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after_sync();
        }
        // epilogue: O for band rows, P[i,0] * V[start] for single-element rows, zero otherwise,
        // staged in the (now free) P tiles in the swizzled layout, one TMA store per 64 columns
        const uint32_t o_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const int t = q * 32 + lane;
        const int64_t real = (int64_t)(u0 + t) * p.stride + res;
        const T* vrow = reinterpret_cast<const T*>(p.kv) + (row0 + me.start) * D;
        float p0 = 0.f;
        if (me.nnz == 1) p0 = to_f<T>(pin[(row0 + real) * p.trailing_dim]);
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
            const int ch = 2 * c + h;   // this warp's 32-column chunks
            if (have_o && ok) {
                tmem_ld32(o_addr + ch * 32, r);
                tmem_ld_wait();
            }
            uint4 outv[4];
            uint32_t* o32 = reinterpret_cast<uint32_t*>(outv);
            if (me.nnz > 1 && have_o && ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 2)
                    o32[j >> 1] = pack2<T>(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            } else if (me.nnz == 1) {
#pragma unroll
                for (int j = 0; j < 32; j += 2)
                    o32[j >> 1] = pack2<T>(p0 * to_f<T>(vrow[ch * 32 + j]), p0 * to_f<T>(vrow[ch * 32 + j + 1]));
            } else {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) outv[q4] = make_uint4(0, 0, 0, 0);
            }
            uint8_t* srow = smem + (ch >> 1) * kSubBytes + t * 128;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
                *reinterpret_cast<uint4*>(srow + ((((ch & 1) * 4 + q4) ^ (t & 7)) << 4)) = outv[q4];
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight row warps, unconditionally
        if (threadIdx.x == 0) {
            for (int sub = 0; sub < L::kSub; ++sub)
                tma_store_4d(&tm_o, smem + sub * kSubBytes, sub * 64, res, u0, (int)bh);
            tma_store_commit();
            tma_store_wait_read();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
template <typename T, int D>
static int32_t launch_sddmm(const CUtensorMap& mq, const CUtensorMap& mk, const Params& prm, int64_t bh,
                            cudaStream_t st) {
    using L = SddmmLayout<D>;
    auto kern = sddmm_band_kernel<T, D>;
    if (!allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kSmemBytes)) return SPLAT_ERR_LAUNCH;
    dim3 grid((unsigned)((prm.rows_v + kTile - 1) / kTile), (unsigned)prm.stride, (unsigned)bh);
    kern<<<grid, kThreads, L::kSmemBytes, st>>>(mq, mk, prm);
    return launch_status();
}
template <typename T, int D>
static int32_t launch_spmm(const CUtensorMap& mv, const CUtensorMap& mo, const Params& prm, int64_t bh,
                           cudaStream_t st) {
    using L = SpmmLayout<D>;
    auto kern = spmm_band_kernel<T, D>;
    if (!allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kSmemBytes)) return SPLAT_ERR_LAUNCH;
    dim3 grid((unsigned)((prm.rows_v + kTile - 1) / kTile), (unsigned)prm.stride, (unsigned)bh);
    kern<<<grid, kThreads, L::kSmemBytes, st>>>(mv, mo, prm);
    return launch_status();
}

#ifdef SPLAT_OPS_TRACE
static long long* g_trace = nullptr;
#endif
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Checks shared by both operators; fills stride.  plan as written by splat_acsr_classify:
// {max_nnz, stride_min, stride_max, misaligned, n_single, max_col+1, n_empty, n_multi}
static int32_t band_applies(const int32_t* plan, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                            int64_t trailing_dim, int32_t dtype, int64_t* stride_out) {
    if (bh < 0 || n_rows < 0 || trailing_dim < 0) return SPLAT_ERR_BAD_ARG;
    if (bh == 0 || n_rows == 0 || trailing_dim == 0) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (dtype != SPLAT_F16 && dtype != SPLAT_BF16) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (d != 64 && d != 128) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (n_rows != n_cols) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    const int64_t stride = plan[7] > 0 ? plan[1] : 1;
    if (plan[7] > 0 && plan[1] != plan[2]) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (plan[3] != 0 || stride < 1 || stride > 65535 || n_rows % stride != 0)
        return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (plan[5] > n_cols || plan[0] > trailing_dim || bh > 65535 || n_rows > INT32_MAX ||
        trailing_dim > INT32_MAX)
        return SPLAT_ERR_UNSUPPORTED_SHAPE;
    *stride_out = stride;
    return SPLAT_OK;
}

}  // namespace ops
}  // namespace band
}  // namespace splat

using namespace splat;
using namespace splat::band;

extern "C" int32_t splat_sddmm_band(const void* q, const void* k, int64_t k_stride_bh, int64_t k_stride_col,
                                    int64_t k_stride_k, void* s_out, const float* sTod_lin,
                                    const float* sTod_tr, const float* nnzs, int64_t bh, int64_t n_rows,
                                    int64_t n_cols, int64_t d, int64_t trailing_dim, int32_t dtype,
                                    const int32_t* plan_i32, int32_t* status_word, void* stream) {
    if (!plan_i32) return SPLAT_ERR_BAD_ARG;
    int64_t stride = 1;
    const int32_t rc = ops::band_applies(plan_i32, bh, n_rows, n_cols, d, trailing_dim, dtype, &stride);
    if (rc != SPLAT_OK) return rc;
    if (!q || !k || !s_out || !sTod_lin || !sTod_tr || !nnzs || !status_word) return SPLAT_ERR_BAD_ARG;
    const bool k_major = k_stride_k == 1 && k_stride_col == d && k_stride_bh == n_cols * d;
    const bool kt_major = k_stride_col == 1 && k_stride_k == n_cols && k_stride_bh == n_cols * d;
    if (!k_major && !(kt_major && stride == 1 && n_cols % 8 == 0)) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (!ops::aligned16(q) || !ops::aligned16(k)) return SPLAT_ERR_MISALIGNED;
    CUtensorMap mq, mk;
    if (!make_map(&mq, q, dtype, bh, n_rows, d, stride, ops::kTile) ||
        !(k_major ? make_map(&mk, k, dtype, bh, n_rows, d, stride, ops::kStep)
                  : make_map_kt(&mk, k, dtype, bh, n_cols, d)))
        return SPLAT_ERR_DRIVER;
    ops::Params prm;
    prm.kt_major = k_major ? 0 : 1;
#ifdef SPLAT_OPS_TRACE
    prm.trace = ops::g_trace;
#endif
    prm.lin = sTod_lin; prm.tr = sTod_tr; prm.nnzs = nnzs; prm.q = q; prm.kv = k; prm.sparse = s_out;
    prm.status = status_word; prm.n_rows = n_rows; prm.rows_v = (int)(n_rows / stride);
    prm.stride = (int)stride; prm.trailing_dim = (int)trailing_dim;
    prm.direct = ops::aligned16(s_out) ? 1 : 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SPLAT_BF16)
        return d == 128 ? ops::launch_sddmm<__nv_bfloat16, 128>(mq, mk, prm, bh, st)
                        : ops::launch_sddmm<__nv_bfloat16, 64>(mq, mk, prm, bh, st);
    return d == 128 ? ops::launch_sddmm<__half, 128>(mq, mk, prm, bh, st)
                    : ops::launch_sddmm<__half, 64>(mq, mk, prm, bh, st);
}

extern "C" int32_t splat_spmm_band(const void* p, const void* v, void* o, const float* sTod_lin,
                                   const float* sTod_tr, const float* nnzs, int64_t bh, int64_t n_rows,
                                   int64_t n_cols, int64_t d, int64_t trailing_dim, int32_t dtype,
                                   const int32_t* plan_i32, int32_t* status_word, void* stream) {
    if (!plan_i32) return SPLAT_ERR_BAD_ARG;
    int64_t stride = 1;
    const int32_t rc = ops::band_applies(plan_i32, bh, n_rows, n_cols, d, trailing_dim, dtype, &stride);
    if (rc != SPLAT_OK) return rc;
    if (!p || !v || !o || !sTod_lin || !sTod_tr || !nnzs || !status_word) return SPLAT_ERR_BAD_ARG;
    if (!ops::aligned16(v) || !ops::aligned16(o)) return SPLAT_ERR_MISALIGNED;
    CUtensorMap mv, mo;
    if (!make_map(&mv, v, dtype, bh, n_rows, d, stride, ops::kStep) ||
        !make_map(&mo, o, dtype, bh, n_rows, d, stride, ops::kTile))
        return SPLAT_ERR_DRIVER;
    ops::Params prm;
#ifdef SPLAT_OPS_TRACE
    prm.trace = nullptr;
#endif
    prm.lin = sTod_lin; prm.tr = sTod_tr; prm.nnzs = nnzs; prm.q = nullptr; prm.kv = v;
    prm.sparse = const_cast<void*>(p);
    prm.status = status_word; prm.n_rows = n_rows; prm.rows_v = (int)(n_rows / stride);
    prm.stride = (int)stride; prm.trailing_dim = (int)trailing_dim;
    prm.direct = 0;
    prm.kt_major = 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SPLAT_BF16)
        return d == 128 ? ops::launch_spmm<__nv_bfloat16, 128>(mv, mo, prm, bh, st)
                        : ops::launch_spmm<__nv_bfloat16, 64>(mv, mo, prm, bh, st);
    return d == 128 ? ops::launch_spmm<__half, 128>(mv, mo, prm, bh, st)
                    : ops::launch_spmm<__half, 64>(mv, mo, prm, bh, st);
}

#ifdef SPLAT_OPS_TRACE
extern "C" void splat_debug_set_ops_trace(void* device_buffer_2x256_i64) {
    splat::band::ops::g_trace = reinterpret_cast<long long*>(device_buffer_2x256_i64);
}
#endif
