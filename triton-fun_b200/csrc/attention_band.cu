// Fused SDDMM -> softmax -> SpMM for ACSR patterns whose rows are contiguous bands after
// regrouping by residue class: TMA-staged tiles, tcgen05 tensor-core MMAs with the scores and the
// output accumulator in tensor memory, online softmax in registers.  16-bit inputs, d = 64 or 128.
//
// Regrouping.  If every row with more than one non-zero has the same stride s and start_i == i
// (mod s), the rows of residue class r = i mod s only ever touch columns of the same class.  With
// u = (i - r)/s and v = (col - r)/s the class is an ordinary stride-1 band problem of L/s rows in
// (u, v) coordinates, and its Q/K/V rows are reached by a tensor map over the view
// (d, s, L/s, BH) of the (BH, L, d) array: box (64, 1, 128, 1) at (chunk, r, u0, bh).
// s = 1 is the plain sliding-window case.
//
// One CTA owns two 128-row Q tiles (A, B) of one (bh, r) and walks the union of their key ranges in
// 128-key steps.  Warps: 0-3 softmax/epilogue for tile A, 4-7 for tile B (thread = row = TMEM
// lane), 8 = TMA producer, 9 = MMA issuer and TMEM owner.  Per key tile n and Q tile X:
//     S_X = Q_X K_n^T        tcgen05.mma, operands in shared memory (128B swizzle, K-major)
//     P_X = exp2(S_X*c - m)   softmax warps: tcgen05.ld, band mask, running max with a lazy O
//                             rescale, P written back over S in tensor memory
//     O_X += P_X V_n          tcgen05.mma, A from tensor memory, B = V tile (MN-major)
// The MMA warp issues [PV_A(n), S_A(n+1)], [PV_B(n), S_B(n+1)] so one tile's MMAs overlap the other
// tile's softmax.  Rows with exactly one non-zero are described by the metadata as column `start`
// whatever their class, so they are excluded from the band and written as O[i] = V[start_i];
// rows with no non-zero are written as zero.
#include <limits.h>
#include <type_traits>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace splat {
namespace band {

using namespace tc;

constexpr int kTile = 128;          // rows per Q tile and keys per K/V tile
constexpr int kSubBytes = kTile * 128;  // one 64-element (128-byte) column chunk of a tile
constexpr int kThreads = 384;          // warps 10, 11 only complete the third warpgroup
constexpr int kRegsSoftmax = 224;       // per-thread register budgets after the re-split below
constexpr int kRegsOther = 48;
constexpr int kTmaWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kTmemCols = 512;
constexpr int kMaxStages = 4;
constexpr float kRescaleThreshold = 8.0f;  // log2 domain: P stays below 2^8 between rescales

// status-word codes (which wait gave up)
enum : int { kErrQ = 1, kErrKvFull = 2, kErrKvEmpty = 3, kErrSReady = 4, kErrPReady = 5 };

// Optional device-side timeline (profiling builds only, -DSPLAT_BAND_TRACE): one CTA records
// (tag, SM clock) pairs per role into a caller-supplied buffer.
#ifdef SPLAT_BAND_TRACE
#define SPLAT_TRACE(role, tag)                                                          \
    do {                                                                                \
        if (trace_on && lane == 0 && trace_n[role] < 1024)                              \
            p.trace[(role) * 1024 + trace_n[role]++] = ((long long)(tag) << 48) | (clock64() & 0xffffffffffffLL); \
    } while (0)
#else
#define SPLAT_TRACE(role, tag) do { } while (0)
#endif

struct Params {
#ifdef SPLAT_BAND_TRACE
    long long* trace;
#endif
    const float* lin;
    const float* tr;
    const float* nnzs;
    const void* v;
    void* o;
    int32_t* status;
    int64_t n_rows;    // L
    int rows_v;        // L / stride: rows of one residue class
    int stride;
    float scale_log2;  // softmax scale * log2(e), > 0
};

struct Control {
    uint64_t q_full;
    uint64_t kv_full[kMaxStages];
    uint64_t kv_empty[kMaxStages];
    uint64_t s_ready[2];
    uint64_t p_ready[2];
    uint64_t drain;
    uint32_t tmem_base;
    int32_t abort_at_entry;
    int32_t red_lo[8];
    int32_t red_hi[8];
};

template <int D> struct Layout {
    static constexpr int kSub = D / 64;
    static constexpr int kTileBytes = kSub * kSubBytes;
    static constexpr int kStages = 4;
    static constexpr int kQOff = 0;
    static constexpr int kRingOff = 2 * kTileBytes;
    static constexpr int kCtrlOff = kRingOff + kStages * kTileBytes;
    static constexpr int kSmemBytes = kCtrlOff + (int)sizeof(Control) + 1024;  // + alignment slack
};

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
// packed fp32x2 arithmetic (one issue slot for two lanes of work)
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

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Wait that ignores the status word (used only while leaving after an error).
__device__ __forceinline__ void mbar_wait_quiet(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > 200000000LL) break;
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 1)
attention_band_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const Params p) {
    using L = Layout<D>;
    constexpr int kStages = L::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* s_q = smem + L::kQOff;
    uint8_t* s_ring = smem + L::kRingOff;
    Control* ctrl = reinterpret_cast<Control*>(smem + L::kCtrlOff);
    volatile int32_t* status = p.status;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef SPLAT_BAND_TRACE
    const bool trace_on = p.trace != nullptr && blockIdx.x == gridDim.x / 2 && blockIdx.y == 0 &&
                          blockIdx.z == gridDim.z / 2;
    int trace_n[4] = {0, 0, 0, 0};
#endif
    const int pair = blockIdx.x, res = blockIdx.y;
    const int64_t bh = blockIdx.z;
    const int u0 = pair * 2 * kTile;

    if (threadIdx.x == 0) {
        ctrl->abort_at_entry = *status;
        mbar_init(&ctrl->q_full, 1);
        for (int i = 0; i < kMaxStages; ++i) {
            mbar_init(&ctrl->kv_full[i], 1);
            mbar_init(&ctrl->kv_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ctrl->s_ready[i], 1);
            mbar_init(&ctrl->p_ready[i], 4);    // one arrival per softmax warp
        }
        mbar_init(&ctrl->drain, 1);
        mbar_fence_init();
    }

    // Per-row metadata in class coordinates (softmax threads only).
    int my_a = 0, my_n = 0, row_nnz = 0, row_start = 0;
    int64_t row_real = -1;
    if (warp < 8) {
        const int x = warp >> 2;
        const int u = u0 + x * kTile + (warp & 3) * 32 + lane;
        int lo = INT_MAX, hi = 0;
        if (u < p.rows_v) {
            row_real = (int64_t)u * p.stride + res;
            const RowAffine ra = row_affine(p.lin, p.tr, p.nnzs, row_real);
            row_nnz = ra.nnz;
            row_start = ra.start;
            if (ra.nnz > 1) {
                my_a = (ra.start - res) / p.stride;
                my_n = ra.nnz;
                lo = my_a / kTile;
                hi = (my_a + my_n + kTile - 1) / kTile;
            }
        }
        lo = warp_min_i(lo);
        hi = warp_max_i(hi);
        if (lane == 0) { ctrl->red_lo[warp] = lo; ctrl->red_hi[warp] = hi; }
    }
    __syncthreads();
    if (ctrl->abort_at_entry != 0) return;  // an earlier CTA gave up: do nothing

    if (warp == kMmaWarp) {
        tmem_alloc(&ctrl->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;

    // Key-tile ranges [lo, hi) of the two Q tiles and their union.
    int rlo[2], rhi[2];
    const int max_tiles = (p.rows_v + kTile - 1) / kTile;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        int lo = INT_MAX, hi = 0;
        for (int w = 0; w < 4; ++w) {
            lo = min(lo, ctrl->red_lo[x * 4 + w]);
            hi = max(hi, ctrl->red_hi[x * 4 + w]);
        }
        hi = min(hi, max_tiles);
        if (lo >= hi) { lo = 0; hi = 0; }
        rlo[x] = lo; rhi[x] = hi;
    }
    const bool has_a = rhi[0] > rlo[0], has_b = rhi[1] > rlo[1];
    const int n_lo = has_a ? (has_b ? min(rlo[0], rlo[1]) : rlo[0]) : rlo[1];
    const int n_hi = max(rhi[0], rhi[1]);
    auto in_range = [&](int x, int n) { return n >= rlo[x] && n < rhi[x]; };

    // The register file is re-split per role below (setmaxnreg): the eight softmax warps keep a
    // whole 128-column score row in registers, the producer / issuer warps need very little.
    if (warp == kTmaWarp) {
        // ------------------------------------------------------------------ TMA producer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (lane == 0 && n_hi > n_lo) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            const uint32_t q_bytes = (uint32_t)((has_a ? 1 : 0) + (has_b ? 1 : 0)) * L::kTileBytes;
            mbar_arrive_expect_tx(&ctrl->q_full, q_bytes);
            for (int x = 0; x < 2; ++x) {
                if (!(x == 0 ? has_a : has_b)) continue;
                for (int sub = 0; sub < L::kSub; ++sub)
                    tma_load_4d(s_q + x * L::kTileBytes + sub * kSubBytes, &tm_q, &ctrl->q_full,
                                sub * 64, res, u0 + x * kTile, (int)bh);
            }
            int item = 0;
            bool ok = true;
            for (int n = n_lo; n < n_hi && ok; ++n) {
                for (int which = 0; which < 2; ++which, ++item) {
                    const int stage = item % kStages;
                    const uint32_t parity = ((uint32_t)(item / kStages) & 1u) ^ 1u;
                    if (!mbar_wait(&ctrl->kv_empty[stage], parity, status, kErrKvEmpty)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&ctrl->kv_full[stage], L::kTileBytes);
                    const CUtensorMap* tm = which == 0 ? &tm_k : &tm_v;
                    for (int sub = 0; sub < L::kSub; ++sub)
                        tma_load_4d(s_ring + stage * L::kTileBytes + sub * kSubBytes, tm,
                                    &ctrl->kv_full[stage], sub * 64, res, n * kTile, (int)bh);
                }
            }
            if (!ok) {
                // leave only after the copies already issued have landed
                mbar_wait_quiet(&ctrl->q_full, 0);
                for (int i = max(0, item - kStages); i < item; ++i)
                    mbar_wait_quiet(&ctrl->kv_full[i % kStages], (uint32_t)(i / kStages) & 1u);
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (lane == 0 && n_hi > n_lo) {
            constexpr uint32_t fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t idesc_qk = instr_desc_f16(fmt, kTile, kTile, 0);
            constexpr uint32_t idesc_pv = instr_desc_f16(fmt, kTile, D, 1);
            const uint32_t q_addr = smem_u32(s_q), ring_addr = smem_u32(s_ring);

            auto issue_s = [&](int x, int stage) {
                const uint32_t a_base = q_addr + x * L::kTileBytes;
                const uint32_t b_base = ring_addr + stage * L::kTileBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kSubBytes + (kk & 3) * 32;
                    mma_ss(tmem_base + x * kTile, smem_desc_sw128(a_base + off, 16, 1024),
                           smem_desc_sw128(b_base + off, 16, 1024), idesc_qk, kk > 0);
                }
            };
            auto issue_pv = [&](int x, int stage, bool acc) {
                const uint32_t d_tmem = tmem_base + 2 * kTile + x * D;
                const uint32_t b_base = ring_addr + stage * L::kTileBytes;
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk) {
                    const uint64_t b_desc = smem_desc_sw128(b_base + kk * 2048, kSubBytes, 1024);
                    const uint32_t accumulate = (acc || kk > 0) ? 1u : 0u;
                    mma_ts(d_tmem, tmem_base + x * kTile + kk * 8, b_desc, idesc_pv, accumulate);
                }
            };
            auto full_wait = [&](int item) {
                return mbar_wait(&ctrl->kv_full[item % kStages], (uint32_t)(item / kStages) & 1u,
                                 status, kErrKvFull);
            };

            bool ok = mbar_wait(&ctrl->q_full, 0, status, kErrQ);
            uint32_t p_phase[2] = {0, 0};
            ok = ok && full_wait(0);
            if (ok) {
                tc_fence_after_sync();
                for (int x = 0; x < 2; ++x)
                    if (in_range(x, n_lo)) {
                        issue_s(x, 0);
                        mma_commit(&ctrl->s_ready[x]);
                    }
                mma_commit(&ctrl->kv_empty[0]);
            }
            for (int n = n_lo; n < n_hi && ok; ++n) {
                const int item_v = 2 * (n - n_lo) + 1, item_k = item_v + 1;
                const bool has_next = n + 1 < n_hi;
                ok = full_wait(item_v);
                if (ok && has_next) ok = full_wait(item_k);
                if (!ok) break;
                tc_fence_after_sync();
                for (int x = 0; x < 2 && ok; ++x) {
                    const bool cur = in_range(x, n), nxt = has_next && in_range(x, n + 1);
                    if (cur) {
                        SPLAT_TRACE(2, 10 + x);
                        ok = mbar_wait(&ctrl->p_ready[x], p_phase[x], status, kErrPReady);
                        if (!ok) break;
                        p_phase[x] ^= 1u;
                        tc_fence_after_sync();
                        SPLAT_TRACE(2, 12 + x);
                        issue_pv(x, item_v % kStages, n > rlo[x]);
                    }
                    if (nxt) issue_s(x, item_k % kStages);
                    SPLAT_TRACE(2, 14 + x);
                    // next scores ready -- or, after the last PV of this tile, its output final
                    if (cur || nxt) mma_commit(&ctrl->s_ready[x]);
                }
                if (!ok) break;
                mma_commit(&ctrl->kv_empty[item_v % kStages]);
                if (has_next) mma_commit(&ctrl->kv_empty[item_k % kStages]);
            }
            if (!ok) {
                // let the tensor pipe drain before tensor memory is released
                mma_commit(&ctrl->drain);
                mbar_wait_quiet(&ctrl->drain, 0);
            }
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ softmax + epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        const int x = warp >> 2;
        const int t = (warp & 3) * 32 + lane;  // row in tile == TMEM lane
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_addr + x * kTile;
        const uint32_t o_addr = lane_addr + 2 * kTile + x * D;
        float m_used = -INFINITY, l_sum = 0.f;
        uint32_t s_phase = 0;
        bool ok = true;
        const float sc = p.scale_log2;
        for (int n = rlo[x]; n < rhi[x]; ++n) {
            if ((warp & 3) == 0) SPLAT_TRACE(x, 1);
            ok = mbar_wait(&ctrl->s_ready[x], s_phase, status, kErrSReady);
            ok = __all_sync(0xffffffffu, ok);  // keep the warp together for the aligned tcgen05 ops
            if (!ok) break;
            s_phase ^= 1u;
            tc_fence_after_sync();
            if ((warp & 3) == 0) SPLAT_TRACE(x, 2);
            const int c0 = n * kTile;
            const int v_lo = my_a - c0;               // valid columns of this tile: [v_lo, v_hi)
            const int v_hi = my_n > 0 ? my_a + my_n - c0 : INT_MIN;
            const bool warp_full = __all_sync(0xffffffffu, v_lo <= 0 && v_hi >= kTile);

            // the whole score row of this thread, one wait for the four loads
            uint32_t r[kTile];
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) tmem_ld32(s_addr + ch * 32, r + ch * 32);
            tmem_ld_wait();
            if ((warp & 3) == 0) SPLAT_TRACE(x, 3);
            if (!warp_full) {   // band edge: columns outside [v_lo, v_hi) become -inf (exp2 -> 0)
#pragma unroll
                for (int j = 0; j < kTile; ++j)
                    r[j] = (j >= v_lo && j < v_hi) ? r[j] : 0xff800000u;
            }
            // row maximum, four independent chains of 3-input max
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < kTile; j += 8) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    mx[c] = fmax3(mx[c], __uint_as_float(r[j + 2 * c]), __uint_as_float(r[j + 2 * c + 1]));
            }
            const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            if ((warp & 3) == 0) SPLAT_TRACE(x, 4);
            const float m_new = fmaxf(m_used, mt * sc);
            const bool need = (m_new - m_used) > kRescaleThreshold;  // false when both are -inf
            const float corr = need ? ex2(m_used - m_new) : 1.f;
            if (need) m_used = m_new;
            l_sum *= corr;
            const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;

            // probabilities: exp2(s*c - m) with packed fp32x2 FMAs, row sum, 16-bit pack in place
            const float2 sc2 = make_float2(sc, sc), nm2 = make_float2(-m_eff, -m_eff);
            float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kTile; j += 4) {
                float2 a0 = fma2(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), sc2, nm2);
                float2 a1 = fma2(make_float2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), sc2, nm2);
                a0.x = ex2(a0.x); a0.y = ex2(a0.y); a1.x = ex2(a1.x); a1.y = ex2(a1.y);
                acc0 = add2(acc0, a0);
                acc1 = add2(acc1, a1);
                r[j >> 1] = pack2<T>(a0.x, a0.y);
                r[(j >> 1) + 1] = pack2<T>(a1.x, a1.y);
            }
            l_sum += (acc0.x + acc0.y) + (acc1.x + acc1.y);
            if ((warp & 3) == 0) SPLAT_TRACE(x, 5);
            tmem_st32(s_addr, r);            // P (64 packed columns) over the first half of S
            tmem_st32(s_addr + 32, r + 32);
            // lazy rescale of the accumulator (rare): only when some row's maximum moved by > 2^8
            if (__any_sync(0xffffffffu, need) && n > rlo[x]) {
                uint32_t o[32];
#pragma unroll
                for (int ch = 0; ch < D / 32; ++ch) {
                    tmem_ld32(o_addr + ch * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
                    tmem_st32(o_addr + ch * 32, o);
                }
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->p_ready[x]);
            if ((warp & 3) == 0) SPLAT_TRACE(x, 6);
        }
        uint32_t r[32];
        const bool have_o = ok && rhi[x] > rlo[x];
        if (have_o) {
            ok = mbar_wait(&ctrl->s_ready[x], s_phase, status, kErrSReady);  // last PV finished
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after_sync();
        }
        // epilogue: O / l for band rows, V[start] for single-element rows, zero otherwise
        T* orow = row_real >= 0 ? reinterpret_cast<T*>(p.o) + (bh * p.n_rows + row_real) * D : nullptr;
        const T* vrow = reinterpret_cast<const T*>(p.v) + (bh * p.n_rows + (int64_t)row_start) * D;
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
            if (have_o && ok) {  // warp-uniform
                tmem_ld32(o_addr + ch * 32, r);
                tmem_ld_wait();
            }
            if (orow == nullptr) continue;
            uint4 out[4];
            if (row_nnz > 1 && have_o && ok) {
                uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
#pragma unroll
                for (int j = 0; j < 32; j += 2)
                    o32[j >> 1] = pack2<T>(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
            } else if (row_nnz == 1) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    out[q4] = *reinterpret_cast<const uint4*>(vrow + ch * 32 + q4 * 8);
            } else {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) out[q4] = make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
                *reinterpret_cast<uint4*>(orow + ch * 32 + q4 * 8) = out[q4];
        }
    } else {
        // warps 10, 11: idle members of the third warpgroup
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
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
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) !=
                cudaSuccess || q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

// (BH, L, d) 16-bit array viewed as (d, stride, L/stride, BH); box (64, 1, 128, 1), 128B swizzle.
static bool make_map(CUtensorMap* map, const void* base, int32_t dtype, int64_t bh, int64_t n_rows,
                     int64_t d, int64_t stride) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)stride, (cuuint64_t)(n_rows / stride),
                                (cuuint64_t)bh};
    const cuuint64_t strides[3] = {(cuuint64_t)(d * 2), (cuuint64_t)(stride * d * 2),
                                   (cuuint64_t)(n_rows * d * 2)};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)kTile, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult rc = fn(map, dtype == SPLAT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

#ifdef SPLAT_BAND_TRACE
static long long* g_trace = nullptr;
#endif

template <typename T, int D>
static int32_t launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                      const Params& prm, int64_t bh, cudaStream_t st) {
    using L = Layout<D>;
    auto kern = attention_band_kernel<T, D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes) !=
        cudaSuccess)
        return SPLAT_ERR_LAUNCH;
    const int pairs = (prm.rows_v + 2 * kTile - 1) / (2 * kTile);
    dim3 grid((unsigned)pairs, (unsigned)prm.stride, (unsigned)bh);
    kern<<<grid, kThreads, L::kSmemBytes, st>>>(mq, mk, mv, prm);
    return launch_status();
}

template <typename T>
static int32_t launch_d(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                        const Params& prm, int64_t bh, int64_t d, cudaStream_t st) {
    return d == 128 ? launch<T, 128>(mq, mk, mv, prm, bh, st) : launch<T, 64>(mq, mk, mv, prm, bh, st);
}

}  // namespace band

int32_t attention_band(const void* q, const void* k, int64_t ksb, int64_t ksc, int64_t ksk,
                       const void* v, void* o, const float* lin, const float* tr,
                       const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                       float scale, int32_t dtype, const int32_t* plan, int32_t* status_word,
                       cudaStream_t st) {
    if (!q || !k || !v || !o || !lin || !tr || !nnzs || !plan || !status_word || bh < 0 ||
        n_rows < 0)
        return SPLAT_ERR_BAD_ARG;
    if (dtype != SPLAT_F16 && dtype != SPLAT_BF16) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (d != 64 && d != 128) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (!(scale > 0.f)) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (n_rows != n_cols || n_rows == 0 || bh == 0) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (ksk != 1 || ksc != d || ksb != n_cols * d) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    // plan: {max_nnz, stride_min, stride_max, misaligned, n_single, max_col+1, n_empty, n_multi}
    const int64_t stride = plan[7] > 0 ? plan[1] : 1;
    if (plan[7] > 0 && plan[1] != plan[2]) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (plan[3] != 0 || stride < 1 || stride > 65535 || n_rows % stride != 0)
        return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (plan[5] > n_cols || bh > 65535 || n_rows > INT32_MAX) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return SPLAT_ERR_MISALIGNED;

    CUtensorMap mq, mk, mv;
    if (!band::make_map(&mq, q, dtype, bh, n_rows, d, stride) ||
        !band::make_map(&mk, k, dtype, bh, n_rows, d, stride) ||
        !band::make_map(&mv, v, dtype, bh, n_rows, d, stride))
        return SPLAT_ERR_DRIVER;
    band::Params prm;
    prm.lin = lin; prm.tr = tr; prm.nnzs = nnzs; prm.v = v; prm.o = o; prm.status = status_word;
    prm.n_rows = n_rows; prm.rows_v = (int)(n_rows / stride); prm.stride = (int)stride;
    prm.scale_log2 = scale * kLog2e;
#ifdef SPLAT_BAND_TRACE
    prm.trace = band::g_trace;
#endif
    if (dtype == SPLAT_BF16) return band::launch_d<__nv_bfloat16>(mq, mk, mv, prm, bh, d, st);
    return band::launch_d<__half>(mq, mk, mv, prm, bh, d, st);
}

}  // namespace splat

#ifdef SPLAT_BAND_TRACE
extern "C" void splat_debug_set_trace(void* device_buffer_4x1024_i64) {
    splat::band::g_trace = reinterpret_cast<long long*>(device_buffer_4x1024_i64);
}
#endif
