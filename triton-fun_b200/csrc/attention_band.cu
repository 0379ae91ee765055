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
// One CTA owns two 128-row Q tiles (A, B) of one (bh, r).  K/V travel through a shared-memory ring
// in 128-key tiles (TMA, 128-byte swizzle); the math advances in 64-key steps k so that the 128
// score columns a Q tile owns in tensor memory form TWO buffers:
//     S_X(k)  = Q_X K(k)^T     tcgen05.mma 128x64x16, operands in shared memory, into buffer k mod 2
//     P_X(k)  = exp2(S c - m)   softmax warps: tcgen05.ld the 64 scores of their row, band mask,
//                               running max with a lazy rescale of O, exp2 with the scale folded
//                               in, 16-bit P stored over the consumed scores of the same buffer
//     O_X    += P_X(k) V(k)     tcgen05.mma 128xdx16, A = P from tensor memory, B = V rows (MN-major)
// While the softmax warps work on buffer k mod 2 the tensor core already fills the other buffer
// with S_X(k+1), so neither side waits for the other in steady state: per Q tile the issue order is
// S(k0), S(k0+1), then for every k: PV(k), S(k+2).
// Warps: 0-3 softmax/epilogue of tile A, 4-7 of tile B (thread = row = TMEM lane), 8 = TMA producer,
// 9 / 10 = MMA issuers of tile A / B (9 also owns tensor memory), 11 idle.
// K operand layouts.  K-major: K rows of d contiguous elements (the transposed view of a (BH, L, d)
// array); ring tiles hold [keys][128 bytes of d] per 64-element chunk of d.  Key-major
// (Params::kt_major): the reference's own contiguous (BH, d, L) K^T; ring tiles then hold
// [d][128 bytes = 64 keys] per 64-key chunk, fetched through a tensor map over (L, d, BH), and the
// QK MMA takes B as an MN-major operand exactly as the PV MMA takes V.
// Rows with exactly one non-zero are described by the metadata as column `start` whatever their
// class, so they are excluded from the band and written as O[i] = V[start_i]; rows with no
// non-zero are written as zero.
#include <limits.h>
#include <stdlib.h>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace splat {
namespace band {

using namespace tc;

constexpr int kTile = 128;              // rows per Q tile and keys per K/V ring tile
constexpr int kStep = 64;               // keys per math step (one score buffer)
constexpr int kSubBytes = kTile * 128;  // one 64-element (128-byte) column chunk of a tile
constexpr int kThreads = 384;
constexpr int kTmaWarp = 8;
constexpr int kMmaWarp = 9;             // 9: tile A (+ TMEM alloc), 10: tile B
constexpr int kTmemCols = 512;
constexpr int kStages = 4;              // K/V ring, one 128-key tile per stage
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
    const void* q;     // raw operands: only the single score of a row with one non-zero is read through
    const void* k;     //   them (log-sum-exp output); everything else goes through the tensor maps
    float* lse;        // (BH, L) natural-log log-sum-exp of every row, or null
    int32_t* status;
    int64_t n_rows;    // L
    int rows_v;        // L / stride: rows of one residue class
    int stride;
    int kt_major;      // 1: K is given as a contiguous (BH, d, L) array (keys innermost); stride 1 only
    float scale_log2;  // softmax scale * log2(e), > 0
};

struct Control {
    uint64_t q_full;
    uint64_t kv_full[kStages];
    uint64_t kv_empty[kStages];  // two arrivals: both MMA issuers release every ring tile
    uint64_t s_ready[2][2];      // [Q tile][buffer] MMA -> softmax: scores ready / previous PV done
    uint64_t p_ready[2][2];      // [Q tile][buffer] softmax -> MMA: P stored (4 warp arrivals)
    uint64_t drain[2];
    uint32_t tmem_base;
    int32_t abort_at_entry;
    int32_t red_lo[8];
    int32_t red_hi[8];
};

template <int D> struct Layout {
    static constexpr int kSub = D / 64;
    static constexpr int kTileBytes = kSub * kSubBytes;
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

// Natural-log log-sum-exp of a row: from the running maximum and sum of a band row (log2 domain), the
// one score scale * q_i . k_start of a row with a single non-zero (computed here from the raw
// operands; such rows are outside the band), -inf for a row without non-zeros.
template <typename T, int D>
__device__ __forceinline__ float row_lse(const Params& p, int64_t bh, int64_t row_real, int row_nnz, int row_start,
                                         float m_used, float l_sum) {
    if (row_nnz > 1) return lse_from_log2(m_used, l_sum);
    if (row_nnz != 1) return -INFINITY;
    const T* qr = reinterpret_cast<const T*>(p.q) + (bh * p.n_rows + row_real) * D;
    const T* kb = reinterpret_cast<const T*>(p.k);
    // K[bh][start][c]: rows of d elements, or column `start` of the (d, L) array
    const float s = p.kt_major ? dot_strided<T>(qr, kb + bh * p.n_rows * D + row_start, p.n_rows, D)
                               : dot_strided<T>(qr, kb + (bh * p.n_rows + row_start) * D, 1, D);
    return s * p.scale_log2 * kLn2;
}

template <typename T, int D, bool kLse>
__global__ void __launch_bounds__(kThreads, 1)
attention_band_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                      const Params p) {
    using L = Layout<D>;
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

    // Prologue, one block-wide barrier: tensor-memory allocation (MMA warp), barrier initialisation
    // (thread 0) and the row metadata (softmax warps) proceed side by side.
    if (warp == kMmaWarp) {
        tmem_alloc(&ctrl->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    if (threadIdx.x == 0) {
        mbar_init(&ctrl->q_full, 1);
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&ctrl->kv_full[i], 1);
            mbar_init(&ctrl->kv_empty[i], 2);
        }
        for (int i = 0; i < 2; ++i) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(&ctrl->s_ready[i][b], 1);
                mbar_init(&ctrl->p_ready[i][b], 4);  // one arrival per softmax warp
            }
            mbar_init(&ctrl->drain[i], 1);
        }
        mbar_fence_init();
        ctrl->abort_at_entry = *status;
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
                lo = my_a / kStep;
                hi = (my_a + my_n + kStep - 1) / kStep;
            }
        }
        lo = warp_min_i(lo);
        hi = warp_max_i(hi);
        if (lane == 0) { ctrl->red_lo[warp] = lo; ctrl->red_hi[warp] = hi; }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;
    if (ctrl->abort_at_entry != 0) {   // an earlier CTA gave up: release tensor memory and leave
        if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
        return;
    }

    // Step ranges [klo, khi) (64-key units) of the two Q tiles and the ring-tile range of their union.
    int klo[2], khi[2];
    const int max_steps = (p.rows_v + kStep - 1) / kStep;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        int lo = INT_MAX, hi = 0;
        for (int w = 0; w < 4; ++w) {
            lo = min(lo, ctrl->red_lo[x * 4 + w]);
            hi = max(hi, ctrl->red_hi[x * 4 + w]);
        }
        hi = min(hi, max_steps);
        if (lo >= hi) { lo = 0; hi = 0; }
        klo[x] = lo; khi[x] = hi;
    }
    const bool has_a = khi[0] > klo[0], has_b = khi[1] > klo[1];
    const int k_min = has_a ? (has_b ? min(klo[0], klo[1]) : klo[0]) : klo[1];
    const int k_max = max(khi[0], khi[1]);
    const int n_lo = k_min >> 1, n_hi = (k_max + 1) >> 1;   // 128-key ring tiles [n_lo, n_hi)
    const bool any_work = k_max > k_min;

    if (warp == kTmaWarp) {
        // ------------------------------------------------------------------ TMA producer
        // Ring items in order K(n_lo), V(n_lo), K(n_lo+1), V(n_lo+1), ...
        if (lane == 0 && any_work) {
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
                    if (which == 0 && p.kt_major) {
                        for (int c = 0; c < kTile / 64; ++c)      // 64-key chunks of [d][64 keys]
                            tma_load_4d(s_ring + stage * L::kTileBytes + c * (D * 128), tm,
                                        &ctrl->kv_full[stage], n * kTile + c * 64, 0, (int)bh, 0);
                        continue;
                    }
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
    } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
        // ------------------------------------------------------------------ MMA issuer of tile x
        // Uses ring item 2(n - n_lo) = K tile n and 2(n - n_lo) + 1 = V tile n; every item is
        // waited for and released exactly once by each issuer, used or not.
        // The whole warp walks the loop on warp-uniform values and one elected lane issues: a
        // single lane in a divergent branch needs about twice the tensor pipe's time per MMA just
        // to get the instruction out.
        const int x = warp - kMmaWarp;
        if (any_work) {
            const bool lead = elect_one();
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            const uint32_t idesc_qk = instr_desc_f16(fmt, kTile, kStep, p.kt_major ? 1u : 0u);
            constexpr uint32_t idesc_pv = instr_desc_f16(fmt, kTile, D, 1);
            const uint32_t ring_addr = smem_u32(s_ring);
            const uint32_t q_base = smem_u32(s_q) + x * L::kTileBytes;
            const uint32_t s_tmem = tmem_base + x * kTile;
            const uint32_t o_tmem = tmem_base + 2 * kTile + x * D;
            const int lo = klo[x], hi = khi[x];
            bool ok = true;

            auto stage_of = [&](int item) { return item % kStages; };
            auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
                const bool r = mbar_wait(bar, parity, status, code);
                return __all_sync(0xffffffffu, r) != 0;
            };
            auto full_wait = [&](int item) {
                return wait_all(&ctrl->kv_full[stage_of(item)], (uint32_t)(item / kStages) & 1u, kErrKvFull);
            };
            auto commit = [&](uint64_t* bar) { if (lead) mma_commit(bar); };
            auto release = [&](int item) { commit(&ctrl->kv_empty[stage_of(item)]); };
            // S(k): 64 keys = rows [64(k&1), +64) of K tile k/2, into score buffer k&1
            auto issue_s = [&](int k) {
                const uint32_t t_base = ring_addr + stage_of(2 * ((k >> 1) - n_lo)) * L::kTileBytes;
                // K-major: key rows [64 (k&1), +64) of each d chunk; key-major: chunk k&1 of [d][64 keys]
                const uint32_t b_base = t_base + (k & 1) * (p.kt_major ? D * 128 : kStep * 128);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kSubBytes + (kk & 3) * 32;
                    const uint64_t da = smem_desc_sw128(q_base + off, 16, 1024);
                    const uint64_t db = p.kt_major ? smem_desc_sw128(b_base + kk * 2048, D * 128, 1024)
                                                   : smem_desc_sw128(b_base + off, 16, 1024);
                    if (lead) mma_ss(s_tmem + (k & 1) * kStep, da, db, idesc_qk, kk > 0);
                }
            };
            // O += P(k) V(k): P packed in the first 32 columns of buffer k&1, V rows [64(k&1), +64)
            auto issue_pv = [&](int k, bool acc) {
                const uint32_t b_base = ring_addr + stage_of(2 * ((k >> 1) - n_lo) + 1) * L::kTileBytes +
                                        (k & 1) * (kStep * 128);
#pragma unroll
                for (int kk = 0; kk < kStep / 16; ++kk) {
                    const uint64_t db = smem_desc_sw128(b_base + kk * 2048, kSubBytes, 1024);
                    if (lead) mma_ts(o_tmem, s_tmem + (k & 1) * kStep + kk * 8, db, idesc_pv,
                                     (acc || kk > 0) ? 1u : 0u);
                }
            };
            // last step of tile x that reads ring tile n
            auto last_user = [&](int k) { return (k & 1) == 1 || k == hi - 1; };

            ok = wait_all(&ctrl->q_full, 0, kErrQ);
            if (hi > lo) {
                const int t_lo = lo >> 1, t_hi = (hi + 1) >> 1;   // ring tiles tile x reads
                // tiles before the range: pass them on untouched
                for (int n = n_lo; n < t_lo && ok; ++n)
                    for (int w = 0; w < 2 && ok; ++w) {
                        ok = full_wait(2 * (n - n_lo) + w);
                        if (ok) release(2 * (n - n_lo) + w);
                    }
                // first two score buffers
                for (int k = lo; k < min(lo + 2, hi) && ok; ++k) {
                    const int item_k = 2 * ((k >> 1) - n_lo);
                    if (k == lo || (k & 1) == 0) ok = full_wait(item_k);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_s(k);
                    commit(&ctrl->s_ready[x][k & 1]);
                    if (last_user(k)) release(item_k);
                }
                uint32_t p_phase[2] = {0, 0};
                for (int k = lo; k < hi && ok; ++k) {
                    const int item_v = 2 * ((k >> 1) - n_lo) + 1;
                    if (k == lo || (k & 1) == 0) ok = full_wait(item_v);
                    if (!ok) break;
                    SPLAT_TRACE(2 + x, 10);
                    ok = wait_all(&ctrl->p_ready[x][k & 1], p_phase[k & 1], kErrPReady);
                    if (!ok) break;
                    p_phase[k & 1] ^= 1u;
                    tc_fence_after_sync();
                    SPLAT_TRACE(2 + x, 11);
                    issue_pv(k, k > lo);
                    if (last_user(k)) release(item_v);
                    if (k + 2 < hi) {
                        const int item_k = 2 * (((k + 2) >> 1) - n_lo);
                        if (((k + 2) & 1) == 0) ok = full_wait(item_k);   // first reader of that K tile
                        if (!ok) break;
                        tc_fence_after_sync();
                        issue_s(k + 2);
                        if (last_user(k + 2)) release(item_k);
                    }
                    // buffer k&1: next scores ready -- and, in any case, PV(k) complete
                    commit(&ctrl->s_ready[x][k & 1]);
                    SPLAT_TRACE(2 + x, 12);
                }
                // tiles after the range
                for (int n = t_hi; n < n_hi && ok; ++n)
                    for (int w = 0; w < 2 && ok; ++w) {
                        ok = full_wait(2 * (n - n_lo) + w);
                        if (ok) release(2 * (n - n_lo) + w);
                    }
            } else {
                for (int item = 0; item < 2 * (n_hi - n_lo) && ok; ++item) {
                    ok = full_wait(item);
                    if (ok) release(item);
                }
            }
            if (!ok) {
                // let the tensor pipe drain before tensor memory is released
                commit(&ctrl->drain[x]);
                mbar_wait_quiet(&ctrl->drain[x], 0);
            }
            __syncwarp();
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ softmax + epilogue
        const int x = warp >> 2;
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_addr + x * kTile;
        const uint32_t o_addr = lane_addr + 2 * kTile + x * D;
        float m_used = -INFINITY, l_sum = 0.f;
        uint32_t s_phase[2] = {0, 0};
        bool pv_waited = false;   // the "PV(k-1) done" phase of the other buffer was consumed early
        bool ok = true;
        const float sc = p.scale_log2;
        const float2 sc2 = make_float2(sc, sc);
        const bool tr = (warp & 3) == 0;
        (void)tr;
        for (int k = klo[x]; k < khi[x]; ++k) {
            const int b = k & 1;
            if (tr) SPLAT_TRACE(x, 1);
            if (!pv_waited) {
                ok = mbar_wait(&ctrl->s_ready[x][b], s_phase[b], status, kErrSReady);
                ok = __all_sync(0xffffffffu, ok);  // keep the warp together for the aligned tcgen05 ops
                if (!ok) break;
                s_phase[b] ^= 1u;
            }
            pv_waited = false;
            tc_fence_after_sync();
            if (tr) SPLAT_TRACE(x, 2);
            const int c0 = k * kStep;
            const int v_lo = my_a - c0;               // valid columns of this step: [v_lo, v_hi)
            const int v_hi = my_n > 0 ? my_a + my_n - c0 : INT_MIN;
            const bool edge = !__all_sync(0xffffffffu, v_lo <= 0 && v_hi >= kStep);

            uint32_t r[kStep];
            tmem_ld32(s_addr + b * kStep, r);
            tmem_ld32(s_addr + b * kStep + 32, r + 32);
            tmem_ld_wait();
            if (tr) SPLAT_TRACE(x, 3);
            if (edge) {   // band edge: columns outside [v_lo, v_hi) become -inf (exp2 -> 0)
#pragma unroll
                for (int j = 0; j < kStep; ++j)
                    r[j] = (j >= v_lo && j < v_hi) ? r[j] : 0xff800000u;
            }
            // row maximum, four independent chains of 3-input max
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < kStep; j += 8) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    mx[c] = fmax3(mx[c], __uint_as_float(r[j + 2 * c]), __uint_as_float(r[j + 2 * c + 1]));
            }
            const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const float m_new = fmaxf(m_used, mt * sc);
            const bool need = (m_new - m_used) > kRescaleThreshold;  // false when both are -inf
            const float corr = need ? ex2(m_used - m_new) : 1.f;
            if (need) m_used = m_new;
            l_sum *= corr;
            const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
            if (tr) SPLAT_TRACE(x, 4);

            // lazy rescale of the accumulator (rare): some row's maximum moved by more than 2^8.
            // PV(k-1) may still be running: its completion is the next arrival on the OTHER
            // buffer's barrier, which is consumed here instead of at the top of step k+1.
            if (k > klo[x] && __any_sync(0xffffffffu, need)) {
                ok = mbar_wait(&ctrl->s_ready[x][b ^ 1], s_phase[b ^ 1], status, kErrSReady);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                s_phase[b ^ 1] ^= 1u;
                pv_waited = true;
                tc_fence_after_sync();
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

            // probabilities: exp2(s*c - m) with packed fp32x2 FMAs, row sum, 16-bit pack in place
            const float2 nm2 = make_float2(-m_eff, -m_eff);
            float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kStep; j += 4) {
                float2 a0 = fma2(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), sc2, nm2);
                float2 a1 = fma2(make_float2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), sc2, nm2);
                a0.x = ex2(a0.x); a0.y = ex2(a0.y); a1.x = ex2(a1.x); a1.y = ex2(a1.y);
                acc0 = add2(acc0, a0);
                acc1 = add2(acc1, a1);
                r[j >> 1] = pack2<T>(a0.x, a0.y);
                r[(j >> 1) + 1] = pack2<T>(a1.x, a1.y);
            }
            l_sum += (acc0.x + acc0.y) + (acc1.x + acc1.y);
            tmem_st32(s_addr + b * kStep, r);   // P: 32 packed columns over the consumed scores
            if (tr) SPLAT_TRACE(x, 5);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->p_ready[x][b]);
            if (tr) SPLAT_TRACE(x, 6);
        }
        const int steps = khi[x] - klo[x];
        const bool have_o = ok && steps > 0;
        if (have_o) {
            // the last PV on each buffer that was used
            for (int i = min(steps, 2); i >= 1 && ok; --i) {
                const int b = (khi[x] - i) & 1;
                if (pv_waited && i == 2) continue;   // already consumed by a late rescale
                ok = mbar_wait(&ctrl->s_ready[x][b], s_phase[b], status, kErrSReady);
                ok = __all_sync(0xffffffffu, ok);
            }
            tc_fence_after_sync();
        }
        // epilogue: O / l for band rows, V[start] for single-element rows, zero otherwise.  Rows are
        // staged in the tile's Q buffer (free: every MMA of the tile has completed) in the
        // 128-byte-swizzled layout and leave through one tiled TMA store per 64-column half (rows
        // past the end of the class are clipped by the tensor map).
        uint32_t r[32];
        const int t = (warp & 3) * 32 + lane;
        uint8_t* s_o = s_q + x * L::kTileBytes;
        const T* vrow = reinterpret_cast<const T*>(p.v) + (bh * p.n_rows + (int64_t)row_start) * D;
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
        if (kLse && row_real >= 0 && ok)   // (the instantiation without this output is the default)
            p.lse[bh * p.n_rows + row_real] = row_lse<T, D>(p, bh, row_real, row_nnz, row_start, m_used, l_sum);
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
            if (have_o && ok) {  // warp-uniform
                tmem_ld32(o_addr + ch * 32, r);
                tmem_ld_wait();
            }
            uint4 out[4];
            if (row_nnz > 1 && have_o && ok) {
                uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
#pragma unroll
                for (int j = 0; j < 32; j += 2)
                    o32[j >> 1] = pack2<T>(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
            } else if (row_nnz == 1 && row_real >= 0) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    out[q4] = *reinterpret_cast<const uint4*>(vrow + ch * 32 + q4 * 8);
            } else {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) out[q4] = make_uint4(0, 0, 0, 0);
            }
            uint8_t* srow = s_o + (ch >> 1) * kSubBytes + t * 128;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
                *reinterpret_cast<uint4*>(srow + ((((ch & 1) * 4 + q4) ^ (t & 7)) << 4)) = out[q4];
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync %0, 128;" ::"r"(1 + x) : "memory");   // the tile's four softmax warps
        if ((warp & 3) == 0 && lane == 0 && u0 + x * kTile < p.rows_v) {
            for (int sub = 0; sub < L::kSub; ++sub)
                tma_store_4d(&tm_o, s_o + sub * kSubBytes, sub * 64, res, u0 + x * kTile, (int)bh);
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
// Single-tile variant: one 128-row Q tile per CTA, 192 threads, 256 tensor-memory columns and
// ~97 KB of shared memory, so TWO CTAs share an SM and one CTA's prologue / epilogue / waits are
// covered by the other's work.  K and V travel in 64-key ring items (one math step each).  Each Q
// tile loads its own K/V, i.e. twice the L2 -> shared-memory traffic of the paired kernel above:
// used for problems whose classes have a single row tile or too few tile pairs to fill the GPU.
// Warps: 0-3 softmax/epilogue, 4 = TMA producer, 5 = MMA issuer and tensor-memory owner.
// ---------------------------------------------------------------------------------------------
constexpr int kThreads1 = 192;
constexpr int kTmemCols1 = 256;
constexpr int kStepBytesPerSub = kStep * 128;   // 64 keys x 128 bytes

struct Control1 {
    uint64_t q_full;
    uint64_t kv_full[kStages];
    uint64_t kv_empty[kStages];
    uint64_t s_ready[2];
    uint64_t p_ready[2];
    uint64_t drain;
    uint32_t tmem_base;
    int32_t abort_at_entry;
    int32_t red_lo[4];
    int32_t red_hi[4];
};

template <int D> struct Layout1 {
    static constexpr int kSub = D / 64;
    static constexpr int kQBytes = kSub * kSubBytes;              // 128 rows
    static constexpr int kItemBytes = kSub * kStepBytesPerSub;    // 64 keys
    static constexpr int kRingOff = kQBytes;
    static constexpr int kCtrlOff = kRingOff + kStages * kItemBytes;
    static constexpr int kSmemBytes = kCtrlOff + (int)sizeof(Control1) + 1024;
};

template <typename T, int D, bool kLse>
__global__ void __launch_bounds__(kThreads1, 2)
attention_band1_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                       const Params p) {
    using L = Layout1<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* s_q = smem;
    uint8_t* s_ring = smem + L::kRingOff;
    Control1* ctrl = reinterpret_cast<Control1*>(smem + L::kCtrlOff);
    volatile int32_t* status = p.status;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int res = blockIdx.y;
    const int64_t bh = blockIdx.z;
    const int u0 = blockIdx.x * kTile;

    // Prologue, one block-wide barrier: tensor-memory allocation (warp 5), barrier initialisation
    // (thread 0) and the row metadata (softmax warps) proceed side by side.
    if (warp == 5) {
        tmem_alloc(&ctrl->tmem_base, kTmemCols1);
        tmem_relinquish();
    }
    if (threadIdx.x == 0) {
        mbar_init(&ctrl->q_full, 1);
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&ctrl->kv_full[i], 1);
            mbar_init(&ctrl->kv_empty[i], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctrl->s_ready[b], 1);
            mbar_init(&ctrl->p_ready[b], 4);
        }
        mbar_init(&ctrl->drain, 1);
        mbar_fence_init();
        ctrl->abort_at_entry = *status;
    }
    int my_a = 0, my_n = 0, row_nnz = 0, row_start = 0;
    int64_t row_real = -1;
    if (warp < 4) {
        const int u = u0 + warp * 32 + lane;
        int lo = INT_MAX, hi = 0;
        if (u < p.rows_v) {
            row_real = (int64_t)u * p.stride + res;
            const RowAffine ra = row_affine(p.lin, p.tr, p.nnzs, row_real);
            row_nnz = ra.nnz;
            row_start = ra.start;
            if (ra.nnz > 1) {
                my_a = (ra.start - res) / p.stride;
                my_n = ra.nnz;
                lo = my_a / kStep;
                hi = (my_a + my_n + kStep - 1) / kStep;
            }
        }
        lo = warp_min_i(lo);
        hi = warp_max_i(hi);
        if (lane == 0) { ctrl->red_lo[warp] = lo; ctrl->red_hi[warp] = hi; }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;
    if (ctrl->abort_at_entry != 0) {   // an earlier CTA gave up: release tensor memory and leave
        if (warp == 5) tmem_dealloc(tmem_base, kTmemCols1);
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

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && steps > 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            mbar_arrive_expect_tx(&ctrl->q_full, L::kQBytes);
            for (int sub = 0; sub < L::kSub; ++sub)
                tma_load_4d(s_q + sub * kSubBytes, &tm_q, &ctrl->q_full, sub * 64, res, u0, (int)bh);
            int item = 0;
            bool ok = true;
            for (int k = klo; k < khi && ok; ++k) {
                for (int which = 0; which < 2; ++which, ++item) {   // K(k) then V(k)
                    const int stage = item % kStages;
                    const uint32_t parity = ((uint32_t)(item / kStages) & 1u) ^ 1u;
                    if (!mbar_wait(&ctrl->kv_empty[stage], parity, status, kErrKvEmpty)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&ctrl->kv_full[stage], L::kItemBytes);
                    const CUtensorMap* tm = which == 0 ? &tm_k : &tm_v;
                    if (which == 0 && p.kt_major) {       // one [d][64 keys] block
                        tma_load_4d(s_ring + stage * L::kItemBytes, tm, &ctrl->kv_full[stage], k * kStep, 0,
                                    (int)bh, 0);
                        continue;
                    }
                    for (int sub = 0; sub < L::kSub; ++sub)
                        tma_load_4d(s_ring + stage * L::kItemBytes + sub * kStepBytesPerSub, tm,
                                    &ctrl->kv_full[stage], sub * 64, res, k * kStep, (int)bh);
                }
            }
            if (!ok) {
                mbar_wait_quiet(&ctrl->q_full, 0);
                for (int i = max(0, item - kStages); i < item; ++i)
                    mbar_wait_quiet(&ctrl->kv_full[i % kStages], (uint32_t)(i / kStages) & 1u);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        // ring item 2(k - klo) = K(k), 2(k - klo) + 1 = V(k); order S(klo), S(klo+1), then per k:
        // PV(k), S(k+2)
        // (whole warp on warp-uniform values, one elected lane issues: see the paired kernel)
        if (steps > 0) {
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            const uint32_t idesc_qk = instr_desc_f16(fmt, kTile, kStep, p.kt_major ? 1u : 0u);
            constexpr uint32_t idesc_pv = instr_desc_f16(fmt, kTile, D, 1);
            const bool lead = elect_one();
            const uint32_t ring_addr = smem_u32(s_ring), q_base = smem_u32(s_q);
            const uint32_t o_tmem = tmem_base + 2 * kStep;
            auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
                const bool r = mbar_wait(bar, parity, status, code);
                return __all_sync(0xffffffffu, r) != 0;
            };
            auto commit = [&](uint64_t* bar) { if (lead) mma_commit(bar); };
            auto full_wait = [&](int item) {
                return wait_all(&ctrl->kv_full[item % kStages], (uint32_t)(item / kStages) & 1u, kErrKvFull);
            };
            auto issue_s = [&](int k) {
                const uint32_t b_base = ring_addr + ((2 * (k - klo)) % kStages) * L::kItemBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t da = smem_desc_sw128(q_base + (kk >> 2) * kSubBytes + (kk & 3) * 32, 16, 1024);
                    const uint64_t db = p.kt_major
                        ? smem_desc_sw128(b_base + kk * 2048, D * 128, 1024)
                        : smem_desc_sw128(b_base + (kk >> 2) * kStepBytesPerSub + (kk & 3) * 32, 16, 1024);
                    if (lead) mma_ss(tmem_base + (k & 1) * kStep, da, db, idesc_qk, kk > 0);
                }
            };
            auto issue_pv = [&](int k, bool acc) {
                const uint32_t b_base = ring_addr + ((2 * (k - klo) + 1) % kStages) * L::kItemBytes;
#pragma unroll
                for (int kk = 0; kk < kStep / 16; ++kk) {
                    const uint64_t db = smem_desc_sw128(b_base + kk * 2048, kStepBytesPerSub, 1024);
                    if (lead) mma_ts(o_tmem, tmem_base + (k & 1) * kStep + kk * 8, db, idesc_pv,
                                     (acc || kk > 0) ? 1u : 0u);
                }
            };
            bool ok = wait_all(&ctrl->q_full, 0, kErrQ);
            for (int k = klo; k < min(klo + 2, khi) && ok; ++k) {
                ok = full_wait(2 * (k - klo));
                if (!ok) break;
                tc_fence_after_sync();
                issue_s(k);
                commit(&ctrl->s_ready[k & 1]);
                commit(&ctrl->kv_empty[(2 * (k - klo)) % kStages]);
            }
            uint32_t p_phase[2] = {0, 0};
            for (int k = klo; k < khi && ok; ++k) {
                const int item_v = 2 * (k - klo) + 1;
                ok = full_wait(item_v);
                if (!ok) break;
                ok = wait_all(&ctrl->p_ready[k & 1], p_phase[k & 1], kErrPReady);
                if (!ok) break;
                p_phase[k & 1] ^= 1u;
                tc_fence_after_sync();
                issue_pv(k, k > klo);
                commit(&ctrl->kv_empty[item_v % kStages]);
                if (k + 2 < khi) {
                    const int item_k = 2 * (k + 2 - klo);
                    ok = full_wait(item_k);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_s(k + 2);
                    commit(&ctrl->kv_empty[item_k % kStages]);
                }
                commit(&ctrl->s_ready[k & 1]);   // next scores ready, and PV(k) complete
            }
            if (!ok) {
                commit(&ctrl->drain);
                mbar_wait_quiet(&ctrl->drain, 0);
            }
            __syncwarp();
        }
    } else if (warp < 4) {
        // ------------------------------------------------------------------ softmax + epilogue
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        const uint32_t s_addr = lane_addr;
        const uint32_t o_addr = lane_addr + 2 * kStep;
        float m_used = -INFINITY, l_sum = 0.f;
        uint32_t s_phase[2] = {0, 0};
        bool pv_waited = false;
        bool ok = true;
        const float sc = p.scale_log2;
        const float2 sc2 = make_float2(sc, sc);
        for (int k = klo; k < khi; ++k) {
            const int b = k & 1;
            if (!pv_waited) {
                ok = mbar_wait(&ctrl->s_ready[b], s_phase[b], status, kErrSReady);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                s_phase[b] ^= 1u;
            }
            pv_waited = false;
            tc_fence_after_sync();
            const int c0 = k * kStep;
            const int v_lo = my_a - c0;
            const int v_hi = my_n > 0 ? my_a + my_n - c0 : INT_MIN;
            const bool edge = !__all_sync(0xffffffffu, v_lo <= 0 && v_hi >= kStep);
            uint32_t r[kStep];
            tmem_ld32(s_addr + b * kStep, r);
            tmem_ld32(s_addr + b * kStep + 32, r + 32);
            tmem_ld_wait();
            if (edge) {
#pragma unroll
                for (int j = 0; j < kStep; ++j)
                    r[j] = (j >= v_lo && j < v_hi) ? r[j] : 0xff800000u;
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < kStep; j += 8) {
#pragma unroll
                for (int cc = 0; cc < 4; ++cc)
                    mx[cc] = fmax3(mx[cc], __uint_as_float(r[j + 2 * cc]), __uint_as_float(r[j + 2 * cc + 1]));
            }
            const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const float m_new = fmaxf(m_used, mt * sc);
            const bool need = (m_new - m_used) > kRescaleThreshold;
            const float corr = need ? ex2(m_used - m_new) : 1.f;
            if (need) m_used = m_new;
            l_sum *= corr;
            const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
            if (k > klo && __any_sync(0xffffffffu, need)) {
                // PV(k-1) may still be running: its completion is the next arrival on the OTHER
                // buffer's barrier, consumed here instead of at the top of step k+1
                ok = mbar_wait(&ctrl->s_ready[b ^ 1], s_phase[b ^ 1], status, kErrSReady);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                s_phase[b ^ 1] ^= 1u;
                pv_waited = true;
                tc_fence_after_sync();
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
            const float2 nm2 = make_float2(-m_eff, -m_eff);
            float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kStep; j += 4) {
                float2 a0 = fma2(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), sc2, nm2);
                float2 a1 = fma2(make_float2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), sc2, nm2);
                a0.x = ex2(a0.x); a0.y = ex2(a0.y); a1.x = ex2(a1.x); a1.y = ex2(a1.y);
                acc0 = add2(acc0, a0);
                acc1 = add2(acc1, a1);
                r[j >> 1] = pack2<T>(a0.x, a0.y);
                r[(j >> 1) + 1] = pack2<T>(a1.x, a1.y);
            }
            l_sum += (acc0.x + acc0.y) + (acc1.x + acc1.y);
            tmem_st32(s_addr + b * kStep, r);   // P: 32 packed columns over the consumed scores
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->p_ready[b]);
        }
        const bool have_o = ok && steps > 0;
        if (have_o) {
            for (int i = min(steps, 2); i >= 1 && ok; --i) {
                const int b = (khi - i) & 1;
                if (pv_waited && i == 2) continue;
                ok = mbar_wait(&ctrl->s_ready[b], s_phase[b], status, kErrSReady);
                ok = __all_sync(0xffffffffu, ok);
            }
            tc_fence_after_sync();
        }
        // epilogue: O / l for band rows, V[start] for single-element rows, zero otherwise.  Rows are
        // staged in the Q buffer (free: every MMA has completed) in the 128-byte-swizzled tile
        // layout and leave through one tiled TMA store per 64-column half (rows past the end of
        // the class are clipped by the tensor map).
        uint32_t r[32];
        const int t = warp * 32 + lane;
        const T* vrow = reinterpret_cast<const T*>(p.v) + (bh * p.n_rows + (int64_t)row_start) * D;
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
        if (kLse && row_real >= 0 && ok)   // (the instantiation without this output is the default)
            p.lse[bh * p.n_rows + row_real] = row_lse<T, D>(p, bh, row_real, row_nnz, row_start, m_used, l_sum);
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
            if (have_o && ok) {
                tmem_ld32(o_addr + ch * 32, r);
                tmem_ld_wait();
            }
            uint4 out[4];
            if (row_nnz > 1 && have_o && ok) {
                uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
#pragma unroll
                for (int j = 0; j < 32; j += 2)
                    o32[j >> 1] = pack2<T>(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
            } else if (row_nnz == 1 && row_real >= 0) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    out[q4] = *reinterpret_cast<const uint4*>(vrow + ch * 32 + q4 * 8);
            } else {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) out[q4] = make_uint4(0, 0, 0, 0);
            }
            // columns [32 ch, 32 ch + 32) = 16-byte chunks 4 (ch & 1) .. +3 of 64-column half ch >> 1
            uint8_t* srow = s_q + (ch >> 1) * kSubBytes + t * 128;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
                *reinterpret_cast<uint4*>(srow + ((((ch & 1) * 4 + q4) ^ (t & 7)) << 4)) = out[q4];
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four softmax warps, unconditionally
        if (threadIdx.x == 0) {
            for (int sub = 0; sub < L::kSub; ++sub)
                tma_store_4d(&tm_o, s_q + sub * kSubBytes, sub * 64, res, u0, (int)bh);
            tma_store_commit();
            tma_store_wait_read();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols1);
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

// Encoded tensor maps of the last calls, so that a caller that launches with the same operands again
// (the module's forward, a benchmark loop) does not pay for four driver encodes per launch.  A map
// depends only on the values in the key, never on what the memory holds.
struct MapKey {
    const void* base;
    int64_t bh, rows, d, stride;
    int32_t dtype, box, kind;   // kind 0: (d, stride, L/stride, BH) view, 1: key-major (L, d, BH)
    bool operator==(const MapKey& o) const {
        return base == o.base && bh == o.bh && rows == o.rows && d == o.d && stride == o.stride &&
               dtype == o.dtype && box == o.box && kind == o.kind;
    }
};
constexpr int kMapCacheSlots = 32;
static std::mutex g_map_mutex;
static MapKey g_map_keys[kMapCacheSlots];
static CUtensorMap g_map_vals[kMapCacheSlots];
static int g_map_used = 0, g_map_next = 0;

static bool map_cache_get(const MapKey& key, CUtensorMap* map) {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    for (int i = 0; i < g_map_used; ++i)
        if (g_map_keys[i] == key) {
            *map = g_map_vals[i];
            return true;
        }
    return false;
}
static void map_cache_put(const MapKey& key, const CUtensorMap& map) {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    const int i = g_map_next;
    g_map_next = (g_map_next + 1) % kMapCacheSlots;
    if (g_map_used < kMapCacheSlots) ++g_map_used;
    g_map_keys[i] = key;
    g_map_vals[i] = map;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize once per kernel and device.
// (also used by the band SDDMM / SpMM kernels in ops_band.cu and by the pair kernel)
bool allow_dynamic_smem(const void* kernel, int bytes) {
    struct Seen { const void* kernel; int device; };
    static std::mutex mutex;
    static Seen seen[64];
    static int n_seen = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    std::lock_guard<std::mutex> lock(mutex);
    for (int i = 0; i < n_seen; ++i)
        if (seen[i].kernel == kernel && seen[i].device == dev) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
        return false;
    if (n_seen < 64) seen[n_seen++] = Seen{kernel, dev};
    return true;
}

// (BH, L, d) 16-bit array viewed as (d, stride, L/stride, BH); box (64, 1, box_rows, 1), 128B swizzle.
// (also used by the band SDDMM / SpMM kernels in ops_band.cu)
bool make_map(CUtensorMap* map, const void* base, int32_t dtype, int64_t bh, int64_t n_rows,
              int64_t d, int64_t stride, int box_rows = kTile) {
    const MapKey key{base, bh, n_rows, d, stride, dtype, box_rows, 0};
    if (map_cache_get(key, map)) return true;
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)stride, (cuuint64_t)(n_rows / stride),
                                (cuuint64_t)bh};
    const cuuint64_t strides[3] = {(cuuint64_t)(d * 2), (cuuint64_t)(stride * d * 2),
                                   (cuuint64_t)(n_rows * d * 2)};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult rc = fn(map, dtype == SPLAT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc == CUDA_SUCCESS) map_cache_put(key, *map);
    return rc == CUDA_SUCCESS;
}

// Contiguous (BH, d, L) K^T viewed as (L, d, BH, 1); box (64 keys, d, 1, 1), 128B swizzle: one
// [d][64 keys] block per copy.  (also used by the pair kernel and the band SDDMM)
bool make_map_kt(CUtensorMap* map, const void* base, int32_t dtype, int64_t bh, int64_t n_cols,
                 int64_t d) {
    const MapKey key{base, bh, n_cols, d, 1, dtype, 64, 1};
    if (map_cache_get(key, map)) return true;
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)n_cols, (cuuint64_t)d, (cuuint64_t)bh, 1};
    const cuuint64_t strides[3] = {(cuuint64_t)(n_cols * 2), (cuuint64_t)(d * n_cols * 2),
                                   (cuuint64_t)(bh * d * n_cols * 2)};
    const cuuint32_t box[4] = {64, (cuuint32_t)d, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult rc = fn(map, dtype == SPLAT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc == CUDA_SUCCESS) map_cache_put(key, *map);
    return rc == CUDA_SUCCESS;
}

#ifdef SPLAT_BAND_TRACE
static long long* g_trace = nullptr;
#endif

template <typename T, int D>
static int32_t launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                      const CUtensorMap& mo, const Params& prm, int64_t bh, cudaStream_t st) {
    using L = Layout<D>;
    auto kern = prm.lse != nullptr ? attention_band_kernel<T, D, true> : attention_band_kernel<T, D, false>;
    if (!allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kSmemBytes)) return SPLAT_ERR_LAUNCH;
    const int pairs = (prm.rows_v + 2 * kTile - 1) / (2 * kTile);
    dim3 grid((unsigned)pairs, (unsigned)prm.stride, (unsigned)bh);
    kern<<<grid, kThreads, L::kSmemBytes, st>>>(mq, mk, mv, mo, prm);
    return launch_status();
}

template <typename T, int D>
static int32_t launch1(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                       const CUtensorMap& mo, const Params& prm, int64_t bh, cudaStream_t st) {
    using L = Layout1<D>;
    auto kern = prm.lse != nullptr ? attention_band1_kernel<T, D, true> : attention_band1_kernel<T, D, false>;
    if (!allow_dynamic_smem(reinterpret_cast<const void*>(kern), L::kSmemBytes)) return SPLAT_ERR_LAUNCH;
    const int tiles = (prm.rows_v + kTile - 1) / kTile;
    dim3 grid((unsigned)tiles, (unsigned)prm.stride, (unsigned)bh);
    kern<<<grid, kThreads1, L::kSmemBytes, st>>>(mq, mk, mv, mo, prm);
    return launch_status();
}

template <typename T>
static int32_t launch1_d(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                         const CUtensorMap& mo, const Params& prm, int64_t bh, int64_t d, cudaStream_t st) {
    return d == 128 ? launch1<T, 128>(mq, mk, mv, mo, prm, bh, st)
                    : launch1<T, 64>(mq, mk, mv, mo, prm, bh, st);
}

template <typename T>
static int32_t launch_d(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                        const CUtensorMap& mo, const Params& prm, int64_t bh, int64_t d, cudaStream_t st) {
    return d == 128 ? launch<T, 128>(mq, mk, mv, mo, prm, bh, st)
                    : launch<T, 64>(mq, mk, mv, mo, prm, bh, st);
}

}  // namespace band

int32_t attention_pair(const void* q, const void* k, int kt_major, const void* v, void* o,
                       const float* lin, const float* tr, const float* nnzs, int64_t bh, int64_t n_rows,
                       int64_t stride, float scale, int32_t dtype, int32_t* status_word, int max_pairs,
                       float* lse, cudaStream_t st);

int32_t attention_band(const void* q, const void* k, int64_t ksb, int64_t ksc, int64_t ksk,
                       const void* v, void* o, const float* lin, const float* tr,
                       const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                       float scale, int32_t dtype, const int32_t* plan, int32_t* status_word,
                       float* lse, cudaStream_t st) {
    if (bh < 0 || n_rows < 0) return SPLAT_ERR_BAD_ARG;
    if (bh == 0 || n_rows == 0) return SPLAT_ERR_UNSUPPORTED_SHAPE;   // empty: left to the generic path
    if (!q || !k || !v || !o || !lin || !tr || !nnzs || !plan || !status_word)
        return SPLAT_ERR_BAD_ARG;
    if (dtype != SPLAT_F16 && dtype != SPLAT_BF16) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (d != 64 && d != 128) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (!(scale > 0.f)) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (n_rows != n_cols || n_rows == 0 || bh == 0) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    // K layouts the tensor-core kernels read: rows of d contiguous elements (the transposed view of a
    // (BH, L, d) array), or the reference's contiguous (BH, d, L) K^T (checked further down: only
    // for stride-1 patterns, and its row pitch L must be a multiple of 16 bytes)
    const bool k_major = ksk == 1 && ksc == d && ksb == n_cols * d;
    const bool kt_major = ksc == 1 && ksk == n_cols && ksb == n_cols * d;
    if (!k_major && !kt_major) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    // plan: {max_nnz, stride_min, stride_max, misaligned, n_single, max_col+1, n_empty, n_multi}
    const int64_t stride = plan[7] > 0 ? plan[1] : 1;
    if (plan[7] > 0 && plan[1] != plan[2]) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (plan[3] != 0 || stride < 1 || stride > 65535 || n_rows % stride != 0)
        return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (plan[5] > n_cols || bh > 65535 || n_rows > INT32_MAX) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (!k_major && (stride != 1 || n_cols % 8 != 0)) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return SPLAT_ERR_MISALIGNED;

    // Kernel choice.  1 (default): one Q tile per CTA, two CTAs per SM -- measured the fastest of the
    // three on every shape tried (5 % ahead of the two-tile kernel on 64 to 256 heads of
    // L = 32768, d = 128, window 1024; level with it on all 512, where both sit at the power cap;
    // 8 % ahead at d = 64).  2: two Q tiles per CTA sharing every K/V tile (half the L2 -> SM
    // traffic).  3: persistent CTA pairs (attention_pair.cu), d = 128 only.
    // SPLAT_B200_BAND_TILES=1|2|3 selects; SPLAT_B200_PAIR_MAX limits the resident pairs of 3.
    int variant = 1;
    if (const char* e = getenv("SPLAT_B200_BAND_TILES"))
        if (e[0] >= '1' && e[0] <= '3') variant = e[0] - '0';
    if (variant == 3 && d == 128) {
        int max_pairs = 0;
        if (const char* e = getenv("SPLAT_B200_PAIR_MAX")) max_pairs = atoi(e);
        const int32_t rc = attention_pair(q, k, kt_major ? 1 : 0, v, o, lin, tr, nnzs, bh, n_rows, stride,
                                          scale, dtype, status_word, max_pairs, lse, st);
        if (rc != SPLAT_ERR_UNSUPPORTED_SHAPE) return rc;
    }
    if (variant == 3) variant = 2;
    const bool single = variant == 1;
    const int kv_box = single ? band::kStep : band::kTile;
    CUtensorMap mq, mk, mv, mo;
    if (!band::make_map(&mq, q, dtype, bh, n_rows, d, stride) ||
        !(kt_major ? band::make_map_kt(&mk, k, dtype, bh, n_cols, d)
                   : band::make_map(&mk, k, dtype, bh, n_rows, d, stride, kv_box)) ||
        !band::make_map(&mv, v, dtype, bh, n_rows, d, stride, kv_box) ||
        !band::make_map(&mo, o, dtype, bh, n_rows, d, stride))
        return SPLAT_ERR_DRIVER;
    band::Params prm;
    prm.kt_major = kt_major ? 1 : 0;
    prm.lin = lin; prm.tr = tr; prm.nnzs = nnzs; prm.v = v; prm.o = o; prm.status = status_word;
    prm.q = q; prm.k = k; prm.lse = lse;
    prm.n_rows = n_rows; prm.rows_v = (int)(n_rows / stride); prm.stride = (int)stride;
    prm.scale_log2 = scale * kLog2e;
#ifdef SPLAT_BAND_TRACE
    prm.trace = band::g_trace;
#endif
    if (single) {
        if (dtype == SPLAT_BF16) return band::launch1_d<__nv_bfloat16>(mq, mk, mv, mo, prm, bh, d, st);
        return band::launch1_d<__half>(mq, mk, mv, mo, prm, bh, d, st);
    }
    if (dtype == SPLAT_BF16) return band::launch_d<__nv_bfloat16>(mq, mk, mv, mo, prm, bh, d, st);
    return band::launch_d<__half>(mq, mk, mv, mo, prm, bh, d, st);
}

}  // namespace splat

#ifdef SPLAT_BAND_TRACE
extern "C" void splat_debug_set_trace(void* device_buffer_4x1024_i64) {
    splat::band::g_trace = reinterpret_cast<long long*>(device_buffer_4x1024_i64);
}
#endif
