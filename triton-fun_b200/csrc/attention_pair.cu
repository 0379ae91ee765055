// Fused SDDMM -> softmax -> SpMM for band patterns (the condition of attention_band.cu) on CTA
// PAIRS: a cluster of two CTAs on two SMs runs one tcgen05 "cta_group::2" instruction stream.
// 16-bit inputs, d = 128.  Used for large problems; the kernels of attention_band.cu cover the rest.
//
// Work item = 256 consecutive class rows (u coordinates, see attention_band.cu for the regrouping
// by residue class) of one (batch*head, residue class): the even CTA of the pair owns rows
// [0, 128) of the item, the odd CTA rows [128, 256).  The kernel is persistent: pair c of C
// processes items c, c + C, c + 2C, ... in a fixed order, so neighbouring pairs work on
// neighbouring row blocks of the same head at the same time and share K/V in L2.
//
// An item with key range [128 n_lo, 128 n_hi) contributes N = n_hi - n_lo STEPS; the steps of all
// the items of a pair form one stream, numbered G = 0, 1, 2, ... across item boundaries.  Per step
// (both CTAs together, every MMA has M = 256: 128 rows per SM):
//     S(G) = Q K^T        8 x tcgen05.mma 256x128x16, A = each CTA's Q tile, B = the key tile: each
//                         CTA holds 64 of the 128 keys in its own shared memory
//     P(G) = exp2(S c - m) softmax warps of each CTA on their own 128 rows (thread = row): scores
//                         from tensor memory, band mask, running max with lazy rescale of O,
//                         16-bit P stored over the consumed scores
//     O  += P(G) V        8 x tcgen05.mma 256x128x16, A = P from each CTA's tensor memory,
//                         B = the value tile: each CTA holds 64 of the 128 value columns
// Each SM's 512 tensor-memory columns hold THREE score buffers (step G uses buffer G mod 3) and O,
// so the tensor core runs up to three steps ahead of the softmax warps, also into the next item:
// issue order S(0) S(1) S(2), then per step PV(G), S(G+3).  Operand halves are loaded by each CTA
// for itself with plain TMA loads (no multicast); the byte counts of both CTAs land on barriers of
// the even CTA, whose MMA thread is the only consumer.
//
// Progress of the tensor core is published as numbered EVENTS: event e is one tcgen05.commit per
// CTA onto barrier e mod 32 of that CTA.  Event G = "S(G) complete", event G + 3 = "PV(G)
// complete" (one commit after PV(G), S(G+3) serves both).  Softmax warps wait for S(G) and for the
// PV of their last step; the TMA producers wait for the event that frees the slot they are about
// to overwrite.  Every role walks the same item list with the per-item (n_lo, N) taken from a
// table in shared memory that each CTA builds from the row metadata at kernel start, so no role
// has to tell another what comes next.
//
// Warps per CTA: 0-3 softmax + epilogue, 4 TMA producer, 5 MMA issuer (even CTA) and tensor-memory
// owner (both).  Every mbarrier wait is bounded; a role that gives up records a code in the status
// word, the others see the word in their own waits, and both CTAs meet at a cluster barrier
// before tensor memory is released and either CTA leaves.
#include <limits.h>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "softmax_math.cuh"
#include "tc_ptx.cuh"

namespace splat {
namespace band {
bool make_map(CUtensorMap* map, const void* base, int32_t dtype, int64_t bh, int64_t n_rows,
              int64_t d, int64_t stride, int box_rows);
}

namespace pair {

using namespace tc;
using namespace sm;

constexpr int D = 128;
constexpr int kTile = 128;             // rows per CTA and keys per step
constexpr int kItemRows = 2 * kTile;   // rows per work item (CTA pair)
constexpr int kThreads = 192;
constexpr int kWarps = kThreads / 32;
constexpr int kTmaWarp = 4;
constexpr int kMmaWarp = 5;
constexpr int kTmemCols = 512;
constexpr int kBufs = 3;               // score buffers = K slots = V slots
constexpr int kEvents = 32;            // event barriers: a wait must be issued before its event is 32 events old
constexpr int kMaxEntries = 2048;      // (residue class, row block) combinations the range table holds
constexpr int kSubBytes = kTile * 128;         // 128 rows of one 64-element column chunk
constexpr int kTileBytes = 2 * kSubBytes;      // Q tile / O staging: 128 rows x 128 columns
constexpr int kSlotBytes = 16384;              // K half (64 keys x 128) or V half (128 keys x 64)
constexpr int kKHalfSub = 64 * 128;            // one 64-element chunk of a K half
constexpr uint32_t kOCol = 3 * kTile;          // tensor-memory column of O
constexpr float kRescaleThreshold = 8.0f;
#ifndef SPLAT_PAIR_POLY_PAIRS
#define SPLAT_PAIR_POLY_PAIRS 0
#endif
constexpr int kPolyPairs = SPLAT_PAIR_POLY_PAIRS;   // of every 4 pairs of exponentials, on the FMA pipes

// status-word codes (which wait gave up)
enum : int { kErrQ = 11, kErrKFull = 12, kErrVFull = 13, kErrEvent = 14, kErrPReady = 15,
             kErrOFree = 16, kErrStage = 17 };

struct Params {
    const float* lin;
    const float* tr;
    const float* nnzs;
    const void* v;
    int32_t* status;
    long long* trace;      // profiling builds only (else null)
    int64_t n_rows;        // L
    int rows_v;            // L / stride: rows of one residue class
    int stride;
    int items_per_class;   // ceil(rows_v / 256)
    int n_entries;         // stride * items_per_class <= kMaxEntries
    int64_t n_items;       // n_entries * bh
    float scale_log2;      // softmax scale * log2(e), > 0
};

struct Control {
    uint64_t ev[kEvents];      // both CTAs: tensor-core progress events
    uint64_t q_full[2];        // even CTA only (as the next four): Q tiles of both CTAs have landed
    uint64_t k_full[kBufs];
    uint64_t v_full[kBufs];
    uint64_t p_ready[kBufs];   // 8 arrivals: the softmax warps of both CTAs
    uint64_t o_free;           // 8 arrivals: O has been read out, the next item may overwrite it
    uint64_t drain;
    uint64_t stage_free;       // own CTA: the previous TMA store has read the output staging buffer
    uint64_t stage_ready;      // own CTA, 4 arrivals: the softmax warps have written their rows
    uint32_t tmem_base;
    int32_t abort_at_entry;
    uint32_t range[kMaxEntries];   // per (class, row block): n_lo | N << 16
};

struct Layout {
    static constexpr int kQOff = 0;                               // two Q tiles (items alternate)
    static constexpr int kStageOff = 2 * kTileBytes;              // output staging
    static constexpr int kKOff = kStageOff + kTileBytes;
    static constexpr int kVOff = kKOff + kBufs * kSlotBytes;
    static constexpr int kCtrlOff = kVOff + kBufs * kSlotBytes;
    static constexpr int kSmemBytes = kCtrlOff + (int)sizeof(Control) + 1024;   // + alignment slack
};

#ifdef SPLAT_PAIR_TRACE
#define PAIR_TRACE(role, tag)                                                                     \
    do {                                                                                          \
        if (trace_on && lane == 0 && (warp == 0 || warp >= 4) && trace_n < 2048)                   \
            p.trace[(role) * 2048 + trace_n++] = ((long long)(tag) << 48) | (clock64() & 0xffffffffffffLL); \
    } while (0)
#else
#define PAIR_TRACE(role, tag) do { } while (0)
#endif

// Row metadata -> band of the row in class coordinates: first column a, count n (0 unless the row
// has at least two non-zeros), plus the raw start column and count.  float32 products are exact
// here: the launcher admits n_rows <= 2^22 only.
__device__ __forceinline__ void row_band(const Params& p, int res, float lin, float tr, float nn,
                                         int& a, int& n, int& start, int& nnz) {
    const float s = fmaxf(rintf(lin), 1.f);
    start = (int)rintf(__fmul_rn(tr, s));
    nnz = max((int)rintf(nn), 0);
    a = 0; n = 0;
    if (nnz > 1) { a = (start - res) / p.stride; n = nnz; }
}

// Position in the stream of steps of this CTA pair.
struct Cursor {
    int64_t w;        // work item
    int64_t G;        // global step
    int i, N, n_lo;   // step within the item, steps of the item, first key tile of the item
    int jq;           // items with steps before this one
    int block, res;
    int64_t bh;
    bool valid;
};

__device__ __forceinline__ void spin_cycles(long long n) {
    const long long t0 = clock64();
    while (clock64() - t0 < n) { }
}

// r[0..127] scores -> r[0..63] packed 16-bit probabilities exp2(s*c - m); row sums into acc0/acc1.
// kPoly of every four pairs are evaluated on the FMA pipes, the rest on the special function unit.
template <typename T, int kPoly>
__device__ __forceinline__ void exp_rows(uint32_t* r, float2 sc2, float2 nm2, float2& acc0, float2& acc1) {
#pragma unroll
    for (int j = 0; j < kTile; j += 8) {
        float2 a[4];
#pragma unroll
        for (int c = 0; c < 4; ++c)
            a[c] = fma2(make_float2(__uint_as_float(r[j + 2 * c]), __uint_as_float(r[j + 2 * c + 1])), sc2, nm2);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (c < kPoly) a[c] = ex2_poly2(a[c]);
            else { a[c].x = ex2(a[c].x); a[c].y = ex2(a[c].y); }
        }
        acc0 = add2(acc0, add2(a[0], a[1]));
        acc1 = add2(acc1, add2(a[2], a[3]));
#pragma unroll
        for (int c = 0; c < 4; ++c) r[(j >> 1) + c] = pack2<T>(a[c].x, a[c].y);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
attention_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                      const Params p) {
    using L = Layout;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* s_q = smem + L::kQOff;
    uint8_t* s_stage = smem + L::kStageOff;
    uint8_t* s_k = smem + L::kKOff;
    uint8_t* s_v = smem + L::kVOff;
    Control* ctrl = reinterpret_cast<Control*>(smem + L::kCtrlOff);
    volatile int32_t* status = p.status;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 = even CTA (issues the MMAs)
    const int64_t first_item = cluster_id_x();
    const int64_t item_step = cluster_count_x();
#ifdef SPLAT_PAIR_TRACE
    const bool trace_on = p.trace != nullptr && first_item == item_step / 2 && rank == 0;
    int trace_n = 0;
#endif

    // ------------------------------------------------------------------ prologue
    if (warp == kMmaWarp) {
        tmem_alloc_pair(&ctrl->tmem_base, kTmemCols);
        tmem_relinquish_pair();
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kEvents; ++i) mbar_init(&ctrl->ev[i], 1);
        for (int i = 0; i < 2; ++i) mbar_init(&ctrl->q_full[i], 1);
        for (int i = 0; i < kBufs; ++i) {
            mbar_init(&ctrl->k_full[i], 1);
            mbar_init(&ctrl->v_full[i], 1);
            mbar_init(&ctrl->p_ready[i], 8);
        }
        mbar_init(&ctrl->o_free, 8);
        mbar_init(&ctrl->drain, 1);
        mbar_init(&ctrl->stage_free, 1);
        mbar_init(&ctrl->stage_ready, 4);
        mbar_fence_init();
        ctrl->abort_at_entry = *status;
    }
    // Range table: for every (class, row block) the key tiles [n_lo, n_lo + N) that cover every band
    // row of the block's 256 rows.  One warp per entry, lane l looks at rows l, l + 32, ...
    for (int e = warp; e < p.n_entries; e += kWarps) {
        const int res = e / p.items_per_class, block = e - res * p.items_per_class;
        int lo = INT_MAX, hi = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int u = block * kItemRows + j * 32 + lane;
            if (u < p.rows_v) {
                const int64_t row = (int64_t)u * p.stride + res;
                int a, n, start, nnz;
                row_band(p, res, __ldg(p.lin + row), __ldg(p.tr + row), __ldg(p.nnzs + row), a, n, start, nnz);
                if (n > 0) { lo = min(lo, a / kTile); hi = max(hi, (a + n + kTile - 1) / kTile); }
            }
        }
        lo = warp_min_i(lo);
        hi = warp_max_i(hi);
        hi = min(hi, (p.rows_v + kTile - 1) / kTile);
        if (lo >= hi) { lo = 0; hi = 0; }
        if (lane == 0) ctrl->range[e] = (uint32_t)lo | ((uint32_t)(hi - lo) << 16);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();      // the other CTA's barriers are initialised before anything targets them
    tc_fence_after_sync();
    const uint32_t tmem_base = ctrl->tmem_base;
    // both CTAs read the same global word; a differing view could only come from a concurrent
    // writer, i.e. a kernel that is giving up right now, and then the bounded waits end this one too
    const bool run = ctrl->abort_at_entry == 0;

    // shared::cluster addresses of the even CTA's barriers (valid from either CTA)
    auto leader_addr = [&](uint64_t* bar) { return map_to_cta(smem_u32(bar), 0); };
    auto event_wait = [&](int64_t e, int code) {
        return mbar_wait(&ctrl->ev[e & (kEvents - 1)], (uint32_t)(e >> 5) & 1u, status, code);
    };
    // item w -> position and range; false when the item has no steps
    auto load_item = [&](Cursor& c) {
        const int e = (int)(c.w % p.n_entries);
        c.bh = c.w / p.n_entries;
        c.res = e / p.items_per_class;
        c.block = e - c.res * p.items_per_class;
        const uint32_t r = ctrl->range[e];
        c.n_lo = (int)(r & 0xffffu);
        c.N = (int)(r >> 16);
        return c.N > 0;
    };
    auto cursor_begin = [&](Cursor& c) {
        c.w = first_item; c.G = 0; c.i = 0; c.jq = 0;
        c.valid = false;
        for (; c.w < p.n_items; c.w += item_step)
            if (load_item(c)) { c.valid = true; break; }
    };
    auto cursor_next = [&](Cursor& c) {
        ++c.G;
        if (++c.i < c.N) return;
        c.i = 0; ++c.jq;
        c.valid = false;
        for (c.w += item_step; c.w < p.n_items; c.w += item_step)
            if (load_item(c)) { c.valid = true; break; }
    };

    if (run && warp == kTmaWarp) {
        // ------------------------------------------------------------------ TMA producer
        // Loads follow the order in which the tensor core consumes them: K(0) K(1) K(2), then
        // V(G), K(G+3) for every step, with the Q tile of an item just before its first K tile.
        // This CTA loads keys [64 rank, +64) of every K tile and value columns [64 rank, +64) of
        // every V tile.
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            int64_t q_last0 = -1, q_last1 = -1;   // last S step of the item that used each Q buffer
            int64_t seen = -1;                    // newest event known complete (events complete in order)
            auto slot_wait = [&](int64_t e) {
                if (e <= seen) return true;
                if (!event_wait(e, kErrEvent)) return false;
                seen = e;
                return true;
            };
            auto load_k = [&](const Cursor& c) {
                if (c.i == 0) {                 // first step of an item: its Q tile
                    const int qb = c.jq & 1;
                    if (!slot_wait(qb ? q_last1 : q_last0)) return false;
                    if (rank == 0) mbar_arrive_expect_tx(&ctrl->q_full[qb], 2 * kTileBytes);
                    const uint32_t bar = leader_addr(&ctrl->q_full[qb]);
                    for (int sub = 0; sub < 2; ++sub)
                        tma_load_4d_pair(s_q + qb * kTileBytes + sub * kSubBytes, &tm_q, bar, sub * 64,
                                         c.res, c.block * kItemRows + (int)rank * kTile, (int)c.bh);
                    if (qb) q_last1 = c.G + c.N - 1; else q_last0 = c.G + c.N - 1;
                    PAIR_TRACE(2, 21);
                }
                const int slot = (int)(c.G % kBufs);
                if (!slot_wait(c.G - kBufs)) return false;       // S(G-3) has read this slot
                if (rank == 0) mbar_arrive_expect_tx(&ctrl->k_full[slot], 2 * kSlotBytes);
                const uint32_t bar = leader_addr(&ctrl->k_full[slot]);
                for (int sub = 0; sub < 2; ++sub)
                    tma_load_4d_pair(s_k + slot * kSlotBytes + sub * kKHalfSub, &tm_k, bar, sub * 64, c.res,
                                     (c.n_lo + c.i) * kTile + (int)rank * 64, (int)c.bh);
                PAIR_TRACE(2, 22);
                return true;
            };
            auto load_v = [&](const Cursor& c) {
                const int slot = (int)(c.G % kBufs);
                if (c.G >= kBufs && !slot_wait(c.G)) return false;   // PV(G-3) has read this slot
                if (rank == 0) mbar_arrive_expect_tx(&ctrl->v_full[slot], 2 * kSlotBytes);
                tma_load_4d_pair(s_v + slot * kSlotBytes, &tm_v, leader_addr(&ctrl->v_full[slot]),
                                 (int)rank * 64, c.res, (c.n_lo + c.i) * kTile, (int)c.bh);
                PAIR_TRACE(2, 23);
                return true;
            };
            Cursor kc, vc;
            cursor_begin(kc);
            cursor_begin(vc);
            bool ok = true;
            for (int t = 0; t < kBufs && kc.valid && ok; ++t) {
                ok = load_k(kc);
                cursor_next(kc);
            }
            while (vc.valid && ok) {
                ok = load_v(vc);
                cursor_next(vc);
                if (ok && kc.valid) {
                    ok = load_k(kc);
                    cursor_next(kc);
                }
            }
            // giving up: copies already issued may still be landing (some counted on the other
            // CTA's barriers); let them finish before either CTA can leave
            if (!ok) spin_cycles(400000);
        }
    } else if (run && warp == kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer (even CTA)
        if (rank == 0 && lane == 0) {
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t idesc_qk = instr_desc_f16(fmt, 2 * kTile, kTile, 0);
            constexpr uint32_t idesc_pv = instr_desc_f16(fmt, 2 * kTile, D, 1);
            const uint32_t q_addr = smem_u32(s_q), k_addr = smem_u32(s_k), v_addr = smem_u32(s_v);
            const uint32_t ev_own = smem_u32(&ctrl->ev[0]);
            const uint32_t ev_peer = map_to_cta(ev_own, 1);
            const uint32_t o_tmem = tmem_base + kOCol;
            uint32_t k_ph = 0, v_ph = 0, p_ph = 0;     // one phase bit per slot
            bool ok = true;
            auto commit_event = [&](int64_t e) {
                const uint32_t off = (uint32_t)(e & (kEvents - 1)) * 8u;
                mma_commit_pair(ev_own + off);
                mma_commit_pair(ev_peer + off);
            };
            // S of the step at cursor c, into score buffer G mod 3
            auto issue_s = [&](const Cursor& c) {
                const int qb = c.jq & 1;
                if (c.i == 0 &&
                    !mbar_wait(&ctrl->q_full[qb], (uint32_t)(c.jq >> 1) & 1u, status, kErrQ))
                    return false;
                const int slot = (int)(c.G % kBufs);
                const bool r = mbar_wait(&ctrl->k_full[slot], (k_ph >> slot) & 1u, status, kErrKFull);
                k_ph ^= 1u << slot;
                if (!r) return false;
                tc_fence_after_sync();
                const uint32_t q_base = q_addr + qb * kTileBytes;
                const uint32_t b_base = k_addr + slot * kSlotBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    mma_ss_pair(tmem_base + slot * kTile,
                                smem_desc_sw128(q_base + (kk >> 2) * kSubBytes + (kk & 3) * 32, 16, 1024),
                                smem_desc_sw128(b_base + (kk >> 2) * kKHalfSub + (kk & 3) * 32, 16, 1024),
                                idesc_qk, kk > 0);
                return true;
            };
            Cursor sc, pc;
            cursor_begin(sc);
            cursor_begin(pc);
            for (int t = 0; t < kBufs && ok; ++t) {
                if (sc.valid) {
                    ok = issue_s(sc);
                    cursor_next(sc);
                }
                if (ok) commit_event(t);
            }
            while (pc.valid && ok) {
                const int slot = (int)(pc.G % kBufs);
                ok = mbar_wait(&ctrl->v_full[slot], (v_ph >> slot) & 1u, status, kErrVFull);
                v_ph ^= 1u << slot;
                if (!ok) break;
                PAIR_TRACE(1, 10);
                ok = mbar_wait(&ctrl->p_ready[slot], (p_ph >> slot) & 1u, status, kErrPReady);
                p_ph ^= 1u << slot;
                if (!ok) break;
                if (pc.i == 0 && pc.jq > 0) {      // the previous item's O has been read out
                    ok = mbar_wait(&ctrl->o_free, (uint32_t)(pc.jq - 1) & 1u, status, kErrOFree);
                    if (!ok) break;
                }
                tc_fence_after_sync();
                PAIR_TRACE(1, 11);
                // O += P V: P packed in the first 64 columns of the step's score buffer
                {
                    const uint32_t b_base = v_addr + slot * kSlotBytes;
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        mma_ts_pair(o_tmem, tmem_base + slot * kTile + kk * 8,
                                    smem_desc_sw128(b_base + kk * 2048, kSlotBytes, 1024), idesc_pv,
                                    (pc.i > 0 || kk > 0) ? 1u : 0u);
                }
                if (sc.valid) {                    // S(G+3) into the buffer PV(G) has just consumed
                    ok = issue_s(sc);
                    if (!ok) break;
                    cursor_next(sc);
                }
                commit_event(pc.G + kBufs);
                PAIR_TRACE(1, 12);
                cursor_next(pc);
            }
            if (!ok) {
                // let the tensor pipe drain before tensor memory is released
                mma_commit_pair(smem_u32(&ctrl->drain));
                const long long t0 = clock64();
                while (!mbar_try_wait(&ctrl->drain, 0))
                    if (clock64() - t0 > 200000000LL) break;
            }
        }
    } else if (run && warp < 4) {
        // ------------------------------------------------------------------ softmax + epilogue
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        const uint32_t o_addr = lane_addr + kOCol;
        const int t = warp * 32 + lane;              // row of this thread within the CTA's tile
        const float sc = p.scale_log2;
        const float2 sc2 = make_float2(sc, sc);
        const uint32_t p_ready_addr = leader_addr(&ctrl->p_ready[0]);
        const uint32_t o_free_addr = leader_addr(&ctrl->o_free);
        int64_t G0 = 0;             // global step of the item's first step
        int n_epi = 0;              // epilogues so far: phase of the staging barriers
        bool ok = true;
        // metadata of this thread's row, loaded one item ahead
        auto own_row = [&](int64_t w, int& u) {
            const int e = (int)(w % p.n_entries);
            const int res = e / p.items_per_class, block = e - res * p.items_per_class;
            u = block * kItemRows + (int)rank * kTile + t;
            return (int64_t)min(u, p.rows_v - 1) * p.stride + res;
        };
        float nx_lin, nx_tr, nx_nn;
        {
            int u;
            const int64_t row = own_row(first_item, u);
            nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
        }
        for (int64_t w = first_item; w < p.n_items; w += item_step) {
            Cursor cur;
            cur.w = w;
            load_item(cur);
            const int N = cur.N, n_lo = cur.n_lo;
            int u_own;
            (void)own_row(w, u_own);
            const bool row_exists = u_own < p.rows_v;
            int my_a, my_n, row_start, row_nnz;
            row_band(p, cur.res, nx_lin, nx_tr, row_exists ? nx_nn : 0.f, my_a, my_n, row_start, row_nnz);
            if (w + item_step < p.n_items) {      // next item's row: in flight during this item's steps
                int u;
                const int64_t row = own_row(w + item_step, u);
                nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
            }
            // last step of this item in which some row of this warp has valid columns (-1: none)
            const int hi_tile = warp_max_i(my_n > 0 ? (my_a + my_n + kTile - 1) / kTile : 0);
            const int last_active = min(hi_tile, n_lo + N) - 1 - n_lo;
            float m_used = -INFINITY, l_sum = 0.f;
            int pending = -1;        // score buffer whose P has been stored but not yet handed over

            // P of the pending buffer is complete in tensor memory: tell the MMA thread
            auto hand_over = [&]() {
                tmem_st_wait();
                PAIR_TRACE(0, 13);
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(p_ready_addr + pending * 8);
                pending = -1;
            };

            for (int i = 0; i < N; ++i) {
                const int64_t G = G0 + i;
                const int slot = (int)(G % kBufs);
                const uint32_t s_addr = lane_addr + slot * kTile;
                const int c0 = (n_lo + i) * kTile;
                const int v_lo = my_a - c0;               // valid columns of this step: [v_lo, v_hi)
                const int v_hi = my_n > 0 ? my_a + my_n - c0 : INT_MIN;
                const bool row_in = my_n > 0 && v_lo < kTile && v_hi > 0;
                const bool warp_in = __any_sync(0xffffffffu, row_in);
                PAIR_TRACE(0, 1);
                ok = event_wait(G, kErrEvent);            // S(G) complete (and PV(G-3): the buffer is free)
                ok = __all_sync(0xffffffffu, ok);         // keep the warp together for the aligned tcgen05 ops
                if (!ok) break;
                tc_fence_after_sync();
                PAIR_TRACE(0, 2);
                uint32_t r[kTile];
                if (!warp_in) {
                    // none of this warp's rows reaches into this step (the other tile's does):
                    // the pair MMA still multiplies these rows, so P must be zero
                    if (pending >= 0) hand_over();
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0u;
                    tmem_st32(s_addr, r);
                    tmem_st32(s_addr + 32, r);
                    pending = slot;
                    continue;
                }
#ifndef SPLAT_ABL_NOLD
                tmem_ld32(s_addr, r);
                tmem_ld32(s_addr + 32, r + 32);
                tmem_ld32(s_addr + 64, r + 64);
                tmem_ld32(s_addr + 96, r + 96);
                tmem_ld_wait();
#else
#pragma unroll
                for (int j = 0; j < kTile; ++j) r[j] = 0x3f800000u + j + lane;
#endif
                PAIR_TRACE(0, 3);
                const bool lo_ok = __all_sync(0xffffffffu, v_lo <= 0);
                const bool hi_ok = __all_sync(0xffffffffu, v_hi >= kTile);
                // band edge: columns outside [v_lo, v_hi) become -inf (exp2 -> 0)
                if (!lo_ok && !hi_ok) {
#pragma unroll
                    for (int j = 0; j < kTile; ++j)
                        r[j] = (j >= v_lo && j < v_hi) ? r[j] : 0xff800000u;
                } else if (!hi_ok) {
#pragma unroll
                    for (int j = 0; j < kTile; ++j) r[j] = j < v_hi ? r[j] : 0xff800000u;
                } else if (!lo_ok) {
#pragma unroll
                    for (int j = 0; j < kTile; ++j) r[j] = j >= v_lo ? r[j] : 0xff800000u;
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
                const float m_new = fmaxf(m_used, mt * sc);
                const bool need = (m_new - m_used) > kRescaleThreshold;  // false when both are -inf
                const float corr = need ? ex2(m_used - m_new) : 1.f;
                if (need) m_used = m_new;
                l_sum *= corr;
                const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
                PAIR_TRACE(0, 4);
                // the previous step's P has had the time of this step's load and maximum to land
                if (pending >= 0) hand_over();
                PAIR_TRACE(0, 9);

                // lazy rescale of the accumulator (rare): some row's maximum moved by more than
                // 2^8.  PV(G-1) may still be running: wait for its event first.
                if (i > 0 && __any_sync(0xffffffffu, need)) {
                    ok = event_wait(G - 1 + kBufs, kErrEvent);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (int ch = 0; ch < D / 16; ++ch) {
                        uint32_t o[16];
                        tmem_ld16(o_addr + ch * 16, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
                        tmem_st16(o_addr + ch * 16, o);
                    }
                }

                // probabilities: exp2(s*c - m) with packed fp32x2 FMAs, row sum, 16-bit pack in place.
                // The special function unit (16 exp2 per clock and SM) is the narrowest pipe here, so
                // in steps without masked columns kPolyPairs of every four pairs take the polynomial
                // on the FMA pipes instead.
                const float2 nm2 = make_float2(-m_eff, -m_eff);
                float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#ifndef SPLAT_ABL_NOEXP
                if (kPolyPairs > 0 && lo_ok && hi_ok)
                    exp_rows<T, kPolyPairs>(r, sc2, nm2, acc0, acc1);
                else
                    exp_rows<T, 0>(r, sc2, nm2, acc0, acc1);
#endif
                l_sum += (acc0.x + acc0.y) + (acc1.x + acc1.y);
#ifndef SPLAT_ABL_NOST
                tmem_st32(s_addr, r);          // P: 64 packed columns over the consumed scores
                tmem_st32(s_addr + 32, r + 32);
#else
                if (r[5] == 0x12345u) tmem_st32(s_addr, r);
#endif
                pending = slot;
                PAIR_TRACE(0, 5);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (ok && pending >= 0) hand_over();
            PAIR_TRACE(0, 6);

            // This warp's rows of O are final once the PV of its last step with valid columns has
            // completed; later steps of the item (the other tile's) add zeros to them.  A warp
            // without such a step still waits for the item's first PV: that MMA is only issued once
            // every warp has released the previous item's O, so no warp can signal "O read" for this
            // item while that barrier is still collecting the previous item's arrivals.
            const bool have_o = ok && last_active >= 0;
            if (ok && N > 0) {
                ok = event_wait(G0 + max(last_active, 0) + kBufs, kErrEvent);
                ok = __all_sync(0xffffffffu, ok);
                tc_fence_after_sync();
            }
            PAIR_TRACE(0, 7);
            // epilogue: O / l for band rows, V[start] for single-element rows, zero otherwise.  Rows
            // are staged in shared memory in the 128-byte-swizzled tile layout and leave through one
            // tiled TMA store per 64-column half (rows past the end of the class are clipped by the
            // tensor map).  The staging buffer is free once the previous item's store has read it.
            if (threadIdx.x == 0) {
                tma_store_wait_read();
                mbar_arrive(&ctrl->stage_free);
            }
            if (!mbar_wait(&ctrl->stage_free, (uint32_t)n_epi & 1u, status, kErrStage)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            {
                uint32_t r[32];
                const T* vrow = reinterpret_cast<const T*>(p.v) + (cur.bh * p.n_rows + (int64_t)row_start) * D;
                const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
#pragma unroll
                for (int ch = 0; ch < D / 32; ++ch) {
                    if (have_o) {  // warp-uniform
                        tmem_ld32(o_addr + ch * 32, r);
                        tmem_ld_wait();
                    }
                    uint4 out[4];
                    if (row_nnz > 1 && have_o) {
                        uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
#pragma unroll
                        for (int j = 0; j < 32; j += 2)
                            o32[j >> 1] = pack2<T>(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
                    } else if (row_nnz == 1 && row_exists) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4)
                            out[q4] = *reinterpret_cast<const uint4*>(vrow + ch * 32 + q4 * 8);
                    } else {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) out[q4] = make_uint4(0, 0, 0, 0);
                    }
                    uint8_t* srow = s_stage + (ch >> 1) * kSubBytes + t * 128;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        *reinterpret_cast<uint4*>(srow + ((((ch & 1) * 4 + q4) ^ (t & 7)) << 4)) = out[q4];
                }
            }
            if (N > 0) {       // O is in registers / shared memory: the next item may overwrite it
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(o_free_addr);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->stage_ready);
            if (threadIdx.x == 0) {
                if (mbar_wait(&ctrl->stage_ready, (uint32_t)n_epi & 1u, status, kErrStage)) {
                    if (cur.block * kItemRows + (int)rank * kTile < p.rows_v) {
                        for (int sub = 0; sub < 2; ++sub)
                            tma_store_4d(&tm_o, s_stage + sub * kSubBytes, sub * 64, cur.res,
                                         cur.block * kItemRows + (int)rank * kTile, (int)cur.bh);
                        tma_store_commit();
                    }
                } else {
                    ok = false;
                }
            }
            ok = __all_sync(0xffffffffu, ok);
            ++n_epi;
            PAIR_TRACE(0, 8);
            G0 += N;
            if (!ok) break;
        }
        if (threadIdx.x == 0) tma_store_wait_read();
    }

    // ------------------------------------------------------------------ exit
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();      // nothing of either CTA is in flight towards the other any more
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static long long* g_trace = nullptr;

// Number of CTA pairs that can be resident at once on the current device (cached per device).
template <typename T>
static int resident_pairs() {
    static std::mutex mu;
    static int cached[64];
    static bool known[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (!known[dev]) {
        auto kern = attention_pair_kernel<T>;
        int n = 0;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout::kSmemBytes) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.gridDim = dim3(2, 1, 1);
            cfg.blockDim = dim3(kThreads, 1, 1);
            cfg.dynamicSmemBytes = Layout::kSmemBytes;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) n = 0;
        }
        (void)cudaGetLastError();
        cached[dev] = n;
        known[dev] = true;
    }
    return cached[dev];
}

template <typename T>
static int32_t launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                      const CUtensorMap& mo, const Params& prm, int max_pairs, cudaStream_t st) {
    int pairs = resident_pairs<T>();
    if (pairs < 1) return SPLAT_ERR_UNSUPPORTED_SHAPE;    // no room for a pair: use the other kernels
    if (max_pairs > 0 && pairs > max_pairs) pairs = max_pairs;
    if ((int64_t)pairs > prm.n_items) pairs = (int)prm.n_items;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Layout::kSmemBytes;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, attention_pair_kernel<T>, mq, mk, mv, mo, prm) != cudaSuccess) {
        (void)cudaGetLastError();
        return SPLAT_ERR_LAUNCH;
    }
    return launch_status();
}

}  // namespace pair

// Band attention on CTA pairs.  Same contract as attention_band (attention_band.cu), which has
// already validated the operands; d must be 128.  Returns SPLAT_ERR_UNSUPPORTED_SHAPE (nothing
// launched) for sequence lengths beyond what its range table or its float32 index arithmetic
// cover.  max_pairs > 0 limits the number of resident pairs (bring-up and tests).
int32_t attention_pair(const void* q, const void* k, const void* v, void* o, const float* lin,
                       const float* tr, const float* nnzs, int64_t bh, int64_t n_rows, int64_t stride,
                       float scale, int32_t dtype, int32_t* status_word, int max_pairs,
                       cudaStream_t st) {
    const int64_t d = pair::D;
    const int64_t rows_v = n_rows / stride;
    const int64_t items_per_class = (rows_v + pair::kItemRows - 1) / pair::kItemRows;
    if (n_rows > (1ll << 22) || items_per_class * stride > pair::kMaxEntries)
        return SPLAT_ERR_UNSUPPORTED_SHAPE;
    CUtensorMap mq, mk, mv, mo;
    if (!band::make_map(&mq, q, dtype, bh, n_rows, d, stride, pair::kTile) ||
        !band::make_map(&mk, k, dtype, bh, n_rows, d, stride, 64) ||
        !band::make_map(&mv, v, dtype, bh, n_rows, d, stride, pair::kTile) ||
        !band::make_map(&mo, o, dtype, bh, n_rows, d, stride, pair::kTile))
        return SPLAT_ERR_DRIVER;
    pair::Params prm;
    prm.lin = lin; prm.tr = tr; prm.nnzs = nnzs; prm.v = v; prm.status = status_word;
    prm.trace = pair::g_trace;
    prm.n_rows = n_rows;
    prm.rows_v = (int)rows_v;
    prm.stride = (int)stride;
    prm.items_per_class = (int)items_per_class;
    prm.n_entries = (int)(items_per_class * stride);
    prm.n_items = (int64_t)prm.n_entries * bh;
    prm.scale_log2 = scale * kLog2e;
    if (dtype == SPLAT_BF16)
        return pair::launch<__nv_bfloat16>(mq, mk, mv, mo, prm, max_pairs, st);
    return pair::launch<__half>(mq, mk, mv, mo, prm, max_pairs, st);
}

}  // namespace splat

#ifdef SPLAT_PAIR_TRACE
extern "C" void splat_debug_set_pair_trace(void* device_buffer_3x2048_i64) {
    splat::pair::g_trace = reinterpret_cast<long long*>(device_buffer_3x2048_i64);
}
#endif
