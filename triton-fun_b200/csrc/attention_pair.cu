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
// the even CTA, whose MMA warp is the only consumer.
//
// Progress of the tensor core is published as numbered EVENTS: event e is one tcgen05.commit per
// CTA onto barrier e mod 32 of that CTA.  Event G = "S(G) complete", event G + 3 = "PV(G)
// complete" (one commit after PV(G), S(G+3) serves both).  Softmax warps wait for S(G); epilogue
// warps for the PV of their rows' last step; the TMA producers for the event that frees the slot
// they are about to overwrite.  Every role walks the same item list with the per-item (n_lo, N)
// taken from a table in shared memory that each CTA builds from the row metadata at kernel start,
// so no role has to tell another what comes next.
//
// Warps per CTA (three warpgroups with their own register budgets): 0-3 softmax (never wait for a
// PV except to rescale O), 4-7 epilogue (normalise O
// with the row sums the softmax warps leave in shared memory, stage, TMA store; this overlaps the
// next item's softmax), 8 TMA producer, 9 MMA issuer (even CTA; the whole warp runs the loop and
// one elected lane issues) and tensor-memory owner (both).  Every mbarrier wait is bounded; a role
// that gives up records a code in the status word, the others see the word in their own waits,
// and both CTAs meet at a cluster barrier before tensor memory is released and either CTA leaves.
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
constexpr int kHalf = 64;              // score columns a softmax thread holds at a time
constexpr int kItemRows = 2 * kTile;   // rows per work item (CTA pair)
constexpr int kThreads = 384;           // 12 warps: softmax 0-3, epilogue 4-7, TMA 8, MMA 9, two idle
constexpr int kWarps = kThreads / 32;
constexpr int kEpiWarp = 4;            // warps 4..7
constexpr int kTmaWarp = 8;
constexpr int kMmaWarp = 9;
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
constexpr int kRegsSoftmax = 232, kRegsEpilogue = 152, kRegsOther = 96;   // 128 * sum <= 64 K registers
#ifndef SPLAT_PAIR_POLY_PAIRS
#define SPLAT_PAIR_POLY_PAIRS 0
#endif
constexpr int kPolyPairs = SPLAT_PAIR_POLY_PAIRS;   // of every 4 pairs of exponentials, on the FMA pipes

// status-word codes (which wait gave up)
enum : int { kErrQ = 11, kErrKFull = 12, kErrVFull = 13, kErrEvent = 14, kErrPReady = 15,
             kErrOFree = 16, kErrStage = 17, kErrRowSum = 18 };

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
    uint64_t l_full[2];        // own CTA, 4 arrivals: row sums of an item are in l_buf (items alternate)
    uint64_t l_free[2];        // own CTA, 4 arrivals: the epilogue warps have read them
    uint64_t stage_free;       // own CTA: the previous TMA store has read the output staging buffer
    uint64_t stage_ready;      // own CTA, 4 arrivals: the epilogue warps have written their rows
    uint32_t tmem_base;
    int32_t abort_at_entry;
    float l_buf[2][kTile];
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
        if (trace_on && lane == 0 && (warp & 3) == (warp < 8 ? 0 : warp & 3) && trace_n < 2048)    \
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

// Position in the item list of this CTA pair (w = e + n_entries * bh, advanced without divisions).
struct ItemPos {
    int64_t w, bh;
    int e;
};
// Position in the stream of steps of this CTA pair.
struct Cursor {
    ItemPos at;
    int64_t G;        // global step
    int i, N, n_lo;   // step within the item, steps of the item, first key tile of the item
    int jq;           // items with steps before this one
    int block, res;
    bool valid;
};

__device__ __forceinline__ void spin_cycles(long long n) {
    const long long t0 = clock64();
    while (clock64() - t0 < n) { }
}

// Keeps the compiler from using registers a tcgen05.ld writes before the wait that follows it.
__device__ __forceinline__ void reg_fence16(uint32_t* r) {
    asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                      "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]),
                      "+r"(r[13]), "+r"(r[14]), "+r"(r[15]));
}
__device__ __forceinline__ void reg_fence64(uint32_t* r) {
    reg_fence16(r); reg_fence16(r + 16); reg_fence16(r + 32); reg_fence16(r + 48);
}

// x[J0..J1) of a 64-score half -> packed 16-bit probabilities exp2(s*c - m) in x[J0/2..J1/2); row
// sums into acc0/acc1.  kPolyPairs of every four pairs are evaluated on the FMA pipes, the rest on
// the special function unit (16 exp2 per clock and SM: the narrowest pipe of the softmax).
template <typename T, int J0, int J1>
__device__ __forceinline__ void exp_part(uint32_t* x, float2 sc2, float2 nm2, float2& acc0, float2& acc1) {
#pragma unroll
    for (int j = J0; j < J1; j += 8) {
        float2 a[4];
#pragma unroll
        for (int c = 0; c < 4; ++c)
            a[c] = fma2(make_float2(__uint_as_float(x[j + 2 * c]), __uint_as_float(x[j + 2 * c + 1])), sc2, nm2);
#ifndef SPLAT_ABL_NOEXP
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (c < kPolyPairs) a[c] = ex2_poly2(a[c]);
            else { a[c].x = ex2(a[c].x); a[c].y = ex2(a[c].y); }
        }
#endif
        acc0 = add2(acc0, add2(a[0], a[1]));
        acc1 = add2(acc1, add2(a[2], a[3]));
#pragma unroll
        for (int c = 0; c < 4; ++c) x[(j >> 1) + c] = pack2<T>(a[c].x, a[c].y);
    }
}

// Band edge: columns of half H outside [v_lo, v_hi) (step-relative) become -inf; then the row maximum.
template <int H>
__device__ __forceinline__ float masked_max(uint32_t* x, int v_lo, int v_hi, bool lo_ok, bool hi_ok) {
    if (!lo_ok && !hi_ok) {
#pragma unroll
        for (int j = 0; j < kHalf; ++j)
            x[j] = (j + H * kHalf >= v_lo && j + H * kHalf < v_hi) ? x[j] : 0xff800000u;
    } else if (!hi_ok) {
#pragma unroll
        for (int j = 0; j < kHalf; ++j) x[j] = j + H * kHalf < v_hi ? x[j] : 0xff800000u;
    } else if (!lo_ok) {
#pragma unroll
        for (int j = 0; j < kHalf; ++j) x[j] = j + H * kHalf >= v_lo ? x[j] : 0xff800000u;
    }
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < kHalf; j += 8) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
            mx[c] = fmax3(mx[c], __uint_as_float(x[j + 2 * c]), __uint_as_float(x[j + 2 * c + 1]));
    }
    return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
}
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
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
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ctrl->q_full[i], 1);
            mbar_init(&ctrl->l_full[i], 4);
            mbar_init(&ctrl->l_free[i], 4);
        }
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
    // walking the item list: w -> w + item_step without 64-bit divisions
    const int step_e = (int)(item_step % p.n_entries);
    const int64_t step_bh = item_step / p.n_entries;
    auto pos_begin = [&](ItemPos& at) {
        at.w = first_item;
        at.e = (int)(first_item % p.n_entries);
        at.bh = first_item / p.n_entries;
    };
    auto pos_next = [&](ItemPos& at) {
        at.w += item_step;
        at.e += step_e;
        at.bh += step_bh;
        if (at.e >= p.n_entries) { at.e -= p.n_entries; ++at.bh; }
    };
    // item at c.at -> class, block and range; false when the item has no steps
    auto load_item = [&](Cursor& c) {
        c.res = c.at.e / p.items_per_class;
        c.block = c.at.e - c.res * p.items_per_class;
        const uint32_t r = ctrl->range[c.at.e];
        c.n_lo = (int)(r & 0xffffu);
        c.N = (int)(r >> 16);
        return c.N > 0;
    };
    auto cursor_begin = [&](Cursor& c) {
        pos_begin(c.at);
        c.G = 0; c.i = 0; c.jq = 0;
        c.valid = false;
        for (; c.at.w < p.n_items; pos_next(c.at))
            if (load_item(c)) { c.valid = true; break; }
    };
    auto cursor_next = [&](Cursor& c) {
        ++c.G;
        if (++c.i < c.N) return;
        c.i = 0; ++c.jq;
        c.valid = false;
        for (pos_next(c.at); c.at.w < p.n_items; pos_next(c.at))
            if (load_item(c)) { c.valid = true; break; }
    };

    // Each warpgroup takes its register budget (the softmax threads keep 128 scores in registers)
    // and then runs its role; the budgets only hold inside these branches.
    if (warp >= kTmaWarp) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
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
                                         c.res, c.block * kItemRows + (int)rank * kTile, (int)c.at.bh);
                    if (qb) q_last1 = c.G + c.N - 1; else q_last0 = c.G + c.N - 1;
                    PAIR_TRACE(2, 21);
                }
                const int slot = (int)(c.G % kBufs);
                if (!slot_wait(c.G - kBufs)) return false;       // S(G-3) has read this slot
                if (rank == 0) mbar_arrive_expect_tx(&ctrl->k_full[slot], 2 * kSlotBytes);
                const uint32_t bar = leader_addr(&ctrl->k_full[slot]);
                for (int sub = 0; sub < 2; ++sub)
                    tma_load_4d_pair(s_k + slot * kSlotBytes + sub * kKHalfSub, &tm_k, bar, sub * 64, c.res,
                                     (c.n_lo + c.i) * kTile + (int)rank * 64, (int)c.at.bh);
                PAIR_TRACE(2, 22);
                return true;
            };
            auto load_v = [&](const Cursor& c) {
                const int slot = (int)(c.G % kBufs);
                if (c.G >= kBufs && !slot_wait(c.G)) return false;   // PV(G-3) has read this slot
                if (rank == 0) mbar_arrive_expect_tx(&ctrl->v_full[slot], 2 * kSlotBytes);
                tma_load_4d_pair(s_v + slot * kSlotBytes, &tm_v, leader_addr(&ctrl->v_full[slot]),
                                 (int)rank * 64, c.res, (c.n_lo + c.i) * kTile, (int)c.at.bh);
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
        // The whole warp walks the loop on warp-uniform values; one elected lane issues.
        if (rank == 0) {
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t idesc_qk = instr_desc_f16(fmt, 2 * kTile, kTile, 0);
            constexpr uint32_t idesc_pv = instr_desc_f16(fmt, 2 * kTile, D, 1);
            const bool lead = elect_one();
            const uint32_t q_addr = smem_u32(s_q), k_addr = smem_u32(s_k), v_addr = smem_u32(s_v);
            const uint32_t ev_own = smem_u32(&ctrl->ev[0]);
            const uint32_t ev_peer = map_to_cta(ev_own, 1);
            const uint32_t o_tmem = tmem_base + kOCol;
            uint32_t k_ph = 0, v_ph = 0, p_ph = 0;     // one phase bit per slot
            bool ok = true;
            auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
                const bool r = mbar_wait(bar, parity, status, code);
                return __all_sync(0xffffffffu, r) != 0;
            };
            auto commit_event = [&](int64_t e) {
                const uint32_t off = (uint32_t)(e & (kEvents - 1)) * 8u;
                if (lead) {
                    mma_commit_pair(ev_own + off);
                    mma_commit_pair(ev_peer + off);
                }
            };
            // S of the step at cursor c, into score buffer G mod 3
            auto issue_s = [&](const Cursor& c) {
                const int qb = c.jq & 1;
                if (c.i == 0 && !wait_all(&ctrl->q_full[qb], (uint32_t)(c.jq >> 1) & 1u, kErrQ)) return false;
                const int slot = (int)(c.G % kBufs);
                const bool r = wait_all(&ctrl->k_full[slot], (k_ph >> slot) & 1u, kErrKFull);
                k_ph ^= 1u << slot;
                if (!r) return false;
                tc_fence_after_sync();
                const uint32_t q_base = q_addr + qb * kTileBytes;
                const uint32_t b_base = k_addr + slot * kSlotBytes;
                const uint32_t d_tmem = tmem_base + slot * kTile;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t da = smem_desc_sw128(q_base + (kk >> 2) * kSubBytes + (kk & 3) * 32, 16, 1024);
                    const uint64_t db = smem_desc_sw128(b_base + (kk >> 2) * kKHalfSub + (kk & 3) * 32, 16, 1024);
                    if (lead) mma_ss_pair(d_tmem, da, db, idesc_qk, kk > 0);
                }
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
                ok = wait_all(&ctrl->v_full[slot], (v_ph >> slot) & 1u, kErrVFull);
                v_ph ^= 1u << slot;
                if (!ok) break;
                PAIR_TRACE(1, 10);
                ok = wait_all(&ctrl->p_ready[slot], (p_ph >> slot) & 1u, kErrPReady);
                p_ph ^= 1u << slot;
                if (!ok) break;
                if (pc.i == 0 && pc.jq > 0) {      // the previous item's O has been read out
                    ok = wait_all(&ctrl->o_free, (uint32_t)(pc.jq - 1) & 1u, kErrOFree);
                    if (!ok) break;
                }
                tc_fence_after_sync();
                PAIR_TRACE(1, 11);
                // O += P V: P packed in the first 64 columns of the step's score buffer
                {
                    const uint32_t b_base = v_addr + slot * kSlotBytes;
                    const uint32_t a_tmem = tmem_base + slot * kTile;
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk) {
                        const uint64_t db = smem_desc_sw128(b_base + kk * 2048, kSlotBytes, 1024);
                        if (lead) mma_ts_pair(o_tmem, a_tmem + kk * 8, db, idesc_pv, (pc.i > 0 || kk > 0) ? 1u : 0u);
                    }
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
            if (!ok && lead) {
                // let the tensor pipe drain before tensor memory is released
                mma_commit_pair(smem_u32(&ctrl->drain));
                const long long t0 = clock64();
                while (!mbar_try_wait(&ctrl->drain, 0))
                    if (clock64() - t0 > 200000000LL) break;
            }
            __syncwarp();
        }
      }
    } else if (warp < kEpiWarp) {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
      if (run) {
        // ------------------------------------------------------------------ softmax
        // Thread = row.  The 128 scores of a step pass through the registers in two halves, A and
        // B: while the exponentials of one half run on the special function unit, the other half
        // (of this step or the next) is loaded, masked and its maximum taken, so the two phases
        // overlap inside one warp.
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        const uint32_t o_addr = lane_addr + kOCol;
        const int t = warp * 32 + lane;              // row of this thread within the CTA's tile
        const float sc = p.scale_log2;
        const float2 sc2 = make_float2(sc, sc);
        const uint32_t p_ready_addr = leader_addr(&ctrl->p_ready[0]);
        int64_t G0 = 0;             // global step of the item's first step
        int n_item = 0;             // items so far
        bool ok = true;
        // metadata of this thread's row, loaded one item ahead
        auto own_row = [&](const ItemPos& at, int& res, int& u) {
            res = at.e / p.items_per_class;
            const int block = at.e - res * p.items_per_class;
            u = block * kItemRows + (int)rank * kTile + t;
            return (int64_t)min(u, p.rows_v - 1) * p.stride + res;
        };
        ItemPos at, nx;
        pos_begin(at);
        float nx_lin, nx_tr, nx_nn;
        {
            int res, u;
            const int64_t row = own_row(at, res, u);
            nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
        }
        for (; at.w < p.n_items; at = nx) {
            const uint32_t rg = ctrl->range[at.e];
            const int n_lo = (int)(rg & 0xffffu), N = (int)(rg >> 16);
            int res, u_own;
            (void)own_row(at, res, u_own);
            int my_a, my_n, row_start, row_nnz;
            row_band(p, res, nx_lin, nx_tr, u_own < p.rows_v ? nx_nn : 0.f, my_a, my_n, row_start, row_nnz);
            nx = at;
            pos_next(nx);
            if (nx.w < p.n_items) {      // next item's row: in flight during this item's steps
                int r2, u2;
                const int64_t row = own_row(nx, r2, u2);
                nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
            }
            float m_used = -INFINITY, l_sum = 0.f;
            int pending = -1;        // score buffer whose P has been stored but not yet handed over
            bool started = false;    // an earlier step of this item had valid columns for this warp: O is live
            bool a_ready = false;    // A holds the first half of the coming step, its maximum in mt_a
            float mt_a = -INFINITY;
            uint32_t A[kHalf], B[kHalf];

            // valid columns [v_lo, v_hi) of this thread's row in step i, relative to the step's first key
            auto step_cols = [&](int i, int& v_lo, int& v_hi, bool& warp_in, bool& lo_ok, bool& hi_ok) {
                const int c0 = (n_lo + i) * kTile;
                v_lo = my_a - c0;
                v_hi = my_n > 0 ? my_a + my_n - c0 : INT_MIN;
                warp_in = __any_sync(0xffffffffu, my_n > 0 && v_lo < kTile && v_hi > 0);
                lo_ok = __all_sync(0xffffffffu, v_lo <= 0);
                hi_ok = __all_sync(0xffffffffu, v_hi >= kTile);
            };
            // P of the pending buffer is complete in tensor memory: tell the MMA warp
            auto hand_over = [&]() {
                tmem_st_wait();
                PAIR_TRACE(0, 13);
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(p_ready_addr + pending * 8);
                pending = -1;
            };
            // New running maximum from the maximum mt of the coming half.  Lazy: the reference m_used
            // only moves when a row's maximum grows by more than 2^8, and then everything already
            // accumulated under the old reference is scaled by corr: l_sum, O (PV(G-1) must have
            // completed) and, when half_done, the first half of P(G) already stored in tensor memory.
            auto new_max = [&](float mt, int64_t G, uint32_t s_addr, bool half_done, float2& acc0,
                               float2& acc1) {
                const float m_new = fmaxf(m_used, mt * sc);
                const bool need = (m_new - m_used) > kRescaleThreshold;   // false when both are -inf
                const float corr = need ? ex2(m_used - m_new) : 1.f;
                if (need) m_used = m_new;
                l_sum *= corr;
                if (!__any_sync(0xffffffffu, need)) return true;
                // sums of the step's first half, not yet in l_sum
                acc0.x *= corr; acc0.y *= corr; acc1.x *= corr; acc1.y *= corr;
                if (started) {
                    bool r = event_wait(G - 1 + kBufs, kErrEvent);
                    r = __all_sync(0xffffffffu, r);
                    if (!r) return false;
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
                if (half_done) {
                    tmem_st_wait();      // the first half of P(G) was stored a moment ago
#pragma unroll
                    for (int ch = 0; ch < 2; ++ch) {
                        uint32_t w[16];
                        tmem_ld16(s_addr + ch * 16, w);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float2 f = unpack2<T>(w[j]);
                            w[j] = pack2<T>(f.x * corr, f.y * corr);
                        }
                        tmem_st16(s_addr + ch * 16, w);
                    }
                }
                return true;
            };

            for (int i = 0; i < N; ++i) {
                const int64_t G = G0 + i;
                const int slot = (int)(G % kBufs);
                const uint32_t s_addr = lane_addr + slot * kTile;
                int v_lo, v_hi;
                bool warp_in, lo_ok, hi_ok;
                step_cols(i, v_lo, v_hi, warp_in, lo_ok, hi_ok);
                PAIR_TRACE(0, 1);
                if (!a_ready) {
                    ok = event_wait(G, kErrEvent);            // S(G) complete (and PV(G-3): the buffer is free)
                    ok = __all_sync(0xffffffffu, ok);         // keep the warp together for the aligned tcgen05 ops
                    if (!ok) break;
                    tc_fence_after_sync();
                }
                PAIR_TRACE(0, 2);
                if (!warp_in) {
                    // none of this warp's rows reaches into this step (the other tile's does):
                    // the pair MMA still multiplies these rows, so P must be zero
                    if (pending >= 0) hand_over();
#pragma unroll
                    for (int j = 0; j < 32; ++j) B[j] = 0u;
                    tmem_st32(s_addr, B);
                    tmem_st32(s_addr + 32, B);
                    pending = slot;
                    a_ready = false;
                    continue;
                }
                if (!a_ready) {
#ifndef SPLAT_ABL_NOLD
                    tmem_ld32(s_addr, A);
                    tmem_ld32(s_addr + 32, A + 32);
                    tmem_ld_wait();
#endif
                    reg_fence64(A);
                    mt_a = masked_max<0>(A, v_lo, v_hi, lo_ok, hi_ok);
                }
                PAIR_TRACE(0, 3);
                // ---- first half: exponentials of A; B is loaded, masked and its maximum taken
#ifndef SPLAT_ABL_NOLD
                tmem_ld32(s_addr + 64, B);
                tmem_ld32(s_addr + 96, B + 32);
#endif
                if (pending >= 0) hand_over();   // the previous step's P has had time to land
                PAIR_TRACE(0, 9);
                float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
                ok = new_max(mt_a, G, s_addr, false, acc0, acc1);
                if (!ok) break;
                {
                    const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
                    const float2 nm2 = make_float2(-m_eff, -m_eff);
                    exp_part<T, 0, 16>(A, sc2, nm2, acc0, acc1);
                    tmem_ld_wait();
                    reg_fence64(B);
                    const float mt_b = masked_max<1>(B, v_lo, v_hi, lo_ok, hi_ok);
                    exp_part<T, 16, kHalf>(A, sc2, nm2, acc0, acc1);
#ifndef SPLAT_ABL_NOST
                    tmem_st32(s_addr, A);          // P of keys 0..63: 32 packed columns
#endif
                    PAIR_TRACE(0, 4);
                    // ---- second half: exponentials of B; the next step's first half goes into A
                    ok = new_max(mt_b, G, s_addr, true, acc0, acc1);
                    if (!ok) break;
                }
                a_ready = false;
                int nv_lo = 0, nv_hi = 0;
                bool n_lo_ok = true, n_hi_ok = true;
                if (i + 1 < N) {
                    bool n_in;
                    step_cols(i + 1, nv_lo, nv_hi, n_in, n_lo_ok, n_hi_ok);
                    const int64_t e = G + 1;
                    const bool ready = mbar_test_wait(&ctrl->ev[e & (kEvents - 1)], (uint32_t)(e >> 5) & 1u);
                    if (n_in && __all_sync(0xffffffffu, ready)) {
                        tc_fence_after_sync();
                        const uint32_t n_addr = lane_addr + (int)(e % kBufs) * kTile;
#ifndef SPLAT_ABL_NOLD
                        tmem_ld32(n_addr, A);
                        tmem_ld32(n_addr + 32, A + 32);
#endif
                        a_ready = true;
                    }
                }
                {
                    const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
                    const float2 nm2 = make_float2(-m_eff, -m_eff);
                    exp_part<T, 0, 16>(B, sc2, nm2, acc0, acc1);
                    if (a_ready) {
                        tmem_ld_wait();
                        reg_fence64(A);
                        mt_a = masked_max<0>(A, nv_lo, nv_hi, n_lo_ok, n_hi_ok);
                    }
                    exp_part<T, 16, kHalf>(B, sc2, nm2, acc0, acc1);
#ifndef SPLAT_ABL_NOST
                    tmem_st32(s_addr + 32, B);     // P of keys 64..127
#endif
                }
                l_sum += (acc0.x + acc0.y) + (acc1.x + acc1.y);
                pending = slot;
                started = true;      // from the next step on O holds this warp's rows of this item
                PAIR_TRACE(0, 5);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (pending >= 0) hand_over();
            PAIR_TRACE(0, 6);
            // row sums to the epilogue warps; the buffer was last used two items ago
            const int par = n_item & 1, use = n_item >> 1;
            if (use > 0) {
                ok = mbar_wait(&ctrl->l_free[par], (uint32_t)(use - 1) & 1u, status, kErrRowSum);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            ctrl->l_buf[par][t] = l_sum;
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->l_full[par]);
            PAIR_TRACE(0, 7);
            G0 += N;
            ++n_item;
        }
      }
    } else {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
      if (run) {
        // ------------------------------------------------------------------ epilogue
        // O / l for band rows, V[start] for single-element rows, zero otherwise.  Rows are staged
        // in shared memory in the 128-byte-swizzled tile layout and leave through one tiled TMA
        // store per 64-column half (rows past the end of the class are clipped by the tensor map).
        const int ew = warp - kEpiWarp;
        const uint32_t o_addr = tmem_base + ((uint32_t)(ew * 32) << 16) + kOCol;
        const int t = ew * 32 + lane;
        const uint32_t o_free_addr = leader_addr(&ctrl->o_free);
        const bool storer = ew == 0 && lane == 0;
        int64_t G0 = 0;
        int n_item = 0;
        bool ok = true;
        auto own_row = [&](const ItemPos& at, int& res, int& block, int& u) {
            res = at.e / p.items_per_class;
            block = at.e - res * p.items_per_class;
            u = block * kItemRows + (int)rank * kTile + t;
            return (int64_t)min(u, p.rows_v - 1) * p.stride + res;
        };
        ItemPos at, nx;
        pos_begin(at);
        float nx_lin, nx_tr, nx_nn;
        {
            int res, block, u;
            const int64_t row = own_row(at, res, block, u);
            nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
        }
        for (; at.w < p.n_items; at = nx) {
            const uint32_t rg = ctrl->range[at.e];
            const int n_lo = (int)(rg & 0xffffu), N = (int)(rg >> 16);
            int res, block, u_own;
            (void)own_row(at, res, block, u_own);
            const bool row_exists = u_own < p.rows_v;
            int my_a, my_n, row_start, row_nnz;
            row_band(p, res, nx_lin, nx_tr, row_exists ? nx_nn : 0.f, my_a, my_n, row_start, row_nnz);
            const int64_t bh = at.bh;
            nx = at;
            pos_next(nx);
            if (nx.w < p.n_items) {
                int r2, b2, u2;
                const int64_t row = own_row(nx, r2, b2, u2);
                nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
            }
            // last step of this item in which some row of this warp has valid columns (-1: none)
            const int hi_tile = warp_max_i(my_n > 0 ? (my_a + my_n + kTile - 1) / kTile : 0);
            const int last_active = min(hi_tile, n_lo + N) - 1 - n_lo;
            PAIR_TRACE(3, 30);
            // row sums of the item (the softmax warps are done with it)
            const int par = n_item & 1, use = n_item >> 1;
            ok = mbar_wait(&ctrl->l_full[par], (uint32_t)use & 1u, status, kErrRowSum);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const float l_sum = ctrl->l_buf[par][t];
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->l_free[par]);
            // This warp's rows of O are final once the PV of its last step with valid columns has
            // completed; later steps of the item (the other tile's) add zeros to them.  A warp
            // without such a step still waits for the item's first PV: that MMA is only issued once
            // every warp has released the previous item's O, so no warp can signal "O read" for this
            // item while that barrier is still collecting the previous item's arrivals.
            const bool have_o = last_active >= 0;
            if (N > 0) {
                ok = event_wait(G0 + max(last_active, 0) + kBufs, kErrEvent);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
            }
            PAIR_TRACE(3, 31);
            // the staging buffer is free once the previous item's store has read it
            if (storer) {
                tma_store_wait_read();
                mbar_arrive(&ctrl->stage_free);
            }
            ok = mbar_wait(&ctrl->stage_free, (uint32_t)n_item & 1u, status, kErrStage);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            {
                const T* vrow = reinterpret_cast<const T*>(p.v) + (bh * p.n_rows + (int64_t)row_start) * D;
                const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t r[64];
                    if (have_o) {  // warp-uniform
                        tmem_ld32(o_addr + half * 64, r);
                        tmem_ld32(o_addr + half * 64 + 32, r + 32);
                        tmem_ld_wait();
                        reg_fence64(r);
                    }
                    if (half == 1 && N > 0) {      // O is in registers: the next item may overwrite it
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(o_free_addr);
                    }
#pragma unroll
                    for (int c2 = 0; c2 < 2; ++c2) {
                        const int ch = half * 2 + c2;      // 32-column chunk of the row
                        uint4 out[4];
                        if (row_nnz > 1 && have_o) {
                            uint32_t* o32 = reinterpret_cast<uint32_t*>(out);
#pragma unroll
                            for (int j = 0; j < 32; j += 2)
                                o32[j >> 1] = pack2<T>(__uint_as_float(r[c2 * 32 + j]) * inv,
                                                       __uint_as_float(r[c2 * 32 + j + 1]) * inv);
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
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->stage_ready);
            if (storer) {
                if (mbar_wait(&ctrl->stage_ready, (uint32_t)n_item & 1u, status, kErrStage)) {
                    if (block * kItemRows + (int)rank * kTile < p.rows_v) {
                        for (int sub = 0; sub < 2; ++sub)
                            tma_store_4d(&tm_o, s_stage + sub * kSubBytes, sub * 64, res,
                                         block * kItemRows + (int)rank * kTile, (int)bh);
                        tma_store_commit();
                    }
                } else {
                    ok = false;
                }
            }
            ok = __all_sync(0xffffffffu, ok);
            PAIR_TRACE(3, 32);
            if (!ok) break;
            G0 += N;
            ++n_item;
        }
        if (storer) tma_store_wait_read();
      }
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
extern "C" void splat_debug_set_pair_trace(void* device_buffer_4x2048_i64) {
    splat::pair::g_trace = reinterpret_cast<long long*>(device_buffer_4x2048_i64);
}
#endif
