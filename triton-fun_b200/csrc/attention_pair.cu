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
//     P(G) = exp2(S c - m) softmax warps on their CTA's 128 rows, TWO threads per row: one for the
//                         step's keys 0..63, one for keys 64..127.  Each keeps its own running
//                         maximum and sum (lazy rescale) and stores its 16-bit P over the scores
//                         it consumed
//     O_h += P_h(G) V_h   per key half h: 4 x tcgen05.mma 256x128x16, A = P from each CTA's tensor
//                         memory, B = the value tile (each CTA holds 64 of the 128 value columns)
// The two key halves are two independent online-softmax streams with their own accumulators O_0,
// O_1; the epilogue merges them: O = (a_0 O_0 + a_1 O_1) / (a_0 l_0 + a_1 l_1), a_h = 2^(m_h - m).
// That puts two softmax warps on every scheduler (one's exponentials cover the other's loads,
// maxima and handshakes) without any exchange between the two threads of a row.  Each SM's 512
// tensor-memory columns hold two score buffers (step G uses buffer G mod 2), O_0 and O_1; the
// tensor core runs up to two steps ahead of the softmax warps, also into the next item: issue
// order S(0) S(1), then per step PV(G), S(G+2).  Operand halves are loaded by each CTA for itself
// with plain TMA loads into its own shared memory; the byte counts of both CTAs land on barriers of the even
// CTA, whose MMA warp is the only consumer.
//
// Progress of the tensor core is published as numbered EVENTS: event e is one tcgen05.commit per
// CTA onto barrier e mod 32 of that CTA.  Event G = "S(G) complete", event G + 2 = "PV(G)
// complete" (one commit after PV(G), S(G+2) serves both).  Softmax warps wait for S(G); epilogue
// warps for the PV of their rows' last step; the TMA producers for the event that frees the slot
// they are about to overwrite.  Every role walks the same item list with the per-item (n_lo, N)
// taken from a table in shared memory that each CTA builds from the row metadata at kernel start,
// so no role has to tell another what comes next.
//
// Warps per CTA: 0-3 softmax of keys 0..63, 4-7 softmax of keys 64..127 (never wait for a PV
// except to rescale their O), 8-11 epilogue (merge and normalise O with the maxima and sums the
// softmax warps leave in shared memory, stage, TMA store; this overlaps the next item's softmax),
// 12 TMA producer, 13 MMA issuer (even CTA; the whole warp runs the loop and one elected lane
// issues) and tensor-memory owner (both), 14-15 idle.  Every mbarrier wait is bounded; a role that
// gives up records a code in the status word, the others see the word in their own waits, and
// both CTAs meet at a cluster barrier before tensor memory is released and either CTA leaves.
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
bool make_map_kt(CUtensorMap* map, const void* base, int32_t dtype, int64_t bh, int64_t n_cols,
                 int64_t d);
}

namespace pair {

using namespace tc;
using namespace sm;

constexpr int D = 128;
constexpr int kTile = 128;             // rows per CTA and keys per step
constexpr int kHalf = 64;              // score columns a softmax thread holds at a time
constexpr int kItemRows = 2 * kTile;   // rows per work item (CTA pair)
constexpr int kThreads = 512;          // 16 warps: softmax 0-7, epilogue 8-11, TMA 12, MMA 13, two idle
constexpr int kWarps = kThreads / 32;
constexpr int kEpiWarp = 8;            // warps 8..11
constexpr int kTmaWarp = 12;
constexpr int kMmaWarp = 13;
constexpr int kTmemCols = 512;
constexpr int kBufs = 2;               // score buffers
constexpr int kSlots = 3;              // K slots = V slots (Cursor::slot counts modulo 3)
constexpr int kEvents = 32;            // event barriers: a wait must be issued before its event is 32 events old
constexpr int kMaxEntries = 2048;      // (residue class, row block) combinations the range table holds
constexpr int kSubBytes = kTile * 128;         // 128 rows of one 64-element column chunk
constexpr int kTileBytes = 2 * kSubBytes;      // Q tile / O staging: 128 rows x 128 columns
constexpr int kSlotBytes = 16384;              // K half (64 keys x 128) or V half (128 keys x 64)
constexpr int kKHalfSub = 64 * 128;            // one 64-element chunk of a K half
constexpr uint32_t kOCol = 2 * kTile;          // tensor-memory column of O_0; O_1 follows
constexpr float kRescaleThreshold = 8.0f;

// status-word codes (which wait gave up)
enum : int { kErrQ = 11, kErrKFull = 12, kErrVFull = 13, kErrEvent = 14, kErrPReady = 15,
             kErrOFree = 16, kErrStage = 17, kErrRowSum = 18 };

struct Params {
    const float* lin;
    const float* tr;
    const float* nnzs;
    const void* v;
    const void* q;         // raw operands: only the single score of a row with one non-zero is read
    const void* k;         //   through them (log-sum-exp output)
    float* lse;            // (BH, L) natural-log log-sum-exp of every row, or null
    int32_t* status;
    long long* trace;      // profiling builds only (else null)
    int64_t n_rows;        // L
    int rows_v;            // L / stride: rows of one residue class
    int stride;
    int items_per_class;   // ceil(rows_v / 256)
    int kt_major;          // 1: K is a contiguous (BH, d, L) array (keys innermost); stride 1 only
    int n_entries;         // stride * items_per_class <= kMaxEntries
    int64_t n_items;       // n_entries * bh
    float scale_log2;      // softmax scale * log2(e), > 0
};

struct Control {
    uint64_t ev[kEvents];      // both CTAs: tensor-core progress events
    uint64_t q_full[2];        // even CTA only (as the next four): Q tiles of both CTAs have landed
    uint64_t k_full[kSlots];
    uint64_t v_full[kSlots];
    uint64_t p_ready[kBufs];   // 16 arrivals: the softmax warps of both CTAs
    uint64_t o_free;           // 8 arrivals: O has been read out, the next item may overwrite it
    uint64_t drain;
    uint64_t l_full[2];        // own CTA, 8 arrivals: maxima and sums of an item are in ml_buf (items alternate)
    uint64_t l_free[2];        // own CTA, 4 arrivals: the epilogue warps have read them
    uint64_t stage_free;       // own CTA: the previous TMA store has read the output staging buffer
    uint64_t stage_ready;      // own CTA, 4 arrivals: the epilogue warps have written their rows
    uint32_t tmem_base;
    int32_t abort_at_entry;
    float2 ml_buf[2][2][kTile];    // [item parity][key half][row] = (running maximum, sum)
    uint32_t range[kMaxEntries];   // per (class, row block): n_lo | N << 16
};

struct Layout {
    static constexpr int kQOff = 0;                               // two Q tiles (items alternate)
    static constexpr int kStageOff = 2 * kTileBytes;              // output staging
    static constexpr int kKOff = kStageOff + kTileBytes;
    static constexpr int kVOff = kKOff + kSlots * kSlotBytes;
    static constexpr int kCtrlOff = kVOff + kSlots * kSlotBytes;
    static constexpr int kSmemBytes = kCtrlOff + (int)sizeof(Control) + 1024;   // + alignment slack
};

#ifdef SPLAT_PAIR_TRACE
#define PAIR_TRACE(role, tag)                                                                     \
    do {                                                                                          \
        if (trace_on && lane == 0 && (warp == 0 || warp == 8 || warp >= 12) && trace_n < 2048) \
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
    int slot;         // G mod kSlots
    int block, res;
    bool valid;
};

// The item list of one CTA pair and its step ranges.  Built inside each role (from special
// registers, so the compiler keeps it there) rather than once per thread: values shared by all
// roles would have to live in registers across the roles' different register budgets.
struct Walk {
    int64_t first, step, step_bh, n_items;
    int step_e, n_entries, items_per_class;
    const uint32_t* range;

    __device__ __forceinline__ void begin(ItemPos& at) const {
        at.w = first;
        at.e = (int)(first % n_entries);
        at.bh = first / n_entries;
    }
    // w -> w + step without 64-bit divisions
    __device__ __forceinline__ void next(ItemPos& at) const {
        at.w += step;
        at.e += step_e;
        at.bh += step_bh;
        if (at.e >= n_entries) { at.e -= n_entries; ++at.bh; }
    }
    // item at c.at -> class, block and range; false when the item has no steps
    __device__ __forceinline__ bool load(Cursor& c) const {
        c.res = c.at.e / items_per_class;
        c.block = c.at.e - c.res * items_per_class;
        const uint32_t r = range[c.at.e];
        c.n_lo = (int)(r & 0xffffu);
        c.N = (int)(r >> 16);
        return c.N > 0;
    }
    __device__ __forceinline__ void cursor_begin(Cursor& c) const {
        begin(c.at);
        c.G = 0; c.i = 0; c.jq = 0; c.slot = 0;
        c.valid = false;
        for (; c.at.w < n_items; next(c.at))
            if (load(c)) { c.valid = true; break; }
    }
    __device__ __forceinline__ void cursor_next(Cursor& c) const {
        ++c.G;
        c.slot = c.slot == 2 ? 0 : c.slot + 1;
        if (++c.i < c.N) return;
        c.i = 0; ++c.jq;
        c.valid = false;
        for (next(c.at); c.at.w < n_items; next(c.at))
            if (load(c)) { c.valid = true; break; }
    }
};

__device__ __forceinline__ void spin_cycles(long long n) {
    const long long t0 = clock64();
    while (clock64() - t0 < n) { }
}

// x[0..64) scores -> packed 16-bit probabilities exp2(s*c - m) in x[0..32); row sums into acc0/acc1.
template <typename T>
__device__ __forceinline__ void exp_half(uint32_t* x, float2 sc2, float2 nm2, float2& acc0, float2& acc1) {
#pragma unroll
    for (int j = 0; j < kHalf; j += 8) {
        float2 a[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            a[c] = fma2(make_float2(__uint_as_float(x[j + 2 * c]), __uint_as_float(x[j + 2 * c + 1])), sc2, nm2);
            a[c].x = ex2(a[c].x);
            a[c].y = ex2(a[c].y);
        }
        acc0 = add2(acc0, add2(a[0], a[1]));
        acc1 = add2(acc1, add2(a[2], a[3]));
#pragma unroll
        for (int c = 0; c < 4; ++c) x[(j >> 1) + c] = pack2<T>(a[c].x, a[c].y);
    }
}

// Band edge: columns outside [v_lo, v_lo + width) (relative to x[0]) become -inf; then the row
// maximum.  One unsigned comparison per column covers both ends.
__device__ __forceinline__ float masked_max(uint32_t* x, int v_lo, int width, bool edge) {
    if (edge) {
#pragma unroll
        for (int j = 0; j < kHalf; ++j)
            x[j] = (uint32_t)(j - v_lo) < (uint32_t)width ? x[j] : 0xff800000u;
    }
    float mx[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) mx[c] = fmaxf(__uint_as_float(x[2 * c]), __uint_as_float(x[2 * c + 1]));
#pragma unroll
    for (int j = 16; j < kHalf; j += 16) {      // eight independent chains of 3-input max
#pragma unroll
        for (int c = 0; c < 8; ++c)
            mx[c] = fmax3(mx[c], __uint_as_float(x[j + 2 * c]), __uint_as_float(x[j + 2 * c + 1]));
    }
    return fmaxf(fmax3(mx[0], mx[1], mx[2]), fmax3(fmax3(mx[3], mx[4], mx[5]), mx[6], mx[7]));
}

// Rare paths of the lazy rescale, kept out of line so that the softmax loop stays small.
// O rows of this thread (128 fp32 columns at o_addr) *= corr.
__device__ __noinline__ void rescale_o(uint32_t o_addr, float corr) {
#pragma unroll 1
    for (int ch = 0; ch < D / 16; ++ch) {
        uint32_t o[16];
        tmem_ld16(o_addr + ch * 16, o);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
        tmem_st16(o_addr + ch * 16, o);
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
#ifdef SPLAT_PAIR_TRACE
    const bool trace_on = p.trace != nullptr && cluster_id_x() == cluster_count_x() / 2 && cluster_ctarank() == 0;
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
            mbar_init(&ctrl->l_full[i], 8);
            mbar_init(&ctrl->l_free[i], 4);
        }
        for (int i = 0; i < kSlots; ++i) {
            mbar_init(&ctrl->k_full[i], 1);
            mbar_init(&ctrl->v_full[i], 1);
        }
        for (int i = 0; i < kBufs; ++i) mbar_init(&ctrl->p_ready[i], 16);
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
    // both CTAs read the same global word; a differing view could only come from a concurrent
    // writer, i.e. a kernel that is giving up right now, and then the bounded waits end this one too
    const bool run = ctrl->abort_at_entry == 0;

    // shared::cluster addresses of the even CTA's barriers (valid from either CTA)
    auto leader_addr = [&](uint64_t* bar) { return map_to_cta(smem_u32(bar), 0); };
    auto event_wait = [&](int64_t e, int code) {
        return mbar_wait(&ctrl->ev[e & (kEvents - 1)], (uint32_t)(e >> 5) & 1u, status, code);
    };
    auto make_walk = [&]() {
        Walk wk;
        wk.first = cluster_id_x();
        wk.step = cluster_count_x();
        wk.n_items = p.n_items;
        wk.n_entries = p.n_entries;
        wk.items_per_class = p.items_per_class;
        wk.step_e = (int)(wk.step % p.n_entries);
        wk.step_bh = wk.step / p.n_entries;
        wk.range = ctrl->range;
        return wk;
    };

    if (run && warp == kTmaWarp) {
        // ------------------------------------------------------------------ TMA producer
        // Loads follow the order in which the tensor core consumes them: K(0) K(1) K(2), then
        // V(G), K(G+3) for every step, with the Q tile of an item just before its first K tile.
        // This CTA loads keys [64 rank, +64) of every K tile and value columns [64 rank, +64) of
        // every V tile.
        if (lane == 0) {
            const uint32_t rank = cluster_ctarank();
            const Walk wk = make_walk();
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
                const int slot = c.slot;
                if (!slot_wait(c.G - kSlots)) return false;      // S(G-3) has read this slot
                if (rank == 0) mbar_arrive_expect_tx(&ctrl->k_full[slot], 2 * kSlotBytes);
                const uint32_t bar = leader_addr(&ctrl->k_full[slot]);
                if (p.kt_major)      // one [d][64 keys] block (see attention_band.cu on K layouts)
                    tma_load_4d_pair(s_k + slot * kSlotBytes, &tm_k, bar, (c.n_lo + c.i) * kTile + (int)rank * 64,
                                     0, (int)c.at.bh, 0);
                else
                    for (int sub = 0; sub < 2; ++sub)
                        tma_load_4d_pair(s_k + slot * kSlotBytes + sub * kKHalfSub, &tm_k, bar, sub * 64, c.res,
                                         (c.n_lo + c.i) * kTile + (int)rank * 64, (int)c.at.bh);
                PAIR_TRACE(2, 22);
                return true;
            };
            auto load_v = [&](const Cursor& c) {
                const int slot = c.slot;
                // PV(G-3) has read this slot: event (G-3) + kBufs
                if (c.G >= kSlots && !slot_wait(c.G - kSlots + kBufs)) return false;
                if (rank == 0) mbar_arrive_expect_tx(&ctrl->v_full[slot], 2 * kSlotBytes);
                tma_load_4d_pair(s_v + slot * kSlotBytes, &tm_v, leader_addr(&ctrl->v_full[slot]),
                                 (int)rank * 64, c.res, (c.n_lo + c.i) * kTile, (int)c.at.bh);
                PAIR_TRACE(2, 23);
                return true;
            };
            Cursor kc, vc;
            wk.cursor_begin(kc);
            wk.cursor_begin(vc);
            bool ok = true;
            for (int t = 0; t < kSlots && kc.valid && ok; ++t) {
                ok = load_k(kc);
                wk.cursor_next(kc);
            }
            while (vc.valid && ok) {
                ok = load_v(vc);
                wk.cursor_next(vc);
                if (ok && kc.valid) {
                    ok = load_k(kc);
                    wk.cursor_next(kc);
                }
            }
            // giving up: copies already issued may still be landing (some counted on the other
            // CTA's barriers); let them finish before either CTA can leave
            if (!ok) spin_cycles(400000);
        }
    } else if (run && warp == kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer (even CTA)
        // The whole warp walks the loop on warp-uniform values; one elected lane issues.
        if (cluster_ctarank() == 0) {
            const Walk wk = make_walk();
            const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            const uint32_t idesc_qk = instr_desc_f16(fmt, 2 * kTile, kTile, p.kt_major ? 1u : 0u);
            constexpr uint32_t idesc_pv = instr_desc_f16(fmt, 2 * kTile, D, 1);
            const bool lead = elect_one();
            const uint32_t q_addr = smem_u32(s_q), k_addr = smem_u32(s_k), v_addr = smem_u32(s_v);
            const uint32_t ev_own = smem_u32(&ctrl->ev[0]);
            const uint32_t ev_peer = map_to_cta(ev_own, 1);
            const uint32_t o_tmem = tmem_base + kOCol;
            uint32_t k_ph = 0, v_ph = 0, p_ph = 0;     // one phase bit per slot / buffer
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
            // S of the step at cursor c, into score buffer G mod 2
            auto issue_s = [&](const Cursor& c) {
                const int qb = c.jq & 1;
                if (c.i == 0 && !wait_all(&ctrl->q_full[qb], (uint32_t)(c.jq >> 1) & 1u, kErrQ)) return false;
                const int slot = c.slot;
                const bool r = wait_all(&ctrl->k_full[slot], (k_ph >> slot) & 1u, kErrKFull);
                k_ph ^= 1u << slot;
                if (!r) return false;
                tc_fence_after_sync();
                const uint32_t q_base = q_addr + qb * kTileBytes;
                const uint32_t b_base = k_addr + slot * kSlotBytes;
                const uint32_t d_tmem = tmem_base + (uint32_t)(c.G & 1) * kTile;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t da = smem_desc_sw128(q_base + (kk >> 2) * kSubBytes + (kk & 3) * 32, 16, 1024);
                    const uint64_t db = p.kt_major
                        ? smem_desc_sw128(b_base + kk * 2048, kSlotBytes, 1024)
                        : smem_desc_sw128(b_base + (kk >> 2) * kKHalfSub + (kk & 3) * 32, 16, 1024);
                    if (lead) mma_ss_pair(d_tmem, da, db, idesc_qk, kk > 0);
                }
                return true;
            };
            Cursor sc, pc;
            wk.cursor_begin(sc);
            wk.cursor_begin(pc);
            for (int t = 0; t < kBufs && ok; ++t) {
                if (sc.valid) {
                    ok = issue_s(sc);
                    wk.cursor_next(sc);
                }
                if (ok) commit_event(t);
            }
            while (pc.valid && ok) {
                const int slot = pc.slot;
                const int buf = (int)(pc.G & 1);
                ok = wait_all(&ctrl->v_full[slot], (v_ph >> slot) & 1u, kErrVFull);
                v_ph ^= 1u << slot;
                if (!ok) break;
                PAIR_TRACE(1, 10);
                ok = wait_all(&ctrl->p_ready[buf], (p_ph >> buf) & 1u, kErrPReady);
                p_ph ^= 1u << buf;
                if (!ok) break;
                if (pc.i == 0 && pc.jq > 0) {      // the previous item's O has been read out
                    ok = wait_all(&ctrl->o_free, (uint32_t)(pc.jq - 1) & 1u, kErrOFree);
                    if (!ok) break;
                }
                tc_fence_after_sync();
                PAIR_TRACE(1, 11);
                // O_h += P_h V_h: the P of key half h is packed in the first 32 of the 64 score
                // columns its threads consumed
                {
                    const uint32_t b_base = v_addr + slot * kSlotBytes;
                    const uint32_t a_tmem = tmem_base + buf * kTile;
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk) {
                        const int h = kk >> 2;
                        const uint64_t db = smem_desc_sw128(b_base + kk * 2048, kSlotBytes, 1024);
                        if (lead) mma_ts_pair(o_tmem + h * D, a_tmem + h * kHalf + (kk & 3) * 8, db, idesc_pv,
                                              (pc.i > 0 || (kk & 3) > 0) ? 1u : 0u);
                    }
                }
                if (sc.valid) {                    // S(G+2) into the buffer PV(G) has just consumed
                    ok = issue_s(sc);
                    if (!ok) break;
                    wk.cursor_next(sc);
                }
                commit_event(pc.G + kBufs);
                PAIR_TRACE(1, 12);
                wk.cursor_next(pc);
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
    } else if (run && warp < kEpiWarp) {
        // ------------------------------------------------------------------ softmax
        // Thread = (row, key half): 64 of the 128 scores of every step.
        const uint32_t rank = cluster_ctarank();
        const Walk wk = make_walk();
        const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
        const int h = warp >> 2;                     // key half
        const int t = (warp & 3) * 32 + lane;        // row of this thread within the CTA's tile
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t o_addr = lane_addr + kOCol + h * D;
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
        wk.begin(at);
        float nx_lin, nx_tr, nx_nn;
        {
            int res, u;
            const int64_t row = own_row(at, res, u);
            nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
        }
        for (; at.w < wk.n_items; at = nx) {
            const uint32_t rg = ctrl->range[at.e];
            const int n_lo = (int)(rg & 0xffffu), N = (int)(rg >> 16);
            int res, u_own;
            (void)own_row(at, res, u_own);
            int my_a, my_n, row_start, row_nnz;
            row_band(p, res, nx_lin, nx_tr, u_own < p.rows_v ? nx_nn : 0.f, my_a, my_n, row_start, row_nnz);
            nx = at;
            wk.next(nx);
            if (nx.w < wk.n_items) {      // next item's row: in flight during this item's steps
                int r2, u2;
                const int64_t row = own_row(nx, r2, u2);
                nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
            }
            float m_used = -INFINITY, l_sum = 0.f;
            int pending = -1;        // score buffer whose P has been stored but not yet handed over
            bool started = false;    // an earlier step of this item had valid columns for this warp: O_h is live
            const int v_lo0 = my_a - n_lo * kTile - h * kHalf;

            // P of the pending buffer is complete in tensor memory: tell the MMA warp
            auto hand_over = [&]() {
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(p_ready_addr + pending * 8);
                pending = -1;
            };

            for (int i = 0; i < N; ++i) {
                const int64_t G = G0 + i;
                const int buf = (int)(G & 1);
                const uint32_t s_addr = lane_addr + buf * kTile + h * kHalf;   // this thread's 64 scores
                // valid columns [v_lo, v_lo + my_n) of the row, relative to this half's first key
                const int v_lo = v_lo0 - i * kTile;
                const bool warp_in = __any_sync(0xffffffffu, my_n > 0 && v_lo < kHalf && v_lo + my_n > 0);
                const bool edge = !__all_sync(0xffffffffu, v_lo <= 0 && v_lo + my_n >= kHalf);
                PAIR_TRACE(0, 1);
                // The previous step's P is normally handed over a little later, under this step's
                // load and maximum; but if this step's scores are not there yet, the tensor core is
                // waiting for that very P (or for work that follows it): hand it over first.
                if (!__all_sync(0xffffffffu, mbar_test_wait(&ctrl->ev[G & (kEvents - 1)], (uint32_t)(G >> 5) & 1u))) {
                    if (pending >= 0) hand_over();
                    ok = event_wait(G, kErrEvent);        // S(G) complete (and PV(G-2): the buffer is free)
                    ok = __all_sync(0xffffffffu, ok);     // keep the warp together for the aligned tcgen05 ops
                    if (!ok) break;
                }
                tc_fence_after_sync();
                PAIR_TRACE(0, 2);
                uint32_t r[kHalf];
                if (!warp_in) {
                    // none of this warp's rows has a valid column here (another warp's does): the
                    // pair MMA still multiplies these rows, so P must be zero
                    if (pending >= 0) hand_over();
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0u;
                    tmem_st32(s_addr, r);
                    pending = buf;
                    continue;
                }
                tmem_ld32(s_addr, r);
                tmem_ld32(s_addr + 32, r + 32);
                tmem_ld_wait();
                PAIR_TRACE(0, 3);
                const float mt = masked_max(r, v_lo, my_n, edge);
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
                // lazy rescale of this half's accumulator (rare): some row's maximum moved by more
                // than 2^8.  PV(G-1) may still be running: wait for its event first.
                if (started && __any_sync(0xffffffffu, need)) {
                    ok = event_wait(G - 1 + kBufs, kErrEvent);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    rescale_o(o_addr, corr);
                }
                // probabilities, row sum, 16-bit pack in place
                const float2 nm2 = make_float2(-m_eff, -m_eff);
                float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
                exp_half<T>(r, sc2, nm2, acc0, acc1);
                l_sum += (acc0.x + acc0.y) + (acc1.x + acc1.y);
                tmem_st32(s_addr, r);          // P: 32 packed columns over the consumed scores
                pending = buf;
                started = true;
                PAIR_TRACE(0, 5);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (pending >= 0) hand_over();
            PAIR_TRACE(0, 6);
            // running maximum and sum to the epilogue warps; the buffer was last used two items ago
            const int par = n_item & 1, use = n_item >> 1;
            if (use > 0) {
                ok = mbar_wait(&ctrl->l_free[par], (uint32_t)(use - 1) & 1u, status, kErrRowSum);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            ctrl->ml_buf[par][h][t] = make_float2(m_used, l_sum);
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->l_full[par]);
            PAIR_TRACE(0, 7);
            G0 += N;
            ++n_item;
        }
    } else if (run && warp < kTmaWarp) {
        // ------------------------------------------------------------------ epilogue
        // (a_0 O_0 + a_1 O_1) / (a_0 l_0 + a_1 l_1) for band rows, V[start] for single-element
        // rows, zero otherwise.  Rows are staged in shared memory in the 128-byte-swizzled tile
        // layout and leave through one tiled TMA store per 64-column half (rows past the end of the
        // class are clipped by the tensor map).
        const int ew = warp - kEpiWarp;
        const uint32_t rank = cluster_ctarank();
        const Walk wk = make_walk();
        const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctrl->tmem_base);
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
        wk.begin(at);
        float nx_lin, nx_tr, nx_nn;
        {
            int res, block, u;
            const int64_t row = own_row(at, res, block, u);
            nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
        }
        for (; at.w < wk.n_items; at = nx) {
            const uint32_t rg = ctrl->range[at.e];
            const int n_lo = (int)(rg & 0xffffu), N = (int)(rg >> 16);
            int res, block, u_own;
            (void)own_row(at, res, block, u_own);
            const bool row_exists = u_own < p.rows_v;
            int my_a, my_n, row_start, row_nnz;
            row_band(p, res, nx_lin, nx_tr, row_exists ? nx_nn : 0.f, my_a, my_n, row_start, row_nnz);
            const int64_t bh = at.bh;
            nx = at;
            wk.next(nx);
            if (nx.w < wk.n_items) {
                int r2, b2, u2;
                const int64_t row = own_row(nx, r2, b2, u2);
                nx_lin = __ldg(p.lin + row); nx_tr = __ldg(p.tr + row); nx_nn = __ldg(p.nnzs + row);
            }
            // last step of this item in which some row of this warp has valid columns (-1: none)
            const int hi_tile = warp_max_i(my_n > 0 ? (my_a + my_n + kTile - 1) / kTile : 0);
            const int last_active = min(hi_tile, n_lo + N) - 1 - n_lo;
            PAIR_TRACE(3, 30);
            // maxima and sums of the item (the softmax warps are done with it)
            const int par = n_item & 1, use = n_item >> 1;
            ok = mbar_wait(&ctrl->l_full[par], (uint32_t)use & 1u, status, kErrRowSum);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const float2 ml0 = ctrl->ml_buf[par][0][t], ml1 = ctrl->ml_buf[par][1][t];
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->l_free[par]);
            // weights of the two key halves: a_h / (a_0 l_0 + a_1 l_1)
            const float m = fmaxf(ml0.x, ml1.x);
            const float a0 = ml0.x == -INFINITY ? 0.f : ex2(ml0.x - m);
            const float a1 = ml1.x == -INFINITY ? 0.f : ex2(ml1.x - m);
            const float l_sum = a0 * ml0.y + a1 * ml1.y;
            const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
            const float w0 = a0 * inv, w1 = a1 * inv;
            if (p.lse != nullptr && row_exists) {
                // band rows from the merged maximum and sum; a row with one non-zero from its single
                // score (outside the band, read from the raw operands); -inf without non-zeros
                const int64_t row_real = (int64_t)u_own * p.stride + res;
                float val = -INFINITY;
                if (row_nnz > 1) {
                    val = lse_from_log2(m, l_sum);
                } else if (row_nnz == 1) {
                    const T* qr = reinterpret_cast<const T*>(p.q) + (bh * p.n_rows + row_real) * D;
                    const T* kb = reinterpret_cast<const T*>(p.k);
                    const float s = p.kt_major ? dot_strided<T>(qr, kb + bh * p.n_rows * D + row_start, p.n_rows, D)
                                               : dot_strided<T>(qr, kb + (bh * p.n_rows + row_start) * D, 1, D);
                    val = s * p.scale_log2 * kLn2;
                }
                p.lse[bh * p.n_rows + row_real] = val;
            }
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
            // O out of tensor memory first (merged, normalised, packed to 16 bits: 64 registers),
            // so that the next item's first PV, which overwrites O, waits as little as possible
            uint32_t packed[D / 2];
            if (have_o) {  // warp-uniform
#pragma unroll
                for (int ch = 0; ch < D / 16; ++ch) {      // 16-column chunk of the row
                    uint32_t r0[16], r1[16];
                    tmem_ld16(o_addr + ch * 16, r0);
                    tmem_ld16(o_addr + D + ch * 16, r1);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j += 2)
                        packed[ch * 8 + (j >> 1)] = pack2<T>(
                            __uint_as_float(r0[j]) * w0 + __uint_as_float(r1[j]) * w1,
                            __uint_as_float(r0[j + 1]) * w0 + __uint_as_float(r1[j + 1]) * w1);
                }
            }
            if (N > 0) {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(o_free_addr);
            }
            PAIR_TRACE(3, 33);
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
#pragma unroll
                for (int ch = 0; ch < D / 32; ++ch) {
                    uint4 out[4];
                    if (row_nnz > 1 && have_o) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4)
                            out[q4] = make_uint4(packed[ch * 16 + q4 * 4], packed[ch * 16 + q4 * 4 + 1],
                                                 packed[ch * 16 + q4 * 4 + 2], packed[ch * 16 + q4 * 4 + 3]);
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

    // ------------------------------------------------------------------ exit
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();      // nothing of either CTA is in flight towards the other any more
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc_pair(ctrl->tmem_base, kTmemCols);
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
int32_t attention_pair(const void* q, const void* k, int kt_major, const void* v, void* o,
                       const float* lin, const float* tr, const float* nnzs, int64_t bh, int64_t n_rows,
                       int64_t stride, float scale, int32_t dtype, int32_t* status_word, int max_pairs,
                       float* lse, cudaStream_t st) {
    const int64_t d = pair::D;
    const int64_t rows_v = n_rows / stride;
    const int64_t items_per_class = (rows_v + pair::kItemRows - 1) / pair::kItemRows;
    if (n_rows > (1ll << 22) || items_per_class * stride > pair::kMaxEntries)
        return SPLAT_ERR_UNSUPPORTED_SHAPE;
    CUtensorMap mq, mk, mv, mo;
    if (!band::make_map(&mq, q, dtype, bh, n_rows, d, stride, pair::kTile) ||
        !(kt_major ? band::make_map_kt(&mk, k, dtype, bh, n_rows, d)
                   : band::make_map(&mk, k, dtype, bh, n_rows, d, stride, 64)) ||
        !band::make_map(&mv, v, dtype, bh, n_rows, d, stride, pair::kTile) ||
        !band::make_map(&mo, o, dtype, bh, n_rows, d, stride, pair::kTile))
        return SPLAT_ERR_DRIVER;
    pair::Params prm;
    prm.lin = lin; prm.tr = tr; prm.nnzs = nnzs; prm.v = v; prm.status = status_word;
    prm.q = q; prm.k = k; prm.lse = lse;
    prm.trace = pair::g_trace;
    prm.kt_major = kt_major;
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
