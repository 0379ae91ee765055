/*
 * C restatement of the reference's three kernels over ACSR, for CPU timing and as a second checker.
 *
 * TEST INFRASTRUCTURE ONLY: used by tests/, by the smoke check and by the CPU-baseline legs of the
 * benchmark.  The shipped library never links or loads this file.
 *
 * What each function follows (paths inside the reference project):
 *   oracle_sddmm ..... SPLAT/r_sddmm.py:16-115   S[i][j] = sum_k Q[i][k] * Kt[k][col(i,j)], fp32
 *                      accumulation, j < nnz_i; layout (BH, L, T)
 *   oracle_softmax ... SPLAT/r_softmax.py:17-59  max-subtracted softmax over the first nnz_i slots
 *                      (the reference has no scale; scale = 1 reproduces it)
 *   oracle_spmm ...... SPLAT/r_spmm.py:14-126    O[i][c] = sum_j P[i][j] * V[col(i,j)][c]
 *   oracle_attention . SPLAT/r_attention.py:77-100  the three in sequence, S and P materialised
 * with col(i,j) = start_i + j*stride_i (integers recovered from the float32 metadata by the
 * caller, see oracle/acsr_oracle.py:affine_ints).  Unlike the reference kernels these loops cover
 * every row and the whole span of every row (the reference kernels' index defects are not
 * reproduced; see the fixtures in tests/golden for where the two agree).
 *
 * Threads: POSIX threads over (batch*head, row); SPLAT_ORACLE_THREADS or oracle_set_num_threads
 * override the default of one thread per online core.
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <unistd.h>

/* ---- a minimal parallel-for over (batch*head, row) pairs with POSIX threads ------------------ */
static int g_threads = 0;

int oracle_num_threads(void) {
    if (g_threads <= 0) {
        const char* e = getenv("SPLAT_ORACLE_THREADS");
        long n = e ? atol(e) : sysconf(_SC_NPROCESSORS_ONLN);
        g_threads = n < 1 ? 1 : (n > 256 ? 256 : (int)n);
    }
    return g_threads;
}
void oracle_set_num_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }

typedef void (*row_fn)(void* ctx, int64_t bh, int64_t i);
typedef struct { row_fn fn; void* ctx; int64_t L, begin, end; } job_t;

static void* worker(void* arg) {
    job_t* j = (job_t*)arg;
    for (int64_t r = j->begin; r < j->end; ++r) j->fn(j->ctx, r / j->L, r % j->L);
    return NULL;
}

static void parallel_rows(row_fn fn, void* ctx, int64_t BH, int64_t L) {
    const int64_t total = BH * L;
    int nt = oracle_num_threads();
    if (nt > total) nt = total > 0 ? (int)total : 1;
    pthread_t tid[256];
    job_t jobs[256];
    for (int t = 0; t < nt; ++t) {
        jobs[t].fn = fn; jobs[t].ctx = ctx; jobs[t].L = L;
        jobs[t].begin = total * t / nt; jobs[t].end = total * (t + 1) / nt;
        if (t > 0) pthread_create(&tid[t], NULL, worker, &jobs[t]);
    }
    worker(&jobs[0]);
    for (int t = 1; t < nt; ++t) pthread_join(tid[t], NULL);
}

/* ---- SDDMM ---------------------------------------------------------------------------------- */
typedef struct {
    const float *q, *kt; int64_t ks_bh, ks_col, ks_k; float* s;
    const int32_t *start, *stride, *nnz; int64_t L, d, T;
} sddmm_t;

static void sddmm_row(void* c, int64_t bh, int64_t i) {
    const sddmm_t* a = (const sddmm_t*)c;
    const float* qi = a->q + (bh * a->L + i) * a->d;
    float* si = a->s + (bh * a->L + i) * a->T;
    const float* kb = a->kt + bh * a->ks_bh;
    for (int64_t j = 0; j < a->T; ++j) {
        float acc = 0.f;
        if (j < a->nnz[i]) {
            const float* kc = kb + ((int64_t)a->start[i] + j * a->stride[i]) * a->ks_col;
            if (a->ks_k == 1)
                for (int64_t k = 0; k < a->d; ++k) acc += qi[k] * kc[k];
            else
                for (int64_t k = 0; k < a->d; ++k) acc += qi[k] * kc[k * a->ks_k];
        }
        si[j] = acc;
    }
}

/* kt is addressed as kt[bh*ks_bh + col*ks_col + k*ks_k] (contiguous K^T: ks_col = 1, ks_k = Lk). */
void oracle_sddmm(const float* q, const float* kt, int64_t ks_bh, int64_t ks_col, int64_t ks_k,
                  float* s, const int32_t* start, const int32_t* stride, const int32_t* nnz,
                  int64_t BH, int64_t L, int64_t d, int64_t T) {
    sddmm_t a = {q, kt, ks_bh, ks_col, ks_k, s, start, stride, nnz, L, d, T};
    parallel_rows(sddmm_row, &a, BH, L);
}

/* ---- softmax -------------------------------------------------------------------------------- */
typedef struct { const float* s; float* p; const int32_t* nnz; int64_t L, T; float scale; } softmax_t;

static void softmax_row(void* c, int64_t bh, int64_t i) {
    const softmax_t* a = (const softmax_t*)c;
    const float* si = a->s + (bh * a->L + i) * a->T;
    float* pi = a->p + (bh * a->L + i) * a->T;
    const int64_t n = a->nnz[i];
    float m = -INFINITY;
    for (int64_t j = 0; j < n; ++j) m = fmaxf(m, si[j] * a->scale);
    float sum = 0.f;
    for (int64_t j = 0; j < n; ++j) { pi[j] = expf(si[j] * a->scale - m); sum += pi[j]; }
    for (int64_t j = 0; j < n; ++j) pi[j] /= sum;
    for (int64_t j = n; j < a->T; ++j) pi[j] = 0.f;
}

void oracle_softmax(const float* s, float* p, const int32_t* nnz, int64_t BH, int64_t L, int64_t T,
                    float scale) {
    softmax_t a = {s, p, nnz, L, T, scale};
    parallel_rows(softmax_row, &a, BH, L);
}

/* ---- SpMM ----------------------------------------------------------------------------------- */
typedef struct {
    const float *p, *v; float* o; const int32_t *start, *stride, *nnz; int64_t L, Lk, d, T;
} spmm_t;

static void spmm_row(void* c, int64_t bh, int64_t i) {
    const spmm_t* a = (const spmm_t*)c;
    const float* pi = a->p + (bh * a->L + i) * a->T;
    float* oi = a->o + (bh * a->L + i) * a->d;
    for (int64_t x = 0; x < a->d; ++x) oi[x] = 0.f;
    for (int64_t j = 0; j < a->nnz[i]; ++j) {
        const float* vr = a->v + (bh * a->Lk + (int64_t)a->start[i] + j * a->stride[i]) * a->d;
        const float pj = pi[j];
        for (int64_t x = 0; x < a->d; ++x) oi[x] += pj * vr[x];
    }
}

void oracle_spmm(const float* p, const float* v, float* o, const int32_t* start,
                 const int32_t* stride, const int32_t* nnz, int64_t BH, int64_t L, int64_t Lk,
                 int64_t d, int64_t T) {
    spmm_t a = {p, v, o, start, stride, nnz, L, Lk, d, T};
    parallel_rows(spmm_row, &a, BH, L);
}

void oracle_attention(const float* q, const float* kt, int64_t ks_bh, int64_t ks_col, int64_t ks_k,
                      const float* v, float* o, float* s_scratch, float* p_scratch,
                      const int32_t* start, const int32_t* stride, const int32_t* nnz, int64_t BH,
                      int64_t L, int64_t d, int64_t T, float scale) {
    oracle_sddmm(q, kt, ks_bh, ks_col, ks_k, s_scratch, start, stride, nnz, BH, L, d, T);
    oracle_softmax(s_scratch, p_scratch, nnz, BH, L, T, scale);
    oracle_spmm(p_scratch, v, o, start, stride, nnz, BH, L, L, d, T);
}
