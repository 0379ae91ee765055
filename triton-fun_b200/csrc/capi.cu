// Entry points that are not tied to one kernel file: version, status strings and the dispatch of
// the fused attention call between the tensor-core band kernel and the general CUDA-core kernel.
#include "common.cuh"
#include "tc_ptx.cuh"

namespace splat {
int32_t attention_generic(const void* q, const void* k, int64_t ksb, int64_t ksc, int64_t ksk,
                          const void* v, void* o, const float* lin, const float* tr,
                          const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                          float scale, int32_t dtype, float* lse, cudaStream_t st);
// Returns SPLAT_ERR_UNSUPPORTED_SHAPE (and launches nothing) when the problem does not qualify.
int32_t attention_band(const void* q, const void* k, int64_t ksb, int64_t ksc, int64_t ksk,
                       const void* v, void* o, const float* lin, const float* tr,
                       const float* nnzs, int64_t bh, int64_t n_rows, int64_t n_cols, int64_t d,
                       float scale, int32_t dtype, const int32_t* plan, int32_t* status_word,
                       float* lse, cudaStream_t st);
}  // namespace splat

namespace splat {
// One CTA waits, with the same bounded wait the band kernels use, on an mbarrier that nothing ever
// arrives on.  The wait must give up after limit_cycles, record the code and let the kernel end.
__global__ void bounded_wait_selftest_kernel(int32_t* status_word, long long limit_cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        tc::mbar_fence_init();
    }
    __syncthreads();
    const bool ok = tc::mbar_wait(&bar, 0, status_word, 99, limit_cycles);
    if (ok) atomicExch(status_word, -1);   // cannot happen: nobody arrives
}
}  // namespace splat

extern "C" int32_t splat_selftest_bounded_wait(int32_t* status_word, int64_t limit_cycles, void* stream) {
    if (!status_word || limit_cycles < 1 || limit_cycles > 2000000000LL) return SPLAT_ERR_BAD_ARG;
    splat::bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status_word, limit_cycles);
    return splat::launch_status();
}

extern "C" int32_t splat_version(void) { return SPLAT_B200_VERSION; }

extern "C" const char* splat_status_string(int32_t status) {
    switch (status) {
        case SPLAT_OK: return "ok";
        case SPLAT_ERR_BAD_ARG: return "bad argument (null pointer, negative or inconsistent size)";
        case SPLAT_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype";
        case SPLAT_ERR_MISALIGNED: return "pointer or stride is not aligned as the path requires";
        case SPLAT_ERR_LAUNCH: return "CUDA error at kernel launch";
        case SPLAT_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
        case SPLAT_ERR_UNSUPPORTED_SHAPE: return "shape not supported by the requested path";
        case SPLAT_ERR_DRIVER: return "CUDA driver call failed (tensor map encode / entry point)";
        case SPLAT_ERR_NO_DEVICE: return "no CUDA device";
        case SPLAT_ERR_SCRATCH_TOO_SMALL:
            return "problem needs more than the fixed 64 MiB intermediate of splat_attention_noalloc";
        default: return "unknown status";
    }
}

extern "C" int32_t splat_attention_fused_lse(const void* q, const void* k, int64_t k_stride_bh,
                                             int64_t k_stride_col, int64_t k_stride_k, const void* v,
                                             void* o, float* lse, const float* sTod_lin,
                                             const float* sTod_tr, const float* nnzs, int64_t bh,
                                             int64_t n_rows, int64_t n_cols, int64_t d, float scale,
                                             int32_t dtype, int32_t path, const int32_t* plan_i32,
                                             int32_t* status_word, int32_t* path_ran, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (path_ran) *path_ran = SPLAT_PATH_AUTO;   // nothing launched yet
    if (path != SPLAT_PATH_AUTO && path != SPLAT_PATH_GENERIC && path != SPLAT_PATH_BAND)
        return SPLAT_ERR_BAD_ARG;
    if (path != SPLAT_PATH_GENERIC && plan_i32 != nullptr && status_word != nullptr) {
        int32_t rc = splat::attention_band(q, k, k_stride_bh, k_stride_col, k_stride_k, v, o,
                                           sTod_lin, sTod_tr, nnzs, bh, n_rows, n_cols, d, scale,
                                           dtype, plan_i32, status_word, lse, st);
        // Under SPLAT_PATH_AUTO a tensor-core path that does not apply -- shape, alignment of the
        // caller's buffers, or a driver without tensor-map support -- hands over to the general
        // kernel, which takes any operands; asked for explicitly, it reports why it cannot run.
        const bool not_applicable = rc == SPLAT_ERR_UNSUPPORTED_SHAPE || rc == SPLAT_ERR_MISALIGNED ||
                                    rc == SPLAT_ERR_DRIVER;
        if (!not_applicable || path == SPLAT_PATH_BAND) {
            if (rc == SPLAT_OK && path_ran) *path_ran = SPLAT_PATH_BAND;
            return rc;
        }
    } else if (path == SPLAT_PATH_BAND) {
        return SPLAT_ERR_BAD_ARG;
    }
    const int32_t rc = splat::attention_generic(q, k, k_stride_bh, k_stride_col, k_stride_k, v, o,
                                                sTod_lin, sTod_tr, nnzs, bh, n_rows, n_cols, d, scale,
                                                dtype, lse, st);
    if (rc == SPLAT_OK && path_ran && bh > 0 && n_rows > 0) *path_ran = SPLAT_PATH_GENERIC;
    return rc;
}

extern "C" int32_t splat_attention_fused_ex(const void* q, const void* k, int64_t k_stride_bh,
                                            int64_t k_stride_col, int64_t k_stride_k, const void* v,
                                            void* o, const float* sTod_lin, const float* sTod_tr,
                                            const float* nnzs, int64_t bh, int64_t n_rows,
                                            int64_t n_cols, int64_t d, float scale, int32_t dtype,
                                            int32_t path, const int32_t* plan_i32,
                                            int32_t* status_word, int32_t* path_ran, void* stream) {
    return splat_attention_fused_lse(q, k, k_stride_bh, k_stride_col, k_stride_k, v, o, nullptr, sTod_lin,
                                     sTod_tr, nnzs, bh, n_rows, n_cols, d, scale, dtype, path, plan_i32,
                                     status_word, path_ran, stream);
}

extern "C" int32_t splat_attention_fused(const void* q, const void* k, int64_t k_stride_bh,
                                         int64_t k_stride_col, int64_t k_stride_k, const void* v,
                                         void* o, const float* sTod_lin, const float* sTod_tr,
                                         const float* nnzs, int64_t bh, int64_t n_rows,
                                         int64_t n_cols, int64_t d, float scale, int32_t dtype,
                                         int32_t path, const int32_t* plan_i32,
                                         int32_t* status_word, void* stream) {
    return splat_attention_fused_ex(q, k, k_stride_bh, k_stride_col, k_stride_k, v, o, sTod_lin,
                                    sTod_tr, nnzs, bh, n_rows, n_cols, d, scale, dtype, path,
                                    plan_i32, status_word, nullptr, stream);
}
