// splat_attention_noalloc: the SDDMM -> softmax -> SpMM chain for callers that cannot allocate.
//
// The three-launch chain needs one intermediate buffer, the (BH, L, trailing_dim) score /
// probability array.  Normally the caller owns it (the reference's preambles allocate it with
// torch).  Some callers cannot do that: code that runs after its host application has frozen its
// memory pool, plug-ins that are handed input and output buffers but have no allocator of their
// own, and anything that must stay away from cudaMalloc because that call synchronises the whole
// device.  For them this file keeps the intermediate in a fixed device array that is part of the
// library image.
#include <mutex>

#include "common.cuh"

// SPLAT_NOALLOC_SCRATCH_BYTES (splat_b200.h, 64 MiB) is the size of the built-in intermediate
// buffer.  Every GPU on which this library is used holds this much memory from the first use until
// the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SPLAT_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices];
bool g_scratch_known[kMaxDevices];

// Device address of the array on the CURRENT device.  In host code the array's name is only a
// handle; the address a kernel can use has to be asked for, once per device.
int32_t scratch_on_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return SPLAT_ERR_NO_DEVICE;
    if (dev < 0 || dev >= kMaxDevices) return SPLAT_ERR_UNSUPPORTED_SHAPE;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_known[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return SPLAT_ERR_DRIVER;
        }
        g_scratch_addr[dev] = p;
        g_scratch_known[dev] = true;
    }
    *out = g_scratch_addr[dev];
    return SPLAT_OK;
}
}  // namespace

// O = softmax(scale * S) V with S = Q K^T at the ACSR non-zeros, as three kernels (the same ones
// splat_sddmm / splat_softmax / splat_spmm launch) with the intermediate in the built-in array.
//
//  * Allocates nothing: no cudaMalloc / cudaFree, no library call that allocates.
//  * Limit: bh * n_rows * trailing_dim * sizeof(element) must not exceed
//    SPLAT_NOALLOC_SCRATCH_BYTES (64 MiB); larger problems get SPLAT_ERR_SCRATCH_TOO_SMALL and
//    nothing is launched.  Split the batch*head axis to stay below it.
//  * The first call on each device looks up the array's device address (and makes the driver load
//    the array on that device).  Make that first call outside any stream capture.
//  * All calls on one device share the one array.  Calls that may overlap on the GPU (different
//    streams, or different host threads on different streams) race on it; keep calls that use this
//    entry point on one stream, or order them yourself.
//  * The array keeps whatever the previous call left there.  Nothing has to start at zero: the
//    first kernel writes every slot (padding included) that the later kernels read.
extern "C" int32_t splat_attention_noalloc(const void* q, const void* k, int64_t k_stride_bh,
                                           int64_t k_stride_col, int64_t k_stride_k, const void* v,
                                           void* o, const float* sTod_lin, const float* sTod_tr,
                                           const float* nnzs, int64_t bh, int64_t n_rows,
                                           int64_t n_cols, int64_t d, int64_t trailing_dim,
                                           float scale, int32_t dtype, void* stream) {
    // sizes and dtype first; a problem without work is fine whatever its (possibly null) pointers
    if (bh < 0 || n_rows < 0 || n_cols < 0 || d < 1 || trailing_dim < 0) return SPLAT_ERR_BAD_ARG;
    if (dtype != SPLAT_F32 && dtype != SPLAT_F16 && dtype != SPLAT_BF16)
        return SPLAT_ERR_UNSUPPORTED_DTYPE;
    if (bh == 0 || n_rows == 0) return SPLAT_OK;
    if (!q || !k || !v || !o || !sTod_lin || !sTod_tr || !nnzs) return SPLAT_ERR_BAD_ARG;
    // overflow-safe size check against the fixed capacity
    const int64_t cap_elems = SPLAT_NOALLOC_SCRATCH_BYTES / splat::elem_size(dtype);
    if (trailing_dim > 0 && (bh > cap_elems / trailing_dim || bh * trailing_dim > cap_elems / n_rows))
        return SPLAT_ERR_SCRATCH_TOO_SMALL;
    void* scratch = nullptr;
    int32_t rc = scratch_on_current_device(&scratch);
    if (rc != SPLAT_OK) return rc;
    if (trailing_dim > 0) {
        rc = splat_sddmm(q, k, k_stride_bh, k_stride_col, k_stride_k, scratch, sTod_lin, sTod_tr,
                         nnzs, bh, n_rows, n_cols, d, trailing_dim, dtype, stream);
        if (rc != SPLAT_OK) return rc;
        rc = splat_softmax(scratch, scratch, nnzs, bh, n_rows, trailing_dim, scale, dtype, stream);
        if (rc != SPLAT_OK) return rc;
    }
    return splat_spmm(scratch, v, o, sTod_lin, sTod_tr, nnzs, bh, n_rows, n_cols, d, trailing_dim,
                      dtype, stream);
}
