"""ctypes binding of libsplat_b200.so (the C ABI declared in include/splat_b200.h).

There is no fallback: if the library is missing this module raises at import, and every wrapper
turns a non-zero status into ``RuntimeError``.  Build the library with
``python triton-fun_b200/build.py`` (nvcc, sm_100a).
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import time

import torch

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("SPLAT_B200_LIB") or os.path.join(_PKG_DIR, "libsplat_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: build it with `python {os.path.join(_PKG_DIR, 'build.py')}` "
        "(this package has no CPU or eager fallback)")

_lib = ctypes.CDLL(LIB_PATH)

_i32, _i64, _f32, _vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p

# name -> argtypes; every function returns int32 except splat_status_string
SIGNATURES = {
    "splat_version": [],
    "splat_mask_row_summary_u8": [_vp, _i64, _i64, _i64, _vp, _vp],
    "splat_pattern_row_summary": [_i32, _i64, _i64, _i64, _vp, _vp],
    "splat_pattern_mask_u8": [_i32, _i64, _i64, _i64, _vp, _i64, _vp],
    "splat_acsr_from_row_summary": [_vp, _i64, _i64, _i32] + [_vp] * 8 + [_vp],
    "splat_acsr_classify": [_vp, _vp, _vp, _i64, _vp, _vp],
    "splat_sddmm": [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64,
                    _i32, _vp],
    "splat_softmax": [_vp, _vp, _vp, _i64, _i64, _i64, _f32, _i32, _vp],
    "splat_spmm": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp],
    "splat_attention_fused": [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                              _i64, _i64, _f32, _i32, _i32, _vp, _vp, _vp],
    "splat_attention_fused_ex": [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                 _i64, _i64, _f32, _i32, _i32, _vp, _vp, _vp, _vp],
    "splat_attention_fused_lse": [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                  _i64, _i64, _f32, _i32, _i32, _vp, _vp, _vp, _vp],
    "splat_sddmm_band": [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64,
                         _i32, _vp, _vp, _vp],
    "splat_spmm_band": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _vp,
                        _vp],
    "splat_selftest_bounded_wait": [_vp, _i64, _vp],
    "splat_debug_check_indices": [_vp],
    "splat_attention_noalloc": [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                _i64, _i64, _i64, _f32, _i32, _vp],
}
for _name, _args in SIGNATURES.items():
    _fn = getattr(_lib, _name)
    _fn.argtypes = _args
    _fn.restype = _i32
_lib.splat_status_string.argtypes = [_i32]
_lib.splat_status_string.restype = ctypes.c_char_p

PATTERN_BLOCKED, PATTERN_WINDOWED, PATTERN_CAUSAL_WINDOWED, PATTERN_STRIDED, PATTERN_DILATED = range(5)
PATH_AUTO, PATH_GENERIC, PATH_BAND = 0, 1, 2
NOALLOC_SCRATCH_BYTES = 64 << 20     # SPLAT_NOALLOC_SCRATCH_BYTES in include/splat_b200.h
DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def status_string(code: int) -> str:
    return _lib.splat_status_string(int(code)).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what}: splat status {code} ({status_string(code)})")


def version() -> int:
    return _lib.splat_version()


def resolve_device(gpu_id) -> torch.device:
    """GPU_ID of the reference API: an int or a torch/cuda device.  'cpu' is rejected."""
    dev = torch.device("cuda", gpu_id) if isinstance(gpu_id, int) else torch.device(gpu_id)
    if dev.type != "cuda":
        raise ValueError(f"device {gpu_id!r}: this implementation runs on CUDA devices only "
                         "(there is no CPU path)")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    return dev


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    try:
        return DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}; expected float32, float16 or bfloat16") from None


def _f32_vec(t: torch.Tensor, n: int, name: str) -> int:
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous() or t.numel() < n:
        raise ValueError(f"{name} must be a contiguous float32 CUDA tensor of at least {n} elements")
    return t.data_ptr()


# ----------------------------------------------------------------------------------------------
# metadata
# ----------------------------------------------------------------------------------------------
def mask_row_summary(mask_u8: torch.Tensor) -> torch.Tensor:
    """(rows, cols) uint8 CUDA mask -> int32 (4, rows): first, second, last set column, count."""
    assert mask_u8.is_cuda and mask_u8.dtype == torch.uint8 and mask_u8.dim() == 2
    if mask_u8.stride(1) != 1:
        mask_u8 = mask_u8.contiguous()
    rows, cols = mask_u8.shape
    out = torch.empty((4, rows), dtype=torch.int32, device=mask_u8.device)
    with torch.cuda.device(mask_u8.device):
        check(_lib.splat_mask_row_summary_u8(mask_u8.data_ptr(), rows, cols, mask_u8.stride(0),
                                             out.data_ptr(), _stream(mask_u8.device)),
              "splat_mask_row_summary_u8")
    return out


def pattern_row_summary(kind: int, n: int, p0: int, p1: int, dev: torch.device) -> torch.Tensor:
    out = torch.empty((4, n), dtype=torch.int32, device=dev)
    with _on(dev):
        check(_lib.splat_pattern_row_summary(kind, n, p0, p1, out.data_ptr(), _stream(dev)),
              "splat_pattern_row_summary")
    return out


def pattern_mask(kind: int, n: int, p0: int, p1: int, dev: torch.device) -> torch.Tensor:
    out = torch.empty((n, n), dtype=torch.uint8, device=dev)
    with _on(dev):
        check(_lib.splat_pattern_mask_u8(kind, n, p0, p1, out.data_ptr(), out.stride(0) if n else 0,
                                         _stream(dev)), "splat_pattern_mask_u8")
    return out


def acsr_from_row_summary(rows_i32: torch.Tensor, n_cols: int, block_height: int):
    """-> (dTos_lin, dTos_tr, sTod_lin, sTod_tr, nnzs, trailing_dim, span_start, span_end)."""
    dev = rows_i32.device
    n_rows = rows_i32.shape[1]
    n_blocks = -(-n_rows // block_height)
    vec = [torch.empty(n_rows, dtype=torch.float32, device=dev) for _ in range(5)]
    spans = [torch.empty(n_blocks, dtype=torch.float32, device=dev) for _ in range(2)]
    td = torch.empty(1, dtype=torch.int32, device=dev)
    with _on(dev):
        check(_lib.splat_acsr_from_row_summary(
            rows_i32.data_ptr(), n_rows, n_cols, block_height, *[v.data_ptr() for v in vec],
            spans[0].data_ptr(), spans[1].data_ptr(), td.data_ptr(), _stream(dev)),
            "splat_acsr_from_row_summary")
    return (*vec, int(td.item()), spans[0], spans[1])


def classify(sTod_lin: torch.Tensor, sTod_tr: torch.Tensor, nnzs: torch.Tensor) -> tuple:
    """Host copy of the 8 plan ints of ``splat_acsr_classify``.  The result is remembered ON the
    ``nnzs`` tensor object (with the identities and versions of all three tensors), so it lives
    exactly as long as that metadata and is recomputed if any of them is modified in place."""
    key = (id(sTod_lin), id(sTod_tr), sTod_lin._version, sTod_tr._version, nnzs._version,
           nnzs.numel())
    hit = getattr(nnzs, "_splat_plan", None)
    if hit is not None and hit[0] == key:
        return hit[1]
    dev = nnzs.device
    n = nnzs.numel()
    plan = torch.empty(8, dtype=torch.int32, device=dev)
    with _on(dev):
        check(_lib.splat_acsr_classify(_f32_vec(sTod_lin, n, "sTod_lin"), _f32_vec(sTod_tr, n, "sTod_tr"),
                                       _f32_vec(nnzs, n, "nnzs"), n, plan.data_ptr(), _stream(dev)),
              "splat_acsr_classify")
    host = tuple(int(v) for v in plan.cpu().tolist())
    # keep the two companions alive with the cache entry so their ids cannot be reused
    nnzs._splat_plan = (key, host, sTod_lin, sTod_tr)
    return host


_STATUS_WORDS: dict = {}
_STATUS_MIRRORS: dict = {}


def status_word(dev: torch.device) -> torch.Tensor:
    """Per-device int32 the band kernel sets when one of its bounded waits gives up."""
    key = (dev.type, dev.index)
    t = _STATUS_WORDS.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _STATUS_WORDS[key] = t
    return t


def _mirror(dev: torch.device) -> dict:
    """Pinned host copy of the status word, refreshed after every tensor-core launch by a copy on
    a side stream, so that the host can look at it without synchronising the device."""
    key = (dev.type, dev.index)
    m = _STATUS_MIRRORS.get(key)
    if m is None:
        m = {"host": torch.zeros(1, dtype=torch.int32).pin_memory(), "stream": torch.cuda.Stream(dev),
             "launched": torch.cuda.Event(), "pending": 0, "stamp": 0.0}
        _STATUS_MIRRORS[key] = m
    return m


def _raise_if_gave_up(dev: torch.device) -> None:
    """Start of every tensor-core launcher: if an earlier launch on this device reported a
    timed-out wait (the kernels do nothing while the word is set), clear the word and raise
    instead of silently returning stale outputs.  Costs one host memory read."""
    m = _STATUS_MIRRORS.get((dev.type, dev.index))
    if m is None or int(m["host"][0]) == 0:
        return
    torch.cuda.synchronize(dev)
    code = int(status_word(dev).item())
    status_word(dev).zero_()
    m["host"].zero_()
    torch.cuda.synchronize(dev)
    raise RuntimeError(f"an earlier tensor-core kernel on {dev} gave up on a device-side wait "
                       f"(code {code}): {status_string(-5)}; its outputs and those of later "
                       "launches are not valid")


_MIRROR_EVERY = 32          # launches between two refreshes of the mirror, at most
_MIRROR_SECONDS = 0.002     # ... or this much time, whichever comes first


def _on(dev: torch.device):
    """Make dev the current device for a library call; free when it already is."""
    if torch.cuda.current_device() == dev.index:
        return contextlib.nullcontext()
    return torch.cuda.device(dev)


def _refresh_mirror(dev: torch.device) -> None:
    """After a tensor-core launch: copy the status word to its pinned mirror behind the launch, on
    a side stream, so the launching stream is not delayed.  Back-to-back launches share a copy (one
    per _MIRROR_EVERY launches or _MIRROR_SECONDS): a launch that gave up is reported that many
    launches later at the latest, and the kernels in between do nothing, as documented."""
    m = _mirror(dev)
    m["pending"] += 1
    now = time.monotonic()
    if m["pending"] < _MIRROR_EVERY and now - m["stamp"] < _MIRROR_SECONDS:
        return
    m["pending"] = 0
    m["stamp"] = now
    m["launched"].record(torch.cuda.current_stream(dev))
    m["stream"].wait_event(m["launched"])
    with torch.cuda.stream(m["stream"]):
        m["host"].copy_(status_word(dev), non_blocking=True)


_INDEX_CODES = {71: "sddmm", 72: "spmm", 73: "fused"}


def check_indices(dev, on: bool = True) -> None:
    """Checked-index mode of the CUDA-core kernels: columns derived from the metadata are clamped to
    [0, n_cols) and a code (71 SDDMM, 72 SpMM, 73 fused) is left in the device's status word, which
    check_status_word() reads.  SPLAT_B200_DEBUG switches it on for every CUDA-core launch."""
    dev = resolve_device(dev)
    check(_lib.splat_debug_check_indices(status_word(dev).data_ptr() if on else None),
          "splat_debug_check_indices")


def _debug_before(dev) -> bool:
    if not os.environ.get("SPLAT_B200_DEBUG"):
        return False
    check_indices(dev, True)
    return True


def check_status_word(dev) -> None:
    """Synchronises the device; raises if a band kernel reported a timed-out wait (and clears it)."""
    dev = resolve_device(dev)
    w = status_word(dev)
    code = int(w.item())
    if code != 0:
        w.zero_()
        m = _STATUS_MIRRORS.get((dev.type, dev.index))
        if m is not None:
            torch.cuda.synchronize(dev)
            m["host"].zero_()
        if code in _INDEX_CODES:
            raise RuntimeError(f"checked-index mode: a column derived from the row metadata lies outside "
                               f"[0, n_cols) in the {_INDEX_CODES[code]} kernel (code {code})")
        raise RuntimeError(f"band kernel gave up on a device-side wait (code {code}): "
                           f"{status_string(-5)}")


# ----------------------------------------------------------------------------------------------
# operators
# ----------------------------------------------------------------------------------------------
def _flat_bh(t: torch.Tensor, name: str):
    """(B, H, X, Y) tensor whose (B, H) dims collapse -> (bh, stride_bh, stride_x, stride_y)."""
    if t.dim() != 4:
        raise ValueError(f"{name} must be 4-dimensional (batch, heads, ., .)")
    B, H = t.shape[0], t.shape[1]
    sb, sh, sx, sy = t.stride()
    if B > 1 and H > 1 and sb != H * sh:
        raise ValueError(f"{name}: batch and head dimensions must be collapsible (stride {t.stride()})")
    stride_bh = sh if H > 1 else (sb if B > 1 else t.shape[2] * t.shape[3])
    return B * H, stride_bh, sx, sy


def _contig(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


ERR_UNSUPPORTED_SHAPE, ERR_MISALIGNED, ERR_DRIVER = -6, -3, -7
# statuses of a tensor-core entry point that mean "this path does not apply, use the general one"
_BAND_NOT_APPLICABLE = (ERR_UNSUPPORTED_SHAPE, ERR_MISALIGNED, ERR_DRIVER)
_warned_cuda_core_16bit = False


def _warn_cuda_core_16bit(what: str) -> None:
    """16-bit operands that land on the CUDA-core kernels run many times slower than on the
    tensor-core path; say so once."""
    global _warned_cuda_core_16bit
    if not _warned_cuda_core_16bit:
        _warned_cuda_core_16bit = True
        import warnings
        warnings.warn(f"{what}: 16-bit operands are running on the CUDA-core kernels (pattern, layout, "
                      "alignment or head size outside what the tensor-core kernels take); expect a "
                      "much lower rate", RuntimeWarning, stacklevel=3)


def _band_candidate(x: torch.Tensor, path: int) -> bool:
    """The tensor-core kernels take 16-bit operands with d = 64 or 128 (the library checks the rest)."""
    return path != PATH_GENERIC and x.dtype in (torch.float16, torch.bfloat16) and x.numel() > 0


def sddmm(x, y, output, sTod_lin, sTod_tr, nnzs, trailing_dim: int, path: int = PATH_AUTO) -> None:
    dev = x.device
    _contig(x, "x"); _contig(output, "output")
    B, H, L, d = x.shape
    bh, ksb, ksk, ksc = _flat_bh(y, "y")          # y is (B, H, d, n): dim 2 = k, dim 3 = column
    n_cols = y.shape[3]
    if y.shape[2] != d or bh != B * H or y.dtype != x.dtype or output.dtype != x.dtype:
        raise ValueError("sddmm: inconsistent operand shapes or dtypes")
    if tuple(output.shape) != (B, H, L, trailing_dim):
        raise ValueError(f"sddmm: output must have shape {(B, H, L, trailing_dim)}")
    # K layouts the tensor-core kernel reads: the transposed view of a contiguous (B,H,L,d) tensor, or
    # the reference's contiguous (B,H,d,L) K^T (the library checks the rest)
    k_layout_ok = ksb == n_cols * d and ((ksk == 1 and ksc == d) or (ksc == 1 and ksk == n_cols))
    if _band_candidate(x, path) and k_layout_ok:
        _raise_if_gave_up(dev)
        plan_arr = (ctypes.c_int32 * 8)(*classify(sTod_lin, sTod_tr, nnzs))
        with _on(dev):
            rc = _lib.splat_sddmm_band(x.data_ptr(), y.data_ptr(), ksb, ksc, ksk, output.data_ptr(),
                                       _f32_vec(sTod_lin, L, "sTod_lin"), _f32_vec(sTod_tr, L, "sTod_tr"),
                                       _f32_vec(nnzs, L, "nnzs"), bh, L, n_cols, d, trailing_dim,
                                       dtype_code(x.dtype), ctypes.cast(plan_arr, ctypes.c_void_p),
                                       status_word(dev).data_ptr(), _stream(dev))
        if rc not in _BAND_NOT_APPLICABLE or path == PATH_BAND:
            check(rc, "splat_sddmm_band")
            _refresh_mirror(dev)
            if os.environ.get("SPLAT_B200_DEBUG"):
                check_status_word(dev)
            return
    if path == PATH_BAND:
        raise RuntimeError("sddmm: the band path does not apply to these operands")
    if x.dtype != torch.float32 and x.numel() > 0:
        _warn_cuda_core_16bit("sddmm")
    debug = _debug_before(dev)
    with _on(dev):
        check(_lib.splat_sddmm(x.data_ptr(), y.data_ptr(), ksb, ksc, ksk, output.data_ptr(),
                               _f32_vec(sTod_lin, L, "sTod_lin"), _f32_vec(sTod_tr, L, "sTod_tr"),
                               _f32_vec(nnzs, L, "nnzs"), bh, L, n_cols, d, trailing_dim,
                               dtype_code(x.dtype), _stream(dev)), "splat_sddmm")
    if debug:
        check_status_word(dev)


def softmax(x, output, nnzs, trailing_dim: int, scale: float = 1.0) -> None:
    dev = x.device
    _contig(x, "x"); _contig(output, "output")
    B, H, L, T = x.shape
    if T != trailing_dim or output.shape != x.shape or output.dtype != x.dtype:
        raise ValueError("softmax: inconsistent operand shapes or dtypes")
    with _on(dev):
        check(_lib.splat_softmax(x.data_ptr(), output.data_ptr(), _f32_vec(nnzs, L, "nnzs"), B * H,
                                 L, T, float(scale), dtype_code(x.dtype), _stream(dev)),
              "splat_softmax")


def spmm(x, y, output, sTod_lin, sTod_tr, nnzs, trailing_dim: int, path: int = PATH_AUTO) -> None:
    dev = x.device
    _contig(x, "x"); _contig(y, "y"); _contig(output, "output")
    B, H, L, T = x.shape
    n_cols, d = y.shape[2], y.shape[3]
    if T != trailing_dim or tuple(output.shape) != (B, H, L, d) or y.dtype != x.dtype or \
            output.dtype != x.dtype or y.shape[:2] != x.shape[:2]:
        raise ValueError("spmm: inconsistent operand shapes or dtypes")
    if _band_candidate(x, path):
        _raise_if_gave_up(dev)
        plan_arr = (ctypes.c_int32 * 8)(*classify(sTod_lin, sTod_tr, nnzs))
        with _on(dev):
            rc = _lib.splat_spmm_band(x.data_ptr(), y.data_ptr(), output.data_ptr(),
                                      _f32_vec(sTod_lin, L, "sTod_lin"), _f32_vec(sTod_tr, L, "sTod_tr"),
                                      _f32_vec(nnzs, L, "nnzs"), B * H, L, n_cols, d, T,
                                      dtype_code(x.dtype), ctypes.cast(plan_arr, ctypes.c_void_p),
                                      status_word(dev).data_ptr(), _stream(dev))
        if rc not in _BAND_NOT_APPLICABLE or path == PATH_BAND:
            check(rc, "splat_spmm_band")
            _refresh_mirror(dev)
            if os.environ.get("SPLAT_B200_DEBUG"):
                check_status_word(dev)
            return
    if path == PATH_BAND:
        raise RuntimeError("spmm: the band path does not apply to these operands")
    if x.dtype != torch.float32 and x.numel() > 0:
        _warn_cuda_core_16bit("spmm")
    debug = _debug_before(dev)
    with _on(dev):
        check(_lib.splat_spmm(x.data_ptr(), y.data_ptr(), output.data_ptr(),
                              _f32_vec(sTod_lin, L, "sTod_lin"), _f32_vec(sTod_tr, L, "sTod_tr"),
                              _f32_vec(nnzs, L, "nnzs"), B * H, L, n_cols, d, T,
                              dtype_code(x.dtype), _stream(dev)), "splat_spmm")
    if debug:
        check_status_word(dev)


def attention_fused(q, kt, v, output, sTod_lin, sTod_tr, nnzs, scale: float = 1.0,
                    path: int = PATH_AUTO, plan=None, lse=None) -> None:
    """q, v, output (B,H,L,d) contiguous; kt (B,H,d,L) -- contiguous (the reference's layout), or
    the transposed view of a contiguous (B,H,L,d) tensor.  The tensor-core path takes both (the
    contiguous one for stride-1 patterns).  lse: optional contiguous float32 (B,H,L) tensor that
    receives each row's log-sum-exp of the scaled scores (natural log, -inf for empty rows)."""
    dev = q.device
    _contig(q, "q"); _contig(v, "v"); _contig(output, "output")
    B, H, L, d = q.shape
    bh, ksb, ksk, ksc = _flat_bh(kt, "kt")
    n_cols = kt.shape[3]
    if kt.shape[2] != d or tuple(v.shape) != (B, H, n_cols, d) or output.shape != q.shape or \
            len({q.dtype, kt.dtype, v.dtype, output.dtype}) != 1:
        raise ValueError("attention: inconsistent operand shapes or dtypes")
    if lse is not None and (lse.dtype != torch.float32 or tuple(lse.shape) != (B, H, L) or
                            not lse.is_contiguous() or lse.device != dev):
        raise ValueError("attention: lse must be a contiguous float32 (B, H, L) tensor on the operands' device")
    plan_arr = None
    tensor_core = _band_candidate(q, path)      # a tensor-core kernel may run (the library decides)
    if path != PATH_GENERIC:
        if plan is None:
            plan = classify(sTod_lin, sTod_tr, nnzs)
        plan_arr = (ctypes.c_int32 * 8)(*plan)
    if tensor_core:
        _raise_if_gave_up(dev)
    sw = status_word(dev)
    ran = ctypes.c_int32(0)
    _debug_before(dev)
    with _on(dev):
        check(_lib.splat_attention_fused_lse(
            q.data_ptr(), kt.data_ptr(), ksb, ksc, ksk, v.data_ptr(), output.data_ptr(),
            lse.data_ptr() if lse is not None and lse.numel() > 0 else None,
            _f32_vec(sTod_lin, L, "sTod_lin"), _f32_vec(sTod_tr, L, "sTod_tr"),
            _f32_vec(nnzs, L, "nnzs"), bh, L, n_cols, d, float(scale), dtype_code(q.dtype),
            int(path), ctypes.cast(plan_arr, _vp) if plan_arr is not None else None,
            sw.data_ptr(), ctypes.byref(ran), _stream(dev)), "splat_attention_fused_lse")
    if ran.value == PATH_BAND:
        _refresh_mirror(dev)
    elif q.dtype != torch.float32 and q.numel() > 0 and path == PATH_AUTO:
        _warn_cuda_core_16bit("attention")
    if os.environ.get("SPLAT_B200_DEBUG"):
        check_status_word(dev)
