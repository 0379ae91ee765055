"""CPU restatement of the reference's ACSR ("affine compressed sparse row") metadata path.

TEST INFRASTRUCTURE ONLY -- never imported by the shipped library.

Reference anchors (paths inside the reference project):
  * mask generators ............ SPLAT/acsr_helpers.py:18-55
  * per-row affine fit ......... SPLAT/acsr_helpers.py:99-142  (instantiate_metadata)
  * float32 packing ............ SPLAT/acsr_helpers.py:145-160 (create_acsr)
  * thread-block tile map ...... SPLAT/r_sddmm.py:117-146      (naive_block_mappings)

Third-party arithmetic on the path: ``numpy.linalg.solve`` (LAPACK gesv) for the 2x2 affine fit
(SPLAT/acsr_helpers.py:122).  The reference pins no numpy version.  ``metadata_literal`` calls
the same routine; ``metadata_from_rows`` is the closed form ``x = 1/(b-a)``, ``y = -a/(b-a)``
whose float32 image is compared with the fixtures in tests/golden.

Two masks in the benchmark configurations have no generator in the reference (column-strided
and dilated windows); ``strided_mask`` / ``dilated_mask`` are written from the configuration
text: "row i attends cols j=(i mod s)+s*k for all j<=i" and "row i attends cols i-dil*k for
k=0..taps-1 (clipped at 0)".
"""
from __future__ import annotations

from math import ceil

import numpy as np

PATTERN_BLOCKED = 0
PATTERN_WINDOWED = 1
PATTERN_CAUSAL_WINDOWED = 2
PATTERN_STRIDED = 3
PATTERN_DILATED = 4


# ----------------------------------------------------------------------------------------------
# Mask generators (dense L x L uint8; only for sizes where L*L bytes is affordable).
# ----------------------------------------------------------------------------------------------
def blocked_mask(s: int, p: int) -> np.ndarray:
    """SPLAT/acsr_helpers.py:18-34.  Rows < p see cols < p; row i >= p sees
    [(i//p - 1)*p, (i//p + 1)*p)."""
    i = np.arange(s)[:, None]
    j = np.arange(s)[None, :]
    start = (i // p - 1) * p
    m = np.where(i < p, j < p, (start <= j) & (j < start + 2 * p))
    return m.astype(np.uint8)


def windowed_mask(s: int, p: int) -> np.ndarray:
    """SPLAT/acsr_helpers.py:36-44.  |i - j| <= p."""
    i = np.arange(s)[:, None]
    j = np.arange(s)[None, :]
    return ((i - p <= j) & (j <= i + p)).astype(np.uint8)


def causal_windowed_mask(s: int, p: int) -> np.ndarray:
    """SPLAT/acsr_helpers.py:46-55.  i - p <= j <= i (window width p + 1)."""
    i = np.arange(s)[:, None]
    j = np.arange(s)[None, :]
    return ((i - p <= j) & (j <= i)).astype(np.uint8)


def strided_mask(s: int, stride: int) -> np.ndarray:
    """Column-periodic causal pattern: j = (i mod stride) + stride*k, j <= i."""
    i = np.arange(s)[:, None]
    j = np.arange(s)[None, :]
    return (((j % stride) == (i % stride)) & (j <= i)).astype(np.uint8)


def dilated_mask(s: int, taps: int, dilation: int) -> np.ndarray:
    """Dilated causal window: j = i - dilation*k for k = 0..taps-1, j >= 0."""
    i = np.arange(s)[:, None]
    j = np.arange(s)[None, :]
    diff = i - j
    return ((diff >= 0) & (diff % dilation == 0) & (diff // dilation < taps)).astype(np.uint8)


def make_mask(kind: int, s: int, p0: int, p1: int = 0) -> np.ndarray:
    if kind == PATTERN_BLOCKED:
        return blocked_mask(s, p0)
    if kind == PATTERN_WINDOWED:
        return windowed_mask(s, p0)
    if kind == PATTERN_CAUSAL_WINDOWED:
        return causal_windowed_mask(s, p0)
    if kind == PATTERN_STRIDED:
        return strided_mask(s, p0)
    if kind == PATTERN_DILATED:
        return dilated_mask(s, p0, p1)
    raise ValueError(f"unknown pattern kind {kind}")


# ----------------------------------------------------------------------------------------------
# Row summaries: (first set column, second set column, last set column, count) per row.
# ----------------------------------------------------------------------------------------------
def row_summary(mask: np.ndarray):
    """What instantiate_metadata extracts from each row (SPLAT/acsr_helpers.py:110-117), plus
    the last set column that naive_block_mappings needs (SPLAT/r_sddmm.py:129-135).
    Missing entries are -1."""
    m = np.asarray(mask) != 0
    rows, cols = m.shape
    count = m.sum(axis=1).astype(np.int64)
    first = np.where(count > 0, m.argmax(axis=1), -1).astype(np.int64)
    m2 = m.copy()
    nz = np.nonzero(count > 0)[0]
    m2[nz, first[nz]] = False
    second = np.where(count > 1, m2.argmax(axis=1), -1).astype(np.int64)
    last = np.where(count > 0, cols - 1 - m[:, ::-1].argmax(axis=1), -1).astype(np.int64)
    return first, second, last, count


def pattern_rows(kind: int, s: int, p0: int, p1: int = 0):
    """Closed-form row summaries of the five patterns -- no L x L mask is materialised."""
    i = np.arange(s, dtype=np.int64)
    if kind == PATTERN_BLOCKED:
        start = np.where(i < p0, 0, (i // p0 - 1) * p0)
        end = np.where(i < p0, p0, start + 2 * p0)
        end = np.minimum(end, s)
        step = np.ones_like(i)
    elif kind == PATTERN_WINDOWED:
        start = np.maximum(i - p0, 0)
        end = np.minimum(i + p0 + 1, s)
        step = np.ones_like(i)
    elif kind == PATTERN_CAUSAL_WINDOWED:
        start = np.maximum(i - p0, 0)
        end = i + 1
        step = np.ones_like(i)
    elif kind == PATTERN_STRIDED:
        start = i % p0
        end = i + 1
        step = np.full_like(i, p0)
    elif kind == PATTERN_DILATED:
        cnt = np.minimum(p0, i // p1 + 1)
        start = i - p1 * (cnt - 1)
        end = i + 1
        step = np.full_like(i, p1)
    else:
        raise ValueError(f"unknown pattern kind {kind}")
    count = np.maximum((end - start + step - 1) // step, 0)
    first = np.where(count > 0, start, -1)
    second = np.where(count > 1, start + step, -1)
    last = np.where(count > 0, start + (count - 1) * step, -1)
    return first, second, last, count


# ----------------------------------------------------------------------------------------------
# Metadata.
# ----------------------------------------------------------------------------------------------
META_KEYS = ("dTos_lin", "dTos_tr", "sTod_lin", "sTod_tr", "nnzs", "span_start", "span_end")


def metadata_literal(mask, block_height: int) -> dict:
    """Row-by-row restatement of instantiate_metadata + create_acsr
    (SPLAT/acsr_helpers.py:99-160) including the call into numpy.linalg.solve.  Slow; use on
    small masks to pin ``metadata_from_rows``."""
    m = np.asarray(mask)
    rows, cols = m.shape
    dl, dt, sl, st, nn = [], [], [], [], []
    spans = [(cols, -1) for _ in range(ceil(rows / block_height))]
    for r in range(rows):
        n = int(m[r].sum())
        if n > 1:
            idx = np.nonzero(m[r] == 1)[0]
            a, b = int(idx[0]), int(idx[1])
            x, y = np.linalg.solve(np.array([[a, 1], [b, 1]]), np.array([0, 1]))
        else:
            x, y = 1, 0
        dl.append(x)
        dt.append(y)
        lin = round(1 / x)
        tr = abs(y)
        sl.append(lin)
        st.append(tr)
        nn.append(n)
        cs, ce = spans[r // block_height]
        spans[r // block_height] = (min(cs, tr), max(ce, n * lin + tr))
    f32 = lambda v: np.asarray(v, dtype=np.float64).astype(np.float32)
    return {
        "dTos_lin": f32(dl), "dTos_tr": f32(dt), "sTod_lin": f32(sl), "sTod_tr": f32(st),
        "nnzs": f32(nn), "trailing_dim": int(m.sum(axis=1).max()) if rows else 0,
        "span_start": f32([s[0] for s in spans]), "span_end": f32([s[1] for s in spans]),
    }


def metadata_from_rows(first, second, count, n_cols: int, block_height: int) -> dict:
    """Closed form of the same computation: with a = first, b = second set column and n the
    row count, (s, a') = (b - a, a) when n > 1 else (1, 0);
    dTos = (1/s, 0.0 - a'/s), sTod = (s, a'/s), span = (min a'/s, max n*s + a'/s) per row block
    (initial values n_cols and -1), everything rounded once from float64 to float32."""
    first = np.asarray(first, dtype=np.int64)
    second = np.asarray(second, dtype=np.int64)
    count = np.asarray(count, dtype=np.int64)
    rows = count.shape[0]
    multi = count > 1
    s = np.where(multi, second - first, 1).astype(np.float64)
    a = np.where(multi, first, 0).astype(np.float64)
    tr = a / s
    nblk = ceil(rows / block_height) if rows else 0
    pad = nblk * block_height - rows
    tr_p = np.concatenate([tr, np.full(pad, np.inf)]).reshape(nblk, block_height)
    end = count.astype(np.float64) * s + tr
    end_p = np.concatenate([end, np.full(pad, -np.inf)]).reshape(nblk, block_height)
    span_start = np.minimum(tr_p.min(axis=1), float(n_cols))
    span_end = np.maximum(end_p.max(axis=1), -1.0)
    return {
        "dTos_lin": (1.0 / s).astype(np.float32),
        "dTos_tr": (0.0 - tr).astype(np.float32),
        "sTod_lin": s.astype(np.float32),
        "sTod_tr": tr.astype(np.float32),
        "nnzs": count.astype(np.float32),
        "trailing_dim": int(count.max()) if rows else 0,
        "span_start": span_start.astype(np.float32),
        "span_end": span_end.astype(np.float32),
    }


def metadata_from_mask(mask, block_height: int) -> dict:
    first, second, _last, count = row_summary(mask)
    return metadata_from_rows(first, second, count, np.asarray(mask).shape[1], block_height)


def metadata_from_pattern(kind: int, s: int, p0: int, p1: int, block_height: int) -> dict:
    first, second, _last, count = pattern_rows(kind, s, p0, p1)
    return metadata_from_rows(first, second, count, s, block_height)


def tile_map_from_rows(first, last, count, n_cols: int, block_height: int, block_width: int):
    """SPLAT/r_sddmm.py:117-146.  Row blocks b < max(rows // BH, 1); per block the min and max
    set column over its rows (initial values n_cols and 0); anchors x = min, min+BW, ... while
    x < max; y = b*BH.  Returns two int32 arrays."""
    first = np.asarray(first, dtype=np.int64)
    last = np.asarray(last, dtype=np.int64)
    count = np.asarray(count, dtype=np.int64)
    rows = count.shape[0]
    xs, ys = [], []
    for blk in range(max(rows // block_height, 1)):
        r0, r1 = blk * block_height, min((blk + 1) * block_height, rows)
        sel = count[r0:r1] > 0
        lo = int(min(n_cols, first[r0:r1][sel].min())) if sel.any() else n_cols
        hi = int(max(0, last[r0:r1][sel].max())) if sel.any() else 0
        x = lo
        while x < hi:
            xs.append(x)
            ys.append(blk * block_height)
            x += block_width
    return np.asarray(xs, dtype=np.int32), np.asarray(ys, dtype=np.int32)


def tile_map_from_mask(mask, block_height: int, block_width: int):
    first, _second, last, count = row_summary(mask)
    return tile_map_from_rows(first, last, count, np.asarray(mask).shape[1],
                              block_height, block_width)


# ----------------------------------------------------------------------------------------------
# From float32 metadata back to integer (start, stride, nnz) and the metadata-effective mask.
# ----------------------------------------------------------------------------------------------
def affine_ints(meta: dict):
    """Sparse slot j of row i is dense column start_i + j*stride_i, j < nnz_i.
    stride = sTod_lin, start = rint(sTod_tr * sTod_lin) (sTod_tr holds start/stride, see
    SPLAT/acsr_helpers.py:124), nnz = nnzs."""
    stride = np.rint(np.asarray(meta["sTod_lin"], dtype=np.float64)).astype(np.int64)
    start = np.rint(np.asarray(meta["sTod_tr"], dtype=np.float64) * stride).astype(np.int64)
    nnz = np.rint(np.asarray(meta["nnzs"], dtype=np.float64)).astype(np.int64)
    return start, stride, nnz


def effective_mask(meta: dict, n_cols: int) -> np.ndarray:
    """The mask the metadata describes.  Equals the input mask for affine rows with more than one
    non-zero; a row with exactly one non-zero is described as column 0
    (SPLAT/acsr_helpers.py:126-130), which is what every kernel then sees."""
    start, stride, nnz = affine_ints(meta)
    rows = start.shape[0]
    m = np.zeros((rows, n_cols), dtype=np.uint8)
    for r in range(rows):
        cols = start[r] + stride[r] * np.arange(nnz[r])
        m[r, cols] = 1
    return m
