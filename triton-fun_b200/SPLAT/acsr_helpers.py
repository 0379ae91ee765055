"""ACSR ("affine compressed sparse row") metadata, built on the GPU.

Drop-in for the reference module of the same name (SPLAT/acsr_helpers.py): same function names,
positional parameters and return values.  Differences, all additive:

  * the mask generators return a ``PatternMask`` -- a read-only sequence that behaves like the
    reference's ``list[list[int]]`` (``len(mask)``, ``mask[i][j]``, ``len(mask[0])``, iteration)
    but carries the closed form, so ``create_acsr`` never materialises L x L entries;
  * ``create_acsr`` also accepts a ``list[list[int]]``, a numpy array or a torch tensor (any
    device) and scans it with a CUDA kernel;
  * two extra generators for patterns the reference has no generator for
    (``create_strided_mask``, ``create_dilated_mask``);
  * ``GPU_ID`` must name a CUDA device -- there is no CPU path.

The returned float32 tensors are bit-identical to the reference's (see tests/golden).
"""
from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass
from typing import Type

import numpy as np
import torch

import splat_native as _n


# ----------------------------------------------------------------------------------------------
# Masks
# ----------------------------------------------------------------------------------------------
def _pattern_row_bounds(kind: int, s: int, p0: int, p1: int, i: int):
    """(start, step, count) of row i -- host mirror of the closed form used on the device."""
    if kind == _n.PATTERN_BLOCKED:
        if i < p0:
            start, end = 0, p0
        else:
            start = (i // p0 - 1) * p0
            end = start + 2 * p0
        return start, 1, max(0, min(end, s) - start)
    if kind == _n.PATTERN_WINDOWED:
        start = max(i - p0, 0)
        return start, 1, max(0, min(i + p0 + 1, s) - start)
    if kind == _n.PATTERN_CAUSAL_WINDOWED:
        start = max(i - p0, 0)
        return start, 1, i + 1 - start
    if kind == _n.PATTERN_STRIDED:
        start = i % p0
        return start, p0, (i - start) // p0 + 1
    if kind == _n.PATTERN_DILATED:
        cnt = min(p0, i // p1 + 1)
        return i - p1 * (cnt - 1), p1, cnt
    raise ValueError(f"unknown pattern kind {kind}")


class PatternMask(Sequence):
    """A square 0/1 mask with a closed form.  Quacks like ``list[list[int]]``."""

    def __init__(self, kind: int, s: int, p0: int, p1: int = 0):
        if s < 0:
            raise ValueError("sequence length must be non-negative")
        if kind in (_n.PATTERN_BLOCKED, _n.PATTERN_STRIDED) and p0 < 1:
            raise ValueError("sparsity parameter must be >= 1")
        if kind in (_n.PATTERN_WINDOWED, _n.PATTERN_CAUSAL_WINDOWED) and p0 < 0:
            raise ValueError("window parameter must be >= 0")
        if kind == _n.PATTERN_DILATED and (p0 < 1 or p1 < 1):
            raise ValueError("taps and dilation must be >= 1")
        self.kind, self.s, self.p0, self.p1 = kind, int(s), int(p0), int(p1)

    def __len__(self) -> int:
        return self.s

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[k] for k in range(*i.indices(self.s))]
        if i < 0:
            i += self.s
        if not 0 <= i < self.s:
            raise IndexError(i)
        start, step, count = _pattern_row_bounds(self.kind, self.s, self.p0, self.p1, i)
        row = [0] * self.s
        if count > 0:
            row[start:start + (count - 1) * step + 1:step] = [1] * count
        return row

    def tolist(self) -> list:
        return [self[i] for i in range(self.s)]

    def to_tensor(self, GPU_ID=0) -> torch.Tensor:
        """The full (s, s) uint8 mask, written by a CUDA kernel."""
        return _n.pattern_mask(self.kind, self.s, self.p0, self.p1, _n.resolve_device(GPU_ID))

    def __repr__(self) -> str:
        return f"PatternMask(kind={self.kind}, s={self.s}, p0={self.p0}, p1={self.p1})"


## s -> sequence length, p -> sparsity parameter (names and meaning as in the reference).
def create_blocked_mask(s: int, p: int) -> PatternMask:
    """Rows < p see cols < p; row i >= p sees [(i//p - 1)p, (i//p + 1)p)
    (reference SPLAT/acsr_helpers.py:18-34)."""
    return PatternMask(_n.PATTERN_BLOCKED, s, p)


def create_windowed_mask(s: int, p: int) -> PatternMask:
    """|i - j| <= p (reference SPLAT/acsr_helpers.py:36-44)."""
    return PatternMask(_n.PATTERN_WINDOWED, s, p)


def create_causal_windowed_mask(s: int, p: int) -> PatternMask:
    """i - p <= j <= i, i.e. window width p + 1 (reference SPLAT/acsr_helpers.py:46-55)."""
    return PatternMask(_n.PATTERN_CAUSAL_WINDOWED, s, p)


def create_strided_mask(s: int, stride: int) -> PatternMask:
    """Row i attends columns (i mod stride) + stride*k <= i.  Not in the reference."""
    return PatternMask(_n.PATTERN_STRIDED, s, stride)


def create_dilated_mask(s: int, taps: int, dilation: int) -> PatternMask:
    """Row i attends columns i - dilation*k >= 0 for k < taps.  Not in the reference."""
    return PatternMask(_n.PATTERN_DILATED, s, taps, dilation)


# ----------------------------------------------------------------------------------------------
# Containers (reference SPLAT/acsr_helpers.py:58-96)
# ----------------------------------------------------------------------------------------------
## This gives the mapping from dense -> sparse.
@dataclass
class AffineIndices:
    linear_transformation: float
    translation: int
    nnz: int


## This gives the mapping from sparse -> dense.
@dataclass
class AffineIndicesInt:
    linear_transformation: int
    translation: int
    nnz: int


class ACSR:
    def __init__(self, affine_indices: list[Type[AffineIndices]],
                 affine_indices_int: list[Type[AffineIndicesInt]],
                 span_specialised_loop_idxs: list[tuple[int]]):
        self.affine_indices = affine_indices
        self.affine_indices_int = affine_indices_int
        self.span_specialised_loop_idxs = span_specialised_loop_idxs

    def get_dTos_linear_transformations(self) -> list[float]:
        return [x.linear_transformation for x in self.affine_indices]

    def get_sTod_linear_transformations(self) -> list[int]:
        return [x.linear_transformation for x in self.affine_indices_int]

    def get_dTos_translations(self) -> list[float]:
        return [x.translation for x in self.affine_indices]

    def get_sTod_translations(self) -> list[int]:
        return [x.translation for x in self.affine_indices_int]

    def get_nnzs(self) -> list[float]:
        return [x.nnz for x in self.affine_indices]

    def get_span_specialised_data(self) -> list[tuple[int]]:
        return self.span_specialised_loop_idxs


# ----------------------------------------------------------------------------------------------
# Metadata
# ----------------------------------------------------------------------------------------------
def mask_shape(mask) -> tuple[int, int]:
    if isinstance(mask, PatternMask):
        return mask.s, mask.s
    if isinstance(mask, (torch.Tensor, np.ndarray)):
        return int(mask.shape[0]), int(mask.shape[1])
    return len(mask), (len(mask[0]) if len(mask) else 0)


def row_summary(mask, dev: torch.device) -> torch.Tensor:
    """int32 (4, rows) on ``dev``: first, second, last set column and count of every row."""
    if isinstance(mask, PatternMask):
        return _n.pattern_row_summary(mask.kind, mask.s, mask.p0, mask.p1, dev)
    if isinstance(mask, torch.Tensor):
        m = mask
        if m.dtype != torch.uint8:
            m = (m != 0).to(torch.uint8)
        m = m.to(dev)
    else:
        m = torch.from_numpy(np.ascontiguousarray(np.asarray(mask) != 0).astype(np.uint8)).to(dev)
    if m.dim() != 2:
        raise ValueError("mask must be 2-dimensional")
    return _n.mask_row_summary(m)


def _create_acsr_on(mask, BLOCK_HEIGHT: int, dev: torch.device):
    rows = row_summary(mask, dev)
    return _n.acsr_from_row_summary(rows, mask_shape(mask)[1], BLOCK_HEIGHT)


## We create all the necessary metadata required for the ACSR.
def instantiate_metadata(mask, BLOCK_HEIGHT: int) -> ACSR:
    """Host-side container of the metadata (reference SPLAT/acsr_helpers.py:99-142).  Computed on
    the current CUDA device and copied back; values are the float32-rounded ones the kernels see."""
    dev = torch.device("cuda", torch.cuda.current_device())
    dl, dt, sl, st, nn, _td, s0, s1 = _create_acsr_on(mask, BLOCK_HEIGHT, dev)
    dl, dt, sl, st, nn = (t.cpu().tolist() for t in (dl, dt, sl, st, nn))
    d2s = [AffineIndices(a, b, int(c)) for a, b, c in zip(dl, dt, nn)]
    s2d = [AffineIndicesInt(int(a), b, int(c)) for a, b, c in zip(sl, st, nn)]
    return ACSR(d2s, s2d, list(zip(s0.cpu().tolist(), s1.cpu().tolist())))


## Now we have to send everything to the GPU!
def create_acsr(mask, BLOCK_HEIGHT: int, GPU_ID):
    """-> (dTos_linear_transformations, dTos_translations, sTod_linear_transformations,
    sTod_translations, nnzs, trailing_dim_acsr, span_spec_loop_start, span_spec_loop_end):
    five float32 tensors of length L, a Python int, two float32 tensors of length
    ceil(L / BLOCK_HEIGHT) -- reference SPLAT/acsr_helpers.py:145-160, computed by CUDA kernels."""
    return _create_acsr_on(mask, BLOCK_HEIGHT, _n.resolve_device(GPU_ID))
