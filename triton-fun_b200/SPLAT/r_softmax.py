"""Row softmax over the first nnz slots of every ACSR row.

Drop-in for the reference module SPLAT/r_softmax.py.  Unlike the reference launch (whose grid
covers only cdiv(L, BLOCK_SIZE_X) rows of a one-row-per-program kernel) every row is processed,
whatever ``grid_dim`` / ``BLOCK_SIZE_X`` say.  The reference applies no scaling; ``scale`` is an
extra keyword (default 1.0) folded into the exponent.
"""
from __future__ import annotations

from math import ceil, log2

import torch

import splat_native as _n
from acsr_helpers import create_acsr, create_blocked_mask, create_windowed_mask, mask_shape  # noqa: F401


def rsoftmax_preamble(mask, output_shape: tuple, BLOCK_SIZE_X: int, GPU_ID, out_dtype: torch.dtype):
    """-> (grid_dim, output, full_shape, trailing_dim_pow_two)  (reference SPLAT/r_softmax.py:108-124)."""
    dev = _n.resolve_device(GPU_ID)
    trailing_dim_pow_two = 2 ** ceil(log2(output_shape[-1])) if output_shape[-1] > 0 else 1
    full_shape = output_shape
    output = torch.empty(tuple(full_shape), dtype=out_dtype, device=dev)
    rows = mask_shape(mask)[0]
    grid_dim = (-(-rows // BLOCK_SIZE_X), output_shape[0] * output_shape[1])
    return (grid_dim, output, full_shape, trailing_dim_pow_two)


def rsoftmax_launcher(x: torch.Tensor, output: torch.Tensor,
                      dTos_linear_transformations: torch.Tensor, dTos_translations: torch.Tensor,
                      sTod_linear_transformations: torch.Tensor, sTod_translations: torch.Tensor,
                      acsr_trailing_dim_true: int, acsr_trailing_dim_power_two: int,
                      nnzs: torch.Tensor, grid_dim, BLOCK_SIZE_X: int, *, scale: float = 1.0):
    """x (B,H,L,trailing_dim) -> output, same shape, in place.  Returns
    (output, sTod_linear_transformations, sTod_translations, nnzs)  (reference
    SPLAT/r_softmax.py:126-150)."""
    _n.softmax(x, output, nnzs, acsr_trailing_dim_true, scale)
    return (output, sTod_linear_transformations, sTod_translations, nnzs)
