"""SpMM over ACSR: O = P V with P in (B, H, L, trailing_dim) ACSR layout.

Drop-in for the reference module SPLAT/r_spmm.py.  All L rows of the output are written and the
whole span of every row is accumulated (the reference kernel only does so for L <= 128 and rows
below the head dimension).
"""
from __future__ import annotations

import torch

import splat_native as _n
from acsr_helpers import create_acsr, create_blocked_mask, create_windowed_mask, mask_shape, row_summary  # noqa: F401


def rspmm_preamble(mask, output_shape: tuple, BLOCK_SIZE_X: int, BLOCK_SIZE_Y: int, GPU_ID,
                   output_dtype: torch.dtype):
    """-> (output, grid_dim, trailing_dim_acsr)  (reference SPLAT/r_spmm.py:128-145)."""
    dev = _n.resolve_device(GPU_ID)
    counts = row_summary(mask, dev)[3]
    trailing_dim_acsr = int(counts.max().item()) if counts.numel() else 0
    output = torch.empty(tuple(output_shape), dtype=output_dtype, device=dev)
    grid_dim = (-(-output_shape[3] // BLOCK_SIZE_X), -(-output_shape[2] // BLOCK_SIZE_Y),
                output_shape[0] * output_shape[1])
    return (output, grid_dim, trailing_dim_acsr)


## Over here, x is an ACSR and y is the Values tensor.
def rspmm_launcher(x: torch.Tensor, y: torch.Tensor, output: torch.Tensor,
                   dTos_linear_transformations: torch.Tensor, dTos_translations: torch.Tensor,
                   sTod_linear_transformations: torch.Tensor, sTod_translations: torch.Tensor,
                   span_loop_start: torch.Tensor, span_loop_end: torch.Tensor,
                   acsr_trailing_dim: int, nnzs: torch.Tensor, grid_dim,
                   BLOCK_SIZE_Y: int, BLOCK_SIZE_X: int):
    """x = P (B,H,L,trailing_dim), y = V (B,H,L,d) -> output (B,H,L,d), in place.  Returns
    (output, sTod_linear_transformations, sTod_translations, nnzs)  (reference
    SPLAT/r_spmm.py:148-164)."""
    _n.spmm(x, y, output, sTod_linear_transformations, sTod_translations, nnzs, acsr_trailing_dim)
    return (output, sTod_linear_transformations, sTod_translations, nnzs)
