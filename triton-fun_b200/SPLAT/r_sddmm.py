"""SDDMM over ACSR: S = (Q K^T) evaluated only at the affine non-zeros.

Drop-in for the reference module SPLAT/r_sddmm.py: ``rsddmm_preamble`` / ``rsddmm_launcher`` /
``gen_block_mappings`` / ``naive_block_mappings`` / ``truth`` keep their positional parameters and
return tuples.  The launcher calls the CUDA library (``splat_sddmm``); ``grid_dim``, ``tb_map_x/y``
and the block sizes are accepted for compatibility and ignored by the kernels (the tile map is
still produced, identical to the reference's).
"""
from __future__ import annotations

import numpy as np
import torch

import splat_native as _n
from acsr_helpers import create_acsr, create_blocked_mask, mask_shape, row_summary  # noqa: F401


def naive_block_mappings(mask, BLOCK_HEIGHT: int, BLOCK_WIDTH: int, GPU_ID):
    """Thread-block anchor points of the reference's tiling (SPLAT/r_sddmm.py:117-146): for every
    row block b < max(L // BLOCK_HEIGHT, 1), x = min_col, min_col + BLOCK_WIDTH, ... while
    x < max_col, y = b * BLOCK_HEIGHT.  Row extents come from a CUDA scan of the mask."""
    dev = _n.resolve_device(GPU_ID)
    rows, cols = mask_shape(mask)
    first, _second, last, count = row_summary(mask, dev).cpu().numpy()
    xs, ys = [], []
    for blk in range(max(rows // BLOCK_HEIGHT, 1)):
        r0, r1 = blk * BLOCK_HEIGHT, min((blk + 1) * BLOCK_HEIGHT, rows)
        sel = count[r0:r1] > 0
        lo = min(cols, int(first[r0:r1][sel].min())) if sel.any() else cols
        hi = max(0, int(last[r0:r1][sel].max())) if sel.any() else 0
        if lo < hi:
            x = np.arange(lo, hi, BLOCK_WIDTH, dtype=np.int32)
            xs.append(x)
            ys.append(np.full_like(x, blk * BLOCK_HEIGHT))
    assert len(xs) > 0, "Issues with generating arrangement!"
    return (torch.from_numpy(np.concatenate(xs)).to(dev), torch.from_numpy(np.concatenate(ys)).to(dev))


def gen_block_mappings(mask, BLOCK_HEIGHT: int, BLOCK_WIDTH: int, GPU_ID, is_naive: bool = True):
    return naive_block_mappings(mask, BLOCK_HEIGHT, BLOCK_WIDTH, GPU_ID)


def rsddmm_preamble(mask, output_shape: tuple, BLOCK_SIZE_X: int, BLOCK_SIZE_Y: int, GPU_ID,
                    out_dtype: torch.dtype):
    """-> (output, grid_dim, tb_map_x, tb_map_y)   (reference SPLAT/r_sddmm.py:154-169).
    ``output`` is the (B, H, L, trailing_dim) ACSR score buffer the launcher writes in place."""
    dev = _n.resolve_device(GPU_ID)
    output = torch.empty(tuple(output_shape), dtype=out_dtype, device=dev)
    tb_map_x, tb_map_y = gen_block_mappings(mask, BLOCK_SIZE_Y, BLOCK_SIZE_X, dev)
    assert tb_map_x.shape == tb_map_y.shape, "Incorrect tiling arrangement!"
    grid_dim = (tb_map_x.shape[0], output_shape[0] * output_shape[1])
    return (output, grid_dim, tb_map_x, tb_map_y)


def rsddmm_launcher(x: torch.Tensor, y: torch.Tensor, output: torch.Tensor,
                    dTos_linear_transformations: torch.Tensor, dTos_translations: torch.Tensor,
                    sTod_linear_transformations: torch.Tensor, sTod_translations: torch.Tensor,
                    trailing_dim: int, nnzs: torch.Tensor, grid_dim, tb_map_x, tb_map_y,
                    BLOCK_SIZE_Y: int, BLOCK_SIZE_X: int):
    """x = Q (B,H,L,d), y = K^T (B,H,d,L) -> output (B,H,L,trailing_dim), written in place.
    Returns (output, sTod_linear_transformations, sTod_translations, nnzs) like the reference
    (SPLAT/r_sddmm.py:171-184).  Slots >= nnz of each row are written as zero."""
    _n.sddmm(x, y, output, sTod_linear_transformations, sTod_translations, nnzs, trailing_dim)
    return (output, sTod_linear_transformations, sTod_translations, nnzs)


def truth(x: torch.Tensor, y: torch.Tensor, GPU_ID) -> torch.Tensor:
    """Dense Q K^T (reference SPLAT/r_sddmm.py:186-188)."""
    return torch.einsum('bnqd, bndk -> bnqk', x, y)
