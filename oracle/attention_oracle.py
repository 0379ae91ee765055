"""CPU restatement of the SDDMM -> row softmax -> SpMM path over ACSR, in fp32 torch.

TEST INFRASTRUCTURE ONLY -- never imported by the shipped library.

Reference anchors:
  * SDDMM semantics ...... SPLAT/r_sddmm.py:16-115 and its checker ``truth``/``is_correct``
                           (SPLAT/r_sddmm.py:186-214): S[b,h,i,slot] = sum_k Q[b,h,i,k] *
                           Kt[b,h,k,col(i,slot)] for slot < nnz_i
  * softmax semantics .... SPLAT/r_softmax.py:17-59: numerically stable softmax over the first
                           nnz_i slots of each row, no scaling (``scale`` here defaults to 1)
  * SpMM semantics ....... SPLAT/r_spmm.py:14-126 and ``is_correct`` (SPLAT/r_spmm.py:166-216):
                           O[b,h,i,c] = sum_{slot<nnz_i} P[b,h,i,slot] * V[b,h,col(i,slot),c]
  * chain ................ SPLAT/r_attention.py:77-100

col(i, slot) = start_i + slot*stride_i with (start, stride, nnz) recovered from the float32
metadata by ``acsr_oracle.affine_ints``.  Inputs are taken in whatever dtype the caller rounded
them to and up-cast to fp32; all arithmetic and results are fp32.  Slots >= nnz_i are returned
as zero (the reference leaves them unwritten).
"""
from __future__ import annotations

import numpy as np
import torch

from .acsr_oracle import affine_ints


def _cols(meta, trailing_dim):
    start, stride, nnz = affine_ints(meta)
    slot = np.arange(trailing_dim)[None, :]
    cols = start[:, None] + slot * stride[:, None]
    valid = slot < nnz[:, None]
    cols = np.where(valid, cols, 0)
    return torch.from_numpy(cols), torch.from_numpy(valid)


def sddmm_acsr(q: torch.Tensor, kt: torch.Tensor, meta: dict, trailing_dim: int) -> torch.Tensor:
    """q (B,H,L,d), kt (B,H,d,L) -> S (B,H,L,trailing_dim) fp32."""
    q = q.float()
    k = kt.float().transpose(2, 3)                      # (B,H,L,d)
    cols, valid = _cols(meta, trailing_dim)             # (L,T)
    B, H, L, d = q.shape
    out = torch.zeros(B, H, L, trailing_dim, dtype=torch.float32)
    chunk = max(1, (1 << 24) // max(1, trailing_dim * d))
    for r0 in range(0, L, chunk):
        r1 = min(L, r0 + chunk)
        kg = k[:, :, cols[r0:r1].reshape(-1), :].reshape(B, H, r1 - r0, trailing_dim, d)
        s = torch.einsum("bhid,bhitd->bhit", q[:, :, r0:r1], kg)
        out[:, :, r0:r1] = s * valid[r0:r1]
    return out


def softmax_acsr(s: torch.Tensor, meta: dict, scale: float = 1.0) -> torch.Tensor:
    """Row softmax of scale*S over slots < nnz_i; other slots 0; rows with nnz 0 are all 0."""
    s = s.float()
    T = s.shape[-1]
    _cols_, valid = _cols(meta, T)
    z = torch.where(valid, s * scale, torch.full_like(s, float("-inf")))
    mx = z.max(dim=-1, keepdim=True).values
    mx = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))
    e = torch.exp(z - mx)
    den = e.sum(dim=-1, keepdim=True)
    return torch.where(den > 0, e / den, torch.zeros_like(e))


def lse_acsr(s: torch.Tensor, meta: dict, scale: float = 1.0) -> torch.Tensor:
    """Per-row log-sum-exp (natural log) of scale*S over slots < nnz_i, (B,H,L) fp32; -inf for rows
    with nnz 0.  The quantity a backward pass recomputes the probabilities from; the reference keeps
    it in registers only (SPLAT/r_softmax.py:17-58)."""
    s = s.float()
    _cols_, valid = _cols(meta, s.shape[-1])
    z = torch.where(valid, s * scale, torch.full_like(s, float("-inf")))
    return torch.logsumexp(z, dim=-1)


def spmm_acsr(p: torch.Tensor, v: torch.Tensor, meta: dict) -> torch.Tensor:
    """p (B,H,L,T) in ACSR layout, v (B,H,L,d) -> O (B,H,L,d) fp32."""
    p = p.float()
    v = v.float()
    B, H, L, T = p.shape
    d = v.shape[-1]
    cols, valid = _cols(meta, T)
    out = torch.zeros(B, H, L, d, dtype=torch.float32)
    chunk = max(1, (1 << 24) // max(1, T * d))
    for r0 in range(0, L, chunk):
        r1 = min(L, r0 + chunk)
        vg = v[:, :, cols[r0:r1].reshape(-1), :].reshape(B, H, r1 - r0, T, d)
        out[:, :, r0:r1] = torch.einsum("bhit,bhitd->bhid", p[:, :, r0:r1] * valid[r0:r1], vg)
    return out


def attention_acsr(q, kt, v, meta: dict, trailing_dim: int, scale: float = 1.0) -> torch.Tensor:
    """The chain of SPLAT/r_attention.py:77-100 on fp32 intermediates."""
    s = sddmm_acsr(q, kt, meta, trailing_dim)
    p = softmax_acsr(s, meta, scale)
    return spmm_acsr(p, v, meta)


def attention_dense_masked(q, kt, v, mask_eff, scale: float = 1.0) -> torch.Tensor:
    """``truth`` (SPLAT/r_sddmm.py:186-187: einsum 'bnqd,bndk->bnqk') -> mask with the
    metadata-effective mask -> softmax -> @V.  O(L^2): small cases only.  Independent of the ACSR
    index arithmetic, so it also checks ``attention_acsr``."""
    s = torch.einsum("bnqd,bndk->bnqk", q.float(), kt.float()) * scale
    m = torch.as_tensor(np.asarray(mask_eff) != 0)
    s = s.masked_fill(~m, float("-inf"))
    mx = s.max(dim=-1, keepdim=True).values
    mx = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))
    e = torch.exp(s - mx)
    den = e.sum(dim=-1, keepdim=True)
    p = torch.where(den > 0, e / den, torch.zeros_like(e))
    return p @ v.float()
