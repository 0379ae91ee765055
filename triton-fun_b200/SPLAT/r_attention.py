"""Sparse-regular attention module: SDDMM -> softmax -> SpMM over one ACSR mask.

Drop-in for the reference module SPLAT/r_attention.py (``RegularAttention``, ``unit``).  The
constructor keeps the reference's positional parameters; keyword-only extras:

  scale  softmax scale folded into the exponent.  Default 1.0 = the reference, which applies none.
  fused  True (default): ``forward`` is ONE kernel and the (B,H,L,trailing_dim) score/probability
         buffers are never allocated.  False: the reference's three launches through
         ``rsddmm_launcher`` / ``rsoftmax_launcher`` / ``rspmm_launcher``.
  path   ``splat_native.PATH_AUTO`` / ``PATH_GENERIC`` / ``PATH_BAND`` for the fused kernel.

``forward([q, k^T, v])`` takes q, v as contiguous (B,H,L,d) and k^T as (B,H,d,L) -- pass
``k.transpose(2, 3)`` of a contiguous (B,H,L,d) tensor to reach the tensor-core path -- and
returns the module-owned output buffer (the same tensor object on every call, as in the reference).
"""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

import splat_native as _n
from acsr_helpers import create_acsr, create_blocked_mask, create_windowed_mask, create_causal_windowed_mask  # noqa: F401
from r_sddmm import rsddmm_launcher, rsddmm_preamble
from r_softmax import rsoftmax_launcher, rsoftmax_preamble
from r_spmm import rspmm_launcher, rspmm_preamble


class RegularAttention(nn.Module):

    def __init__(self, batch: int, seq_length: int, num_heads: int, head_dim: int, mask,
                 BLOCK_SIZE_Y: int, BLOCK_SIZE_X: int, GPU_ID: Any, out_dtype: torch.dtype, *,
                 scale: float = 1.0, fused: bool = True, path: int = _n.PATH_AUTO, lse: bool = False):
        """Positional parameters as in the reference (SPLAT/r_attention.py:14-16).  Keyword-only
        additions: scale (softmax scale, the reference applies none), fused (one kernel instead of
        the three launches), path (kernel selection), lse (fused path only: keep a float32 (B,H,L)
        buffer self.lse that every forward fills with the rows' log-sum-exp of the scaled scores)."""
        super().__init__()
        self.device = _n.resolve_device(GPU_ID)
        self.scale, self.fused, self.path = float(scale), bool(fused), int(path)
        self.out_dtype = out_dtype
        self._shape = (batch, num_heads, seq_length, head_dim)

        ## Create the ACSR (reference SPLAT/r_attention.py:23-26).
        (self.dTos_linear_transformations, self.dTos_translations,
         self.sTod_linear_transformations, self.sTod_translations,
         self.nnzs, self.acsr_trailing_dim,
         self.span_loop_start, self.span_loop_end) = create_acsr(mask, BLOCK_SIZE_Y, self.device)
        self.plan = _n.classify(self.sTod_linear_transformations, self.sTod_translations, self.nnzs)

        self.BLOCK_SIZE_Y = BLOCK_SIZE_Y
        self.BLOCK_SIZE_X = BLOCK_SIZE_X

        if lse and not self.fused:
            raise ValueError("lse=True needs the fused path (the three launches keep no row sums)")
        self.lse = (torch.empty((batch, num_heads, seq_length), dtype=torch.float32, device=self.device)
                    if lse else None)
        self.rsddmm_output = self.rsoftmax_output = None
        self.rsddmm_grid_dim = self.rsddmm_tb_map_x = self.rsddmm_tb_map_y = None
        self.rsoftmax_grid_dim = self.rsoftmax_trailing_dim_pow_two = None
        self._mask = mask
        if not self.fused:
            self._unfused_preambles()

        ## rSpMM preamble: owns the (B,H,L,d) output buffer of both paths.
        self.rspmm_output, self.rspmm_grid_dim, _ = rspmm_preamble(
            mask, (batch, num_heads, seq_length, head_dim), BLOCK_SIZE_X, BLOCK_SIZE_Y,
            self.device, out_dtype)

    def _unfused_preambles(self):
        batch, num_heads, seq_length, _ = self._shape
        acsr_shape = (batch, num_heads, seq_length, self.acsr_trailing_dim)
        (self.rsddmm_output, self.rsddmm_grid_dim, self.rsddmm_tb_map_x,
         self.rsddmm_tb_map_y) = rsddmm_preamble(self._mask, acsr_shape, self.BLOCK_SIZE_X,
                                                 self.BLOCK_SIZE_Y, self.device, self.out_dtype)
        (self.rsoftmax_grid_dim, self.rsoftmax_output, _,
         self.rsoftmax_trailing_dim_pow_two) = rsoftmax_preamble(
            self._mask, acsr_shape, self.BLOCK_SIZE_X, self.device, self.out_dtype)

    ## Input x should already be in query/key/value post RoPe application.
    def forward(self, x):
        q, k, v = x
        if self.fused:
            _n.attention_fused(q, k, v, self.rspmm_output, self.sTod_linear_transformations,
                               self.sTod_translations, self.nnzs, self.scale, self.path, self.plan,
                               lse=self.lse)
            return self.rspmm_output
        if self.rsddmm_output is None:
            self._unfused_preambles()
        rsddmm_launcher(q, k, self.rsddmm_output,
                        self.dTos_linear_transformations, self.dTos_translations,
                        self.sTod_linear_transformations, self.sTod_translations,
                        self.acsr_trailing_dim, self.nnzs,
                        self.rsddmm_grid_dim, self.rsddmm_tb_map_x,
                        self.rsddmm_tb_map_y, self.BLOCK_SIZE_Y, self.BLOCK_SIZE_X)
        rsoftmax_launcher(self.rsddmm_output, self.rsoftmax_output,
                          self.dTos_linear_transformations, self.dTos_translations,
                          self.sTod_linear_transformations, self.sTod_translations,
                          self.acsr_trailing_dim, self.rsoftmax_trailing_dim_pow_two, self.nnzs,
                          self.rsoftmax_grid_dim, self.BLOCK_SIZE_X, scale=self.scale)
        rspmm_launcher(self.rsoftmax_output, v, self.rspmm_output,
                       self.dTos_linear_transformations, self.dTos_translations,
                       self.sTod_linear_transformations, self.sTod_translations,
                       self.span_loop_start, self.span_loop_end, self.acsr_trailing_dim,
                       self.nnzs, self.rspmm_grid_dim, self.BLOCK_SIZE_Y, self.BLOCK_SIZE_X)
        return self.rspmm_output

    def forward_host(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
                     out_host: torch.Tensor, chunk_heads: int = 32) -> torch.Tensor:
        """Attention over HOST-resident operands (pinned (B,H,L,d) tensors; k is row-major, not
        transposed).  The flat batch*head axis is streamed through the device in chunks of
        ``chunk_heads``: the host->device copy of chunk i+1 and the device->host copy of chunk
        i-1 overlap the fused kernel of chunk i (three streams, two staging buffers, allocated on
        first use).  Work is enqueued asynchronously; the caller's current stream waits for the last
        device->host copy, so synchronising that stream makes ``out_host`` valid.  Not in the
        reference, whose operands are always device tensors."""
        B, H, L, d = q_host.shape
        bh = B * H
        qh, kh, vh, oh = (t.view(1, bh, L, d) for t in (q_host, k_host, v_host, out_host))
        chunk = max(1, min(chunk_heads, bh))
        st = getattr(self, "_host_stage", None)
        if st is None or st["chunk"] != chunk or st["shape"] != (L, d):
            mk = lambda: torch.empty((1, chunk, L, d), dtype=self.out_dtype, device=self.device)
            st = {"chunk": chunk, "shape": (L, d),
                  "bufs": [{"q": mk(), "k": mk(), "v": mk(), "o": mk(),
                            "in_ready": torch.cuda.Event(), "done": torch.cuda.Event(),
                            "out_free": torch.cuda.Event()} for _ in range(2)],
                  "s_in": torch.cuda.Stream(self.device), "s_out": torch.cuda.Stream(self.device)}
            self._host_stage = st
        cur = torch.cuda.current_stream(self.device)
        s_in, s_out = st["s_in"], st["s_out"]
        s_in.wait_stream(cur)
        for i, b in enumerate(range(0, bh, chunk)):
            e = min(bh, b + chunk)
            n = e - b
            buf = st["bufs"][i % 2]
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(buf["done"])        # kernel of chunk i-2 has read its inputs
                buf["q"][:, :n].copy_(qh[:, b:e], non_blocking=True)
                buf["k"][:, :n].copy_(kh[:, b:e], non_blocking=True)
                buf["v"][:, :n].copy_(vh[:, b:e], non_blocking=True)
                buf["in_ready"].record(s_in)
            cur.wait_event(buf["in_ready"])
            if i >= 2:
                cur.wait_event(buf["out_free"])         # output of chunk i-2 has left the device
            _n.attention_fused(buf["q"][:, :n], buf["k"][:, :n].transpose(2, 3), buf["v"][:, :n],
                               buf["o"][:, :n], self.sTod_linear_transformations,
                               self.sTod_translations, self.nnzs, self.scale, self.path, self.plan)
            buf["done"].record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(buf["done"])
                oh[:, b:e].copy_(buf["o"][:, :n], non_blocking=True)
                buf["out_free"].record(s_out)
        cur.wait_stream(s_out)
        return out_host

    def check_status(self) -> None:
        """Synchronise and raise if the tensor-core kernel reported a timed-out device wait."""
        _n.check_status_word(self.device)


def unit(q, k, v, w_q, w_k, w_v, attn: RegularAttention):
    """Per-head projections followed by attention (reference SPLAT/r_attention.py:102-110).  The
    projections are emitted head-major, (B, heads, L, d), which is the layout the kernels index."""
    q = torch.einsum('bsd, dnh -> bnsh', q, w_q).contiguous()
    k = torch.einsum('bsd, dnh -> bnsh', k, w_k).contiguous()
    v = torch.einsum('bsd, dnh -> bnsh', v, w_v).contiguous()
    return attn([q, k.transpose(2, 3), v])
