"""GPU: the five benchmark configurations.  Config 1 in full against the oracle; configs 2-5 on
reduced head counts against the oracle (full sequence length, sampled heads) and, at full size,
through size-independent properties: agreement of two independent kernels, V = const gives
O = const on rows with non-zeros, and invariance under (batch, head) sharding."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from oracle import acsr_oracle as ao
from oracle import attention_oracle as at

pytestmark = pytest.mark.gpu

#  name: (B, H, L, d, dtype, pattern kind, p0, p1, input scale, seed)
CONFIGS = {
    1: (1, 2, 256, 32, torch.float32, ao.PATTERN_CAUSAL_WINDOWED, 31, 0, 1.0, 0),
    2: (4, 16, 4096, 64, torch.float16, ao.PATTERN_CAUSAL_WINDOWED, 255, 0, 1.0, 1),
    3: (2, 32, 8192, 128, torch.bfloat16, ao.PATTERN_STRIDED, 64, 0, 1.0, 2),
    4: (1, 32, 16384, 128, torch.bfloat16, ao.PATTERN_DILATED, 512, 2, 0.5, 3),
    5: (8, 64, 32768, 128, torch.bfloat16, ao.PATTERN_CAUSAL_WINDOWED, 1023, 0, 1.0, 4),
}


def _inputs(cfg, heads, device="cuda"):
    B, H, L, d, dtype, kind, p0, p1, spread, seed = CONFIGS[cfg]
    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda: (torch.randn(1, heads, L, d, generator=g, device=device) * spread).to(dtype)
    return mk(), mk(), mk()


def _module(cfg, heads, **kw):
    import acsr_helpers as ah
    import r_attention
    B, H, L, d, dtype, kind, p0, p1, spread, seed = CONFIGS[cfg]
    mask = ah.PatternMask(kind, L, p0, p1)
    return r_attention.RegularAttention(1, L, heads, d, mask, 16, 16, 0, dtype, scale=d ** -0.5, **kw)


def test_config1_full():
    import splat_native as n
    B, H, L, d, dtype, kind, p0, p1, spread, seed = CONFIGS[1]
    meta = ao.metadata_from_pattern(kind, L, p0, p1, 16)
    torch.manual_seed(seed)
    q, k, v = (torch.randn(B, H, L, d) for _ in range(3))
    ref = at.attention_acsr(q, k.transpose(2, 3), v, meta, 32, d ** -0.5)
    for fused in (True, False):
        attn = _module(1, H, fused=fused)
        out = attn([q.cuda(), k.cuda().transpose(2, 3), v.cuda()])
        assert_close(out, ref, dtype, f"config 1 fused={fused}")


@pytest.mark.parametrize("cfg", [2, 3, 4, 5])
def test_config_sampled_heads_against_oracle(cfg, monkeypatch):
    """Full sequence length and pattern, two heads, every row compared with the CPU oracle -- for
    the kernel the library picks at this size and for each of the three band kernels forced
    (1: one Q tile per CTA, 2: two Q tiles per CTA, the kernel the full-size benchmark of
    configuration 5 runs, 3: CTA pairs)."""
    import splat_native as n
    B, H, L, d, dtype, kind, p0, p1, spread, seed = CONFIGS[cfg]
    heads = 2
    q, k, v = _inputs(cfg, heads)
    meta = ao.metadata_from_pattern(kind, L, p0, p1, 16)
    ref = at.attention_acsr(q.cpu(), k.cpu().transpose(2, 3), v.cpu(), meta, meta["trailing_dim"],
                            d ** -0.5)
    for variant in (None, "1", "2", "3"):
        if variant is None:
            monkeypatch.delenv("SPLAT_B200_BAND_TILES", raising=False)
        else:
            monkeypatch.setenv("SPLAT_B200_BAND_TILES", variant)
        attn = _module(cfg, heads, path=n.PATH_BAND)
        out = attn([q, k.transpose(2, 3), v])
        attn.check_status()
        assert_close(out, ref, dtype, f"config {cfg} band kernel {variant or 'auto'}")
    monkeypatch.delenv("SPLAT_B200_BAND_TILES", raising=False)
    # the three-launch path of the reference API on the same inputs (one head: S and P are large)
    attn3 = _module(cfg, 1, fused=False)
    out3 = attn3([q[:, :1].contiguous(), k[:, :1].contiguous().transpose(2, 3), v[:, :1].contiguous()])
    assert_close(out3, ref[:, :1], dtype, f"config {cfg} three-launch")


@pytest.mark.parametrize("cfg", [2, 3, 4, 5])
def test_config_full_size_properties(cfg):
    import splat_native as n
    from sharding import shard_range
    B, H, L, d, dtype, kind, p0, p1, spread, seed = CONFIGS[cfg]
    heads = B * H
    q, k, v = _inputs(cfg, heads)
    attn = _module(cfg, heads, path=n.PATH_BAND)
    out = attn([q, k.transpose(2, 3), v]).clone()
    attn.check_status()
    assert torch.isfinite(out.float()).all()
    # (1) two independent kernels agree on a slab of heads
    hs = slice(0, min(heads, 4))
    gen = torch.empty_like(out[:, hs])
    n.attention_fused(q[:, hs].contiguous(), k[:, hs].contiguous().transpose(2, 3),
                      v[:, hs].contiguous(), gen, attn.sTod_linear_transformations,
                      attn.sTod_translations, attn.nnzs, d ** -0.5, n.PATH_GENERIC)
    assert_close(out[:, hs], gen.float(), dtype, f"config {cfg} band vs generic")
    # (2) sharding invariance: each rank's slice computed alone is bit-identical
    for world in (2, 8):
        b, e = shard_range(heads, world, world - 1)
        part = _module(cfg, e - b, path=n.PATH_BAND)
        o = part([q[:, b:e].contiguous(), k[:, b:e].contiguous().transpose(2, 3),
                  v[:, b:e].contiguous()])
        assert torch.equal(o, out[:, b:e]), f"config {cfg} shard {world}"
    # (3) probabilities sum to one: constant V comes back unchanged
    ones = torch.full_like(v, 0.5)
    o1 = attn([q, k.transpose(2, 3), ones])
    attn.check_status()
    assert (o1.float() - 0.5).abs().max() < 4e-3
