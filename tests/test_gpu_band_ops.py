"""GPU: the tensor-core SDDMM and SpMM for band patterns against the CPU oracle and against the
CUDA-core kernels, over the same patterns as the fused band kernel plus rows without a band."""
import pytest
import torch

from conftest import assert_close
from oracle import acsr_oracle as ao
from oracle import attention_oracle as at

pytestmark = pytest.mark.gpu

#        kind, L, p0, p1
PATTERNS = [
    (ao.PATTERN_CAUSAL_WINDOWED, 512, 63, 0),
    (ao.PATTERN_CAUSAL_WINDOWED, 200, 31, 0),     # ragged: L not a multiple of 64
    (ao.PATTERN_CAUSAL_WINDOWED, 1024, 1023, 0),  # dense causal
    (ao.PATTERN_WINDOWED, 640, 100, 0),
    (ao.PATTERN_BLOCKED, 512, 96, 0),
    (ao.PATTERN_STRIDED, 512, 4, 0),              # residue classes, single-element rows
    (ao.PATTERN_STRIDED, 1024, 64, 0),
    (ao.PATTERN_DILATED, 1024, 40, 2),
    (ao.PATTERN_DILATED, 768, 200, 3),
]


def _meta(kind, L, p0, p1):
    import acsr_helpers as ah
    acsr = ah.create_acsr(ah.PatternMask(kind, L, p0, p1), 16, 0)
    return acsr, ao.metadata_from_pattern(kind, L, p0, p1, 16)


def _check_ops(acsr, meta, L, d, dtype, seed, what):
    import splat_native as n
    torch.manual_seed(seed)
    T = int(meta["trailing_dim"])
    B, H = 1, 3
    q, k, v = (torch.randn(B, H, L, d).to(dtype) for _ in range(3))
    # --- SDDMM
    s_ref = at.sddmm_acsr(q, k.transpose(2, 3), meta, T)
    s_band = torch.full((B, H, L, T), float("nan"), dtype=dtype, device="cuda")
    n.sddmm(q.cuda(), k.cuda().transpose(2, 3), s_band, acsr[2], acsr[3], acsr[4], T, n.PATH_BAND)
    n.check_status_word(0)
    assert_close(s_band, s_ref, dtype, f"sddmm band {what}")
    s_gen = torch.full_like(s_band, float("nan"))
    n.sddmm(q.cuda(), k.cuda().transpose(2, 3), s_gen, acsr[2], acsr[3], acsr[4], T, n.PATH_GENERIC)
    # both round an fp32 sum once; the summation order differs
    assert (s_band.float() - s_gen.float()).abs().max() <= 0.02 * (1 + s_gen.float().abs().max())
    _cols, valid = at._cols(meta, T)
    assert torch.count_nonzero(s_band.cpu().float() * (~valid)) == 0, "padding slots must be zero"
    # --- SpMM: probabilities in the sparse layout, NaN in the padding (must not be read)
    p = torch.rand(B, H, L, T)
    p_dev = torch.where(valid, p, torch.full_like(p, float("nan"))).to(dtype).cuda()
    o_ref = at.spmm_acsr(p.to(dtype), v, meta)
    o_band = torch.full((B, H, L, d), float("nan"), dtype=dtype, device="cuda")
    n.spmm(p_dev, v.cuda(), o_band, acsr[2], acsr[3], acsr[4], T, n.PATH_BAND)
    n.check_status_word(0)
    assert_close(o_band, o_ref, dtype, f"spmm band {what}")


@pytest.mark.parametrize("d", [128, 64])
def test_band_ops_first_light(d):
    acsr, meta = _meta(ao.PATTERN_CAUSAL_WINDOWED, 256, 99, 0)
    _check_ops(acsr, meta, 256, d, torch.bfloat16, 1, f"first light d={d}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [128, 64])
def test_band_ops_patterns(d, dtype):
    for i, (kind, L, p0, p1) in enumerate(PATTERNS):
        acsr, meta = _meta(kind, L, p0, p1)
        _check_ops(acsr, meta, L, d, dtype, 200 + i, f"{(kind, L, p0, p1)} d={d}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [128, 64])
def test_band_sddmm_contiguous_kt(d, dtype):
    """The reference's K^T layout, contiguous (B,H,d,L) (SPLAT/r_sddmm.py:24-37), through the
    tensor-core SDDMM for the stride-1 patterns; bit-identical to the transposed-view layout."""
    import splat_native as n
    for i, (kind, L, p0, p1) in enumerate(PATTERNS):
        if kind in (ao.PATTERN_STRIDED, ao.PATTERN_DILATED) or L % 8 != 0:
            continue
        acsr, meta = _meta(kind, L, p0, p1)
        T = int(meta["trailing_dim"])
        torch.manual_seed(400 + i)
        q, k = (torch.randn(1, 3, L, d).to(dtype) for _ in range(2))
        s_ref = at.sddmm_acsr(q, k.transpose(2, 3), meta, T)
        outs = []
        for kt in (k.cuda().transpose(2, 3).contiguous(), k.cuda().transpose(2, 3)):
            s_band = torch.full((1, 3, L, T), float("nan"), dtype=dtype, device="cuda")
            n.sddmm(q.cuda(), kt, s_band, acsr[2], acsr[3], acsr[4], T, n.PATH_BAND)
            n.check_status_word(0)
            outs.append(s_band)
        assert_close(outs[0], s_ref, dtype, f"sddmm band, contiguous K^T {(kind, L, p0, p1)} d={d}")
        assert torch.equal(outs[0], outs[1])


def test_band_ops_rows_without_a_band():
    """Empty rows, a row with one non-zero away from column 0, odd trailing dimension."""
    import acsr_helpers as ah
    L = 256
    mask = ao.causal_windowed_mask(L, 40)
    mask[5:9, :] = 0
    mask[100, :] = 0
    mask[100, 37] = 1
    mask[255, :] = 0
    acsr = ah.create_acsr(mask.tolist(), 16, 0)
    meta = ao.metadata_from_mask(mask, 16)
    assert int(meta["trailing_dim"]) % 2 == 1
    _check_ops(acsr, meta, L, 64, torch.bfloat16, 5, "rows without a band")


def test_unfused_module_uses_the_band_ops_and_matches_the_fused_kernel():
    import acsr_helpers as ah
    import r_attention
    torch.manual_seed(9)
    B, H, L, d = 1, 2, 1024, 128
    mask = ah.create_causal_windowed_mask(L, 255)
    q, k, v = (torch.randn(B, H, L, d, device="cuda").to(torch.bfloat16) for _ in range(3))
    outs = []
    for fused in (False, True):
        attn = r_attention.RegularAttention(B, L, H, d, mask, 16, 16, 0, torch.bfloat16,
                                            scale=d ** -0.5, fused=fused)
        outs.append(attn([q, k.transpose(2, 3), v]).float().clone())
        attn.check_status()
    meta = ao.metadata_from_pattern(ao.PATTERN_CAUSAL_WINDOWED, L, 255, 0, 16)
    ref = at.attention_acsr(q.cpu(), k.cpu().transpose(2, 3), v.cpu(), meta, int(meta["trailing_dim"]), d ** -0.5)
    assert_close(outs[0], ref, torch.bfloat16, "unfused chain")
    assert_close(outs[1], ref, torch.bfloat16, "fused kernel")
