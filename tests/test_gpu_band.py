"""GPU: the TMA + tcgen05 band kernels (one Q tile per CTA, two Q tiles per CTA, CTA pairs) against the CPU oracle, over window / blocked / strided / dilated patterns, ragged sizes and both 16-bit dtypes."""
import pytest
import torch

from conftest import assert_close
from oracle import acsr_oracle as ao
from oracle import attention_oracle as at

pytestmark = pytest.mark.gpu

#        kind, L, p0, p1
PATTERNS = [
    (ao.PATTERN_CAUSAL_WINDOWED, 512, 63, 0),     # several key tiles, clipped head rows
    (ao.PATTERN_CAUSAL_WINDOWED, 384, 255, 0),    # second Q tile of the last pair partly empty
    (ao.PATTERN_CAUSAL_WINDOWED, 200, 31, 0),     # L < 256, not a multiple of 128
    (ao.PATTERN_CAUSAL_WINDOWED, 1024, 1023, 0),  # dense causal
    (ao.PATTERN_WINDOWED, 640, 100, 0),           # two-sided window
    (ao.PATTERN_BLOCKED, 512, 96, 0),             # block-banded
    (ao.PATTERN_STRIDED, 512, 4, 0),              # 4 residue classes of 128 rows; single-nnz rows
    (ao.PATTERN_STRIDED, 1024, 64, 0),            # 64 classes of 16 rows
    (ao.PATTERN_DILATED, 1024, 40, 2),            # two classes, window 40
    (ao.PATTERN_DILATED, 768, 200, 3),            # three classes
]


@pytest.fixture(params=["1", "2", "3"], ids=["one-tile-ctas", "paired-tile-ctas", "cta-pairs"], autouse=True)
def band_variant(request, monkeypatch):
    """Every test runs against the three band kernels: one Q tile per CTA (two CTAs per SM), two Q
    tiles per CTA, and persistent CTA pairs (cta_group::2; d = 128 only, d = 64 falls back to the
    two-tile kernel).  The library reads the override at each call."""
    monkeypatch.setenv("SPLAT_B200_BAND_TILES", request.param)
    return request.param


def _run(kind, L, p0, p1, d, dtype, seed, BH=(1, 3), scale=None, spread=1.0, kt_contiguous=False):
    """kt_contiguous: pass K^T as a contiguous (B,H,d,L) tensor, the layout the reference's kernels
    index (SPLAT/r_sddmm.py:24-37), instead of the transposed view of a (B,H,L,d) tensor."""
    import acsr_helpers as ah
    import splat_native as n
    torch.manual_seed(seed)
    acsr = ah.create_acsr(ah.PatternMask(kind, L, p0, p1), 16, 0)
    meta = ao.metadata_from_pattern(kind, L, p0, p1, 16)
    B, H = BH
    q, k, v = (torch.randn(B, H, L, d).mul_(spread).to(dtype) for _ in range(3))
    scale = d ** -0.5 if scale is None else scale
    out = torch.full((B, H, L, d), float("nan"), dtype=dtype, device="cuda")
    kt = k.cuda().transpose(2, 3)
    if kt_contiguous:
        kt = kt.contiguous()
    n.attention_fused(q.cuda(), kt, v.cuda(), out, acsr[2], acsr[3], acsr[4], scale, n.PATH_BAND)
    n.check_status_word(0)
    ref = at.attention_acsr(q, k.transpose(2, 3), v, meta, meta["trailing_dim"], scale)
    return out, ref


@pytest.mark.parametrize("d", [128, 64])
def test_band_first_light(d):
    """Smallest interesting case first: if this fails the rest is skipped by -x."""
    out, ref = _run(ao.PATTERN_CAUSAL_WINDOWED, 256, 99, 0, d, torch.bfloat16, 1)
    assert_close(out, ref, torch.bfloat16, f"first light d={d}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [128, 64])
def test_band_patterns(d, dtype):
    for i, (kind, L, p0, p1) in enumerate(PATTERNS):
        out, ref = _run(kind, L, p0, p1, d, dtype, 100 + i)
        assert_close(out, ref, dtype, f"pattern {(kind, L, p0, p1)} d={d}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [128, 64])
def test_band_contiguous_kt(d, dtype):
    """The reference's own K^T layout, contiguous (B,H,d,L), on the tensor-core path: every
    stride-1 pattern of the list (strided and dilated patterns take that layout on the CUDA-core
    path only and are refused here)."""
    import splat_native as n
    for i, (kind, L, p0, p1) in enumerate(PATTERNS):
        if L % 8 != 0:
            continue
        if kind in (ao.PATTERN_STRIDED, ao.PATTERN_DILATED):
            with pytest.raises(RuntimeError):
                _run(kind, L, p0, p1, d, dtype, 300 + i, kt_contiguous=True)
            continue
        out, ref = _run(kind, L, p0, p1, d, dtype, 300 + i, kt_contiguous=True)
        assert_close(out, ref, dtype, f"contiguous K^T, pattern {(kind, L, p0, p1)} d={d}")


def test_band_unscaled_scores_need_the_running_max():
    """scale = 1 with d = 128 gives scores of sigma ~ 11: exercises the lazy rescale of O."""
    for d in (128, 64):
        out, ref = _run(ao.PATTERN_CAUSAL_WINDOWED, 1024, 511, 0, d, torch.bfloat16, 7, scale=1.0)
        assert_close(out, ref, torch.bfloat16, f"unscaled d={d}")


def test_band_matches_generic_kernel_and_is_deterministic():
    import acsr_helpers as ah
    import splat_native as n
    torch.manual_seed(9)
    L, d = 2048, 128
    acsr = ah.create_acsr(ah.create_causal_windowed_mask(L, 300), 16, 0)
    q, k, v = (torch.randn(2, 4, L, d, device="cuda").to(torch.bfloat16) for _ in range(3))
    outs = []
    for path in (n.PATH_BAND, n.PATH_BAND, n.PATH_GENERIC):
        o = torch.empty_like(q)
        n.attention_fused(q, k.transpose(2, 3), v, o, acsr[2], acsr[3], acsr[4], d ** -0.5, path)
        outs.append(o)
    n.check_status_word(0)
    assert torch.equal(outs[0], outs[1])
    assert_close(outs[0], outs[2].float(), torch.bfloat16, "band vs generic")


def test_band_path_refuses_what_it_cannot_do():
    import acsr_helpers as ah
    import splat_native as n
    L, d = 256, 128
    acsr = ah.create_acsr(ah.create_causal_windowed_mask(L, 31), 16, 0)
    q = torch.randn(1, 1, L, d, device="cuda").to(torch.bfloat16)
    o = torch.empty_like(q)
    kt_contig = q.transpose(2, 3).contiguous()
    # contiguous K^T is fine for a stride-1 pattern ...
    n.attention_fused(q, kt_contig, q, o, acsr[2], acsr[3], acsr[4], 1.0, n.PATH_BAND)
    # ... but a pattern with stride > 1 takes that layout on the CUDA-core kernels only
    acsr_d = ah.create_acsr(ah.create_dilated_mask(L, 20, 2), 16, 0)
    with pytest.raises(RuntimeError):
        n.attention_fused(q, kt_contig, q, o, acsr_d[2], acsr_d[3], acsr_d[4], 1.0, n.PATH_BAND)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        n.attention_fused(q, kt_contig, q, o, acsr_d[2], acsr_d[3], acsr_d[4], 1.0, n.PATH_AUTO)  # falls back
    q32 = q.float()
    with pytest.raises(RuntimeError):      # fp32 has no band path
        n.attention_fused(q32, q32.transpose(2, 3), q32, torch.empty_like(q32), acsr[2], acsr[3],
                          acsr[4], 1.0, n.PATH_BAND)
    torch.cuda.synchronize()


def test_auto_path_takes_operands_the_band_path_cannot():
    """Operands that are not 16-byte aligned: the tensor-core path refuses them when asked for
    explicitly and SPLAT_PATH_AUTO computes the result with the general kernel."""
    import acsr_helpers as ah
    import splat_native as n
    L, d = 256, 128
    acsr = ah.create_acsr(ah.create_causal_windowed_mask(L, 63), 16, 0)
    meta = ao.metadata_from_pattern(ao.PATTERN_CAUSAL_WINDOWED, L, 63, 0, 16)
    torch.manual_seed(3)
    pool = torch.randn(2, L * d + 8, device="cuda").to(torch.bfloat16)
    # Q and K views that start one element (2 bytes) into their allocation; V and O stay aligned
    # (the general fused kernel reads V and writes O in 16-byte vectors)
    q, k = (pool[i, 1:1 + L * d].view(1, 1, L, d) for i in range(2))
    v = torch.randn(1, 1, L, d, device="cuda").to(torch.bfloat16)
    o = torch.empty_like(v)
    assert q.data_ptr() % 16 != 0 and k.data_ptr() % 16 != 0
    with pytest.raises(RuntimeError):
        n.attention_fused(q, k.transpose(2, 3), v, o, acsr[2], acsr[3], acsr[4], d ** -0.5, n.PATH_BAND)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        n.attention_fused(q, k.transpose(2, 3), v, o, acsr[2], acsr[3], acsr[4], d ** -0.5, n.PATH_AUTO)
    ref = at.attention_acsr(q.cpu(), k.cpu().transpose(2, 3), v.cpu(), meta, meta["trailing_dim"], d ** -0.5)
    assert_close(o, ref, torch.bfloat16, "unaligned operands through AUTO")


def test_launcher_reports_an_earlier_timeout():
    """The Python launchers keep a pinned mirror of the status word: launches made after a kernel
    gave up raise (within _MIRROR_EVERY launches) instead of returning untouched output buffers."""
    import acsr_helpers as ah
    import splat_native as n
    L, d = 256, 128
    acsr = ah.create_acsr(ah.create_causal_windowed_mask(L, 63), 16, 0)
    q = torch.randn(1, 1, L, d, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    dev = torch.device("cuda", 0)
    n.attention_fused(q, q.transpose(2, 3), q, out, acsr[2], acsr[3], acsr[4], 0.125, n.PATH_BAND)
    torch.cuda.synchronize()
    n.status_word(dev).fill_(5)            # as if a wait had run out inside that kernel
    # later launches are no-ops on the device; the mirror is refreshed at least once per
    # _MIRROR_EVERY launches, so one of them must raise
    with pytest.raises(RuntimeError):
        for _ in range(n._MIRROR_EVERY + 2):
            n.attention_fused(q, q.transpose(2, 3), q, out, acsr[2], acsr[3], acsr[4], 0.125, n.PATH_BAND)
            torch.cuda.synchronize()       # lets a mirror copy land
    # the raise cleared the word: back to normal
    n.attention_fused(q, q.transpose(2, 3), q, out, acsr[2], acsr[3], acsr[4], 0.125, n.PATH_BAND)
    n.check_status_word(0)


def test_bounded_wait_gives_up_and_reports(band_variant):
    """A device-side wait that can never complete (an mbarrier nothing arrives on) must run out
    after its cycle limit, leave code 99 in the status word and end the kernel normally; the band
    kernel must still work afterwards and must do nothing while the status word is set."""
    import acsr_helpers as ah
    import splat_native as n
    if band_variant != "1":
        pytest.skip("one run is enough")
    word = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = n._lib.splat_selftest_bounded_wait(word.data_ptr(), 200000, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert word.item() == 99
    # a band kernel launched while the status word is set leaves the output untouched ...
    L, d = 256, 64
    acsr = ah.create_acsr(ah.create_causal_windowed_mask(L, 63), 16, 0)
    q = torch.randn(1, 1, L, d, device="cuda").to(torch.bfloat16)
    sw = n.status_word(torch.device("cuda", 0))
    sw.fill_(7)
    out = torch.full_like(q, 3.0)
    n.attention_fused(q, q.transpose(2, 3), q, out, acsr[2], acsr[3], acsr[4], 0.125, n.PATH_BAND)
    torch.cuda.synchronize()
    assert (out == 3.0).all()
    with pytest.raises(RuntimeError):
        n.check_status_word(0)          # reports and clears
    # ... and works again once it is cleared
    n.attention_fused(q, q.transpose(2, 3), q, out, acsr[2], acsr[3], acsr[4], 0.125, n.PATH_BAND)
    n.check_status_word(0)
    assert torch.isfinite(out.float()).all() and not (out == 3.0).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_band_log_sum_exp_output(dtype, band_variant):
    """The optional (B,H,L) fp32 output of the fused call: log-sum-exp of the scaled scores of every
    row, from each tensor-core kernel -- band rows, rows with a single non-zero (the strided
    pattern has them), rows without non-zeros would be -inf."""
    import acsr_helpers as ah
    import splat_native as n
    d = 128
    for i, (kind, L, p0, p1) in enumerate([PATTERNS[0], PATTERNS[2], PATTERNS[4], PATTERNS[6], PATTERNS[8]]):
        torch.manual_seed(500 + i)
        acsr = ah.create_acsr(ah.PatternMask(kind, L, p0, p1), 16, 0)
        meta = ao.metadata_from_pattern(kind, L, p0, p1, 16)
        q, k, v = (torch.randn(1, 3, L, d).to(dtype) for _ in range(3))
        out = torch.empty(1, 3, L, d, dtype=dtype, device="cuda")
        lse = torch.full((1, 3, L), float("nan"), dtype=torch.float32, device="cuda")
        scale = d ** -0.5
        n.attention_fused(q.cuda(), k.cuda().transpose(2, 3), v.cuda(), out, acsr[2], acsr[3], acsr[4], scale,
                          n.PATH_BAND, lse=lse)
        n.check_status_word(0)
        s = at.sddmm_acsr(q, k.transpose(2, 3), meta, meta["trailing_dim"])
        ref = at.lse_acsr(s, meta, scale)
        got = lse.cpu()
        assert torch.isfinite(got).all(), f"pattern {(kind, L, p0, p1)}: non-finite lse"
        err = (got - ref).abs().max().item()
        assert err < 2e-2, f"pattern {(kind, L, p0, p1)} {dtype}: lse max abs err {err}"
        assert_close(out, at.attention_acsr(q, k.transpose(2, 3), v, meta, meta["trailing_dim"], scale), dtype,
                     f"output with lse, pattern {(kind, L, p0, p1)}")
