"""CPU: the oracle restatement against fixtures produced by the reference itself (tests/golden)."""
import numpy as np
import pytest
import torch

from conftest import META_KEYS, bits_equal, golden_case
from oracle import acsr_oracle as ao
from oracle import attention_oracle as at


def _names(g):
    return [str(n) for n in g["names"]]


def test_metadata_three_restatements_bit_exact(golden_meta):
    """closed form from the mask, closed form from the pattern, and the literal row loop through
    numpy.linalg.solve all reproduce create_acsr bit for bit."""
    for name in _names(golden_meta):
        ref = golden_case(golden_meta, name)
        kind, s, p0, p1, bh = ref["params"]
        mask = ao.make_mask(kind, s, p0, p1)
        for label, meta in (("mask", ao.metadata_from_mask(mask, bh)),
                            ("pattern", ao.metadata_from_pattern(kind, s, p0, p1, bh)),
                            ("literal", ao.metadata_literal(mask, bh))):
            for k in META_KEYS:
                assert bits_equal(meta[k], ref[k]), f"{name}/{label}/{k}"
            assert meta["trailing_dim"] == ref["trailing_dim"], f"{name}/{label}"


def test_tile_map_matches_reference(golden_meta):
    for name in _names(golden_meta):
        kind, s, p0, p1, bh = golden_case(golden_meta, name)["params"]
        tx, ty = ao.tile_map_from_mask(ao.make_mask(kind, s, p0, p1), bh, 16)
        assert np.array_equal(tx, golden_meta[f"{name}/tb_x"]), name
        assert np.array_equal(ty, golden_meta[f"{name}/tb_y"]), name


def test_config_patterns_bit_exact(golden_meta_configs):
    """The four large benchmark patterns (L = 4096 ... 32768): closed form vs the reference."""
    for name in _names(golden_meta_configs):
        ref = golden_case(golden_meta_configs, name)
        kind, s, p0, p1, bh = ref["params"]
        meta = ao.metadata_from_pattern(kind, s, p0, p1, bh)
        for k in META_KEYS:
            assert bits_equal(meta[k], ref[k]), f"{name}/{k}"
        assert meta["trailing_dim"] == ref["trailing_dim"]


def test_single_nonzero_rows_are_described_as_column_zero(golden_meta):
    """A row with exactly one non-zero at column a != 0 gets (stride 1, start 0) from the reference
    (SPLAT/acsr_helpers.py:126-130); the oracle's effective mask must follow the metadata."""
    ref = golden_case(golden_meta, "strided_256_64")
    start, stride, nnz = ao.affine_ints(ref)
    assert nnz[3] == 1 and start[3] == 0 and stride[3] == 1
    eff = ao.effective_mask(ref, 256)
    assert eff[3, 0] == 1 and eff[3, 3] == 0
    dense = ao.strided_mask(256, 64)
    multi = nnz > 1
    assert np.array_equal(eff[multi], dense[multi])


def test_pattern_rows_match_dense_masks():
    for kind, s, p0, p1 in [(0, 37, 5, 0), (0, 64, 64, 0), (1, 50, 7, 0), (1, 20, 40, 0),
                            (2, 70, 9, 0), (2, 33, 0, 0), (3, 90, 8, 0), (3, 40, 1, 0),
                            (4, 77, 5, 3), (4, 64, 100, 2)]:
        a = ao.row_summary(ao.make_mask(kind, s, p0, p1))
        b = ao.pattern_rows(kind, s, p0, p1)
        for x, y in zip(a, b):
            assert np.array_equal(x, y), (kind, s, p0, p1)


def test_kernels_on_reference_self_test_shapes(golden_meta, golden_reftests):
    """The reference's own nine self-test shapes (blocked masks, integer inputs): SDDMM and SpMM
    exactly, softmax to fp32 rounding."""
    g = golden_reftests
    for name in _names(g):
        n, p, T = (int(v) for v in g[f"{name}/params"])
        meta = golden_case(golden_meta, name)
        _, _, nnz = ao.affine_ints(meta)
        valid = torch.from_numpy(np.arange(T)[None, :] < nnz[:, None])
        t = lambda key: torch.from_numpy(g[f"{name}/{key}"])
        s = at.sddmm_acsr(t("sddmm_x"), t("sddmm_y"), meta, T)
        assert torch.equal(s * valid, t("sddmm_out") * valid), name
        sm = at.softmax_acsr(t("softmax_x"), meta)
        assert ((sm - t("softmax_out")) * valid).abs().max() < 1e-6, name
        # the reference's own property: every row with non-zeros sums to one (1e-2)
        rows = (sm * valid).sum(-1)
        assert ((rows - 1).abs() < 1e-2)[..., nnz > 0].all(), name
        o = at.spmm_acsr(t("spmm_x"), t("spmm_y"), meta)
        assert torch.equal(o, t("spmm_out")), name


def test_kernels_on_config1(golden_meta, golden_cfg1):
    c = golden_cfg1
    meta = golden_case(golden_meta, "causal_256_31")
    T = int(c["trailing_dim"])
    q, k, v = (torch.from_numpy(c[x]) for x in "qkv")
    kt = k.transpose(2, 3).contiguous()
    s = at.sddmm_acsr(q, kt, meta, T)
    assert (s - torch.from_numpy(c["sddmm_out"])).abs().max() < 1e-4
    p = at.softmax_acsr(s, meta)
    assert (p - torch.from_numpy(c["softmax_out"])).abs().max() < 1e-5
    o = at.spmm_acsr(p, v, meta)
    assert (o[:, :, :32] - torch.from_numpy(c["spmm_out_rows_lt_d"])).abs().max() < 1e-4
    # independent dense-masked evaluation of the same chain
    od = at.attention_dense_masked(q, kt, v, ao.effective_mask(meta, 256))
    assert (o - od).abs().max() < 1e-4
    s16 = at.sddmm_acsr(q.half(), kt.half(), meta, T)
    assert (s16 - torch.from_numpy(c["sddmm_out_fp16"]).float()).abs().max() < 2e-2


def test_dense_and_acsr_oracles_agree_on_strided_and_dilated(golden_meta):
    torch.manual_seed(5)
    for name in ("strided_96_3", "dilated_128_16_3", "strided_256_64", "windowed_100_7"):
        meta = golden_case(golden_meta, name)
        L = meta["params"][1]
        q, k, v = (torch.randn(1, 2, L, 16) for _ in range(3))
        kt = k.transpose(2, 3)
        a = at.attention_acsr(q, kt, v, meta, meta["trailing_dim"], scale=0.25)
        b = at.attention_dense_masked(q, kt, v, ao.effective_mask(meta, L), scale=0.25)
        assert (a - b).abs().max() < 1e-5, name
