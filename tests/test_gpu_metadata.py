"""GPU: ACSR metadata and tile maps built by the CUDA kernels, bit-exact against the fixtures made
by the reference's create_acsr / naive_block_mappings, for every way of handing in a mask."""
import numpy as np
import pytest
import torch

from conftest import META_KEYS, bits_equal, golden_case
from oracle import acsr_oracle as ao

pytestmark = pytest.mark.gpu


def _check(out, ref, what):
    for i, k in enumerate(("dTos_lin", "dTos_tr", "sTod_lin", "sTod_tr", "nnzs")):
        assert out[i].dtype == torch.float32 and out[i].is_cuda
        assert bits_equal(out[i].cpu().numpy(), ref[k]), f"{what}/{k}"
    assert isinstance(out[5], int) and out[5] == ref["trailing_dim"], what
    assert bits_equal(out[6].cpu().numpy(), ref["span_start"]), f"{what}/span_start"
    assert bits_equal(out[7].cpu().numpy(), ref["span_end"]), f"{what}/span_end"


def _pattern(ah, kind, s, p0, p1):
    return [ah.create_blocked_mask, ah.create_windowed_mask, ah.create_causal_windowed_mask,
            ah.create_strided_mask, lambda s_, p_: ah.create_dilated_mask(s_, p_, p1)][kind](s, p0)


def test_create_acsr_bit_exact_all_mask_forms(golden_meta):
    import acsr_helpers as ah
    for name in (str(n) for n in golden_meta["names"]):
        ref = golden_case(golden_meta, name)
        kind, s, p0, p1, bh = ref["params"]
        dense = ao.make_mask(kind, s, p0, p1)
        forms = {"pattern": _pattern(ah, kind, s, p0, p1), "list": dense.astype(int).tolist(),
                 "numpy": dense, "bool_tensor": torch.from_numpy(dense != 0),
                 "cuda_tensor": torch.from_numpy(dense).cuda()}
        for label, m in forms.items():
            _check(ah.create_acsr(m, bh, 0), ref, f"{name}/{label}")


def test_create_acsr_unaligned_mask_rows():
    """Row stride not a multiple of 16 bytes and an offset base pointer take the scalar scan."""
    import acsr_helpers as ah
    dense = ao.causal_windowed_mask(77, 9)
    big = torch.zeros(80, 99, dtype=torch.uint8, device="cuda")
    view = big[1:78, 3:80]
    view.copy_(torch.from_numpy(dense))
    ref = ao.metadata_from_mask(dense, 16)
    out = ah.create_acsr(view, 16, 0)
    for i, k in enumerate(("dTos_lin", "dTos_tr", "sTod_lin", "sTod_tr", "nnzs")):
        assert bits_equal(out[i].cpu().numpy(), ref[k]), k


def test_config_patterns_bit_exact(golden_meta_configs):
    """The four large benchmark patterns, from the closed form and (L <= 8192) from a full mask
    scanned on the device."""
    import acsr_helpers as ah
    for name in (str(n) for n in golden_meta_configs["names"]):
        ref = golden_case(golden_meta_configs, name)
        kind, s, p0, p1, bh = ref["params"]
        pm = _pattern(ah, kind, s, p0, p1)
        _check(ah.create_acsr(pm, bh, 0), ref, f"{name}/pattern")
        if s <= 16384:
            _check(ah.create_acsr(pm.to_tensor(0), bh, 0), ref, f"{name}/device-mask")


def test_pattern_mask_kernel_matches_oracle_masks():
    import acsr_helpers as ah
    for kind, s, p0, p1 in [(0, 37, 5, 0), (1, 50, 7, 0), (2, 70, 9, 0), (3, 90, 8, 0), (4, 77, 5, 3),
                            (2, 256, 31, 0), (0, 16, 16, 0)]:
        got = _pattern(ah, kind, s, p0, p1).to_tensor(0).cpu().numpy()
        assert np.array_equal(got, ao.make_mask(kind, s, p0, p1)), (kind, s, p0, p1)


def test_tile_map_matches_reference(golden_meta):
    import acsr_helpers as ah
    import r_sddmm
    for name in (str(n) for n in golden_meta["names"]):
        kind, s, p0, p1, bh = golden_case(golden_meta, name)["params"]
        tx, ty = r_sddmm.naive_block_mappings(_pattern(ah, kind, s, p0, p1), bh, 16, 0)
        assert tx.dtype == torch.int32 and ty.dtype == torch.int32
        assert np.array_equal(tx.cpu().numpy(), golden_meta[f"{name}/tb_x"]), name
        assert np.array_equal(ty.cpu().numpy(), golden_meta[f"{name}/tb_y"]), name


def test_instantiate_metadata_container(golden_meta):
    import acsr_helpers as ah
    ref = golden_case(golden_meta, "blocked_32_10")
    acsr = ah.instantiate_metadata(ah.create_blocked_mask(32, 10), 16)
    assert np.array_equal(np.asarray(acsr.get_sTod_linear_transformations(), dtype=np.float32), ref["sTod_lin"])
    assert np.array_equal(np.asarray(acsr.get_dTos_translations(), dtype=np.float32), ref["dTos_tr"])
    assert np.array_equal(np.asarray(acsr.get_nnzs(), dtype=np.float32), ref["nnzs"])
    spans = acsr.get_span_specialised_data()
    assert [s[0] for s in spans] == ref["span_start"].tolist()
    assert [s[1] for s in spans] == ref["span_end"].tolist()


def test_classify_plan():
    import acsr_helpers as ah
    import splat_native as n
    for pm, stride, single in [(ah.create_causal_windowed_mask(256, 31), 1, 1),
                               (ah.create_strided_mask(256, 64), 64, 64),
                               (ah.create_dilated_mask(256, 8, 2), 2, 2),
                               (ah.create_windowed_mask(100, 7), 1, 0)]:
        a = ah.create_acsr(pm, 16, 0)
        plan = n.classify(a[2], a[3], a[4])
        assert plan[0] == a[5]
        assert plan[1] == plan[2] == stride and plan[3] == 0
        assert plan[4] == single and plan[5] == len(pm) and plan[6] == 0
