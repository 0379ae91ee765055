"""GPU: SDDMM, softmax, SpMM and the fused CUDA-core chain through the reference-shaped launchers,
against the CPU oracle and against the fixtures recorded from the reference kernels."""
import numpy as np
import pytest
import torch

from conftest import assert_close, golden_case
from oracle import acsr_oracle as ao
from oracle import attention_oracle as at

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _acsr_for(name, golden_meta):
    import acsr_helpers as ah
    ref = golden_case(golden_meta, name)
    kind, s, p0, p1, bh = ref["params"]
    acsr = ah.create_acsr(ao.make_mask(kind, s, p0, p1), bh, 0)
    return ref, acsr


def _run_sddmm(mask_like, acsr, q, kt, dtype):
    import r_sddmm
    B, H, L, _ = q.shape
    out, grid, tx, ty = r_sddmm.rsddmm_preamble(mask_like, (B, H, L, acsr[5]), 16, 16, 0, dtype)
    out.fill_(float("nan"))
    ret = r_sddmm.rsddmm_launcher(q, kt, out, acsr[0], acsr[1], acsr[2], acsr[3], acsr[5], acsr[4],
                                  grid, tx, ty, 16, 16)
    assert ret[0] is out and ret[1] is acsr[2] and ret[2] is acsr[3] and ret[3] is acsr[4]
    return out


def _run_softmax(mask_like, acsr, x, dtype, bsx=16, scale=None):
    import r_softmax
    B, H, L, T = x.shape
    grid, out, _shape, pow2 = r_softmax.rsoftmax_preamble(mask_like, (B, H, L, T), bsx, 0, dtype)
    out.fill_(float("nan"))
    kw = {} if scale is None else {"scale": scale}
    r_softmax.rsoftmax_launcher(x, out, acsr[0], acsr[1], acsr[2], acsr[3], T, pow2, acsr[4], grid,
                                bsx, **kw)
    return out


def _run_spmm(mask_like, acsr, p, v, dtype):
    import r_spmm
    B, H, L, d = v.shape
    out, grid, T = r_spmm.rspmm_preamble(mask_like, (B, H, L, d), 16, 16, 0, dtype)
    assert T == acsr[5]
    out.fill_(float("nan"))
    r_spmm.rspmm_launcher(p, v, out, acsr[0], acsr[1], acsr[2], acsr[3], acsr[6], acsr[7], T,
                          acsr[4], grid, 16, 16)
    return out


def test_reference_self_test_shapes(golden_meta, golden_reftests):
    """The reference's nine self-test shapes with the recorded inputs: SDDMM and SpMM on integer
    data are exact in fp32; softmax within fp32 rounding; padding slots are zero."""
    g = golden_reftests
    for name in (str(n) for n in g["names"]):
        n, p, T = (int(v) for v in g[f"{name}/params"])
        ref, acsr = _acsr_for(name, golden_meta)
        mask = ao.blocked_mask(n, p)
        _, _, nnz = ao.affine_ints(ref)
        valid = torch.from_numpy(np.arange(T)[None, :] < nnz[:, None])
        t = lambda key: torch.from_numpy(g[f"{name}/{key}"]).cuda()
        s = _run_sddmm(mask, acsr, t("sddmm_x"), t("sddmm_y"), torch.float32).cpu()
        assert torch.equal(s * valid, t("sddmm_out").cpu() * valid), name
        assert (s * ~valid == 0).all(), name
        sm = _run_softmax(mask, acsr, t("softmax_x"), torch.float32).cpu()
        assert ((sm - t("softmax_out").cpu()) * valid).abs().max() < 2e-5, name
        assert ((sm * valid).sum(-1) - 1).abs().max() < 1e-2, name     # the reference's own check
        o = _run_spmm(mask, acsr, t("spmm_x"), t("spmm_y"), torch.float32).cpu()
        assert torch.equal(o, t("spmm_out").cpu()), name


def test_config1_against_reference_kernels(golden_meta, golden_cfg1):
    c = golden_cfg1
    ref, acsr = _acsr_for("causal_256_31", golden_meta)
    mask = ao.causal_windowed_mask(256, 31)
    q, k, v = (torch.from_numpy(c[x]).cuda() for x in "qkv")
    kt = k.transpose(2, 3).contiguous()
    s = _run_sddmm(mask, acsr, q, kt, torch.float32)
    assert_close(s, torch.from_numpy(c["sddmm_out"]), torch.float32, "sddmm")
    p = _run_softmax(mask, acsr, s, torch.float32, bsx=16)   # all rows, whatever BLOCK_SIZE_X says
    assert_close(p, torch.from_numpy(c["softmax_out"]), torch.float32, "softmax")
    o = _run_spmm(mask, acsr, p, v, torch.float32)
    assert_close(o[:, :, :32], torch.from_numpy(c["spmm_out_rows_lt_d"]), torch.float32, "spmm")
    s16 = _run_sddmm(mask, acsr, q.half(), kt.half(), torch.float16)
    assert_close(s16, torch.from_numpy(c["sddmm_out_fp16"]).float(), torch.float16, "sddmm fp16")


CASES = ["blocked_128_57", "windowed_100_7", "causal_300_127", "strided_256_64", "strided_200_7",
         "dilated_256_8_2", "dilated_250_6_11", "causal_128_200", "windowed_33_0", "blocked_10_7"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kt_contiguous", [True, False])
def test_ops_against_oracle(golden_meta, dtype, kt_contiguous):
    torch.manual_seed(11)
    for name in CASES:
        ref, acsr = _acsr_for(name, golden_meta)
        kind, L, p0, p1, _bh = ref["params"]
        mask = ao.make_mask(kind, L, p0, p1)
        T = ref["trailing_dim"]
        for d in (32, 64, 24):
            B, H = 2, 2
            q, k, v = (torch.randn(B, H, L, d).to(dtype) for _ in range(3))
            kt = k.transpose(2, 3).contiguous() if kt_contiguous else k.transpose(2, 3)
            ktd = (k.cuda().transpose(2, 3).contiguous() if kt_contiguous else k.cuda().transpose(2, 3))
            s = _run_sddmm(mask, acsr, q.cuda(), ktd, dtype)
            s_ref = at.sddmm_acsr(q, kt, ref, T)
            assert_close(s, s_ref, dtype, f"{name} d={d} sddmm")
            scale = 1.0 / d ** 0.5
            p = _run_softmax(mask, acsr, s, dtype, scale=scale)
            p_ref = at.softmax_acsr(s.float().cpu(), ref, scale)
            assert_close(p, p_ref, dtype, f"{name} d={d} softmax")
            o = _run_spmm(mask, acsr, p, v.cuda(), dtype)
            o_ref = at.spmm_acsr(p.float().cpu(), v, ref)
            assert_close(o, o_ref, dtype, f"{name} d={d} spmm")


@pytest.mark.parametrize("dtype", DTYPES)
def test_fused_generic_against_oracle(golden_meta, dtype):
    import splat_native as n
    torch.manual_seed(12)
    for name in CASES:
        ref, acsr = _acsr_for(name, golden_meta)
        L, T = ref["params"][1], ref["trailing_dim"]
        for d, contig in ((32, False), (64, True), (128, False)):
            q, k, v = (torch.randn(1, 3, L, d).to(dtype) for _ in range(3))
            kt = k.transpose(2, 3)
            ktd = k.cuda().transpose(2, 3).contiguous() if contig else k.cuda().transpose(2, 3)
            out = torch.full((1, 3, L, d), float("nan"), dtype=dtype, device="cuda")
            scale = 1.0 / d ** 0.5
            n.attention_fused(q.cuda(), ktd, v.cuda(), out, acsr[2], acsr[3], acsr[4], scale,
                              n.PATH_GENERIC)
            o_ref = at.attention_acsr(q, kt, v, ref, T, scale)
            assert_close(out, o_ref, dtype, f"{name} d={d} fused generic")


def test_softmax_in_place_and_odd_trailing_dim():
    """Trailing dims that break 16-byte rows take the scalar kernel; in-place is allowed."""
    import acsr_helpers as ah
    torch.manual_seed(3)
    for L, p in ((50, 6), (40, 2)):
        mask = ao.causal_windowed_mask(L, p)
        acsr = ah.create_acsr(mask, 16, 0)
        meta = ao.metadata_from_mask(mask, 16)
        x = torch.randn(2, 2, L, acsr[5]) * 3
        for dtype in DTYPES:
            xd = x.to(dtype).cuda()
            ref = at.softmax_acsr(x.to(dtype), meta)
            import r_softmax
            r_softmax.rsoftmax_launcher(xd, xd, acsr[0], acsr[1], acsr[2], acsr[3], acsr[5], 8, acsr[4],
                                        (1, 1), 16)
            assert_close(xd, ref, dtype, f"in-place softmax L={L}")


def test_module_unfused_and_fused_agree_with_oracle(golden_meta):
    import acsr_helpers as ah
    import r_attention
    torch.manual_seed(4)
    ref = golden_case(golden_meta, "causal_256_31")
    B, H, L, d = 1, 2, 256, 32
    mask = ah.create_causal_windowed_mask(L, 31)
    q, k, v = (torch.randn(B, H, L, d) for _ in range(3))
    o_ref = at.attention_acsr(q, k.transpose(2, 3), v, ref, 32, 1.0)
    for fused in (False, True):
        attn = r_attention.RegularAttention(B, L, H, d, mask, 16, 16, 0, torch.float32, fused=fused)
        out = attn([q.cuda(), k.cuda().transpose(2, 3), v.cuda()])
        assert out is attn.rspmm_output                     # module-owned buffer, as in the reference
        assert_close(out, o_ref, torch.float32, f"module fused={fused}")
        assert attn([q.cuda(), k.cuda().transpose(2, 3), v.cuda()]) is out
    # unit(): projections then attention
    attn = r_attention.RegularAttention(B, L, H, d, mask, 16, 16, 0, torch.float32, scale=d ** -0.5)
    x = torch.randn(B, L, H * d) * 0.2
    w = [torch.randn(H * d, H, d) * 0.2 for _ in range(3)]
    out = r_attention.unit(x.cuda(), x.cuda(), x.cuda(), *[t.cuda() for t in w], attn)
    qp, kp, vp = (torch.einsum('bsd,dnh->bnsh', x, t) for t in w)
    assert_close(out, at.attention_acsr(qp, kp.transpose(2, 3), vp, ref, 32, d ** -0.5),
                 torch.float32, "unit")


def test_empty_batch_and_rows_without_nonzeros():
    """Edge inputs: a batch of zero heads launches nothing and returns; rows of the mask with no
    non-zero give zero output rows and rows with one non-zero copy the V row the metadata names
    (column 0: the reference describes single-element rows that way), on every path."""
    import acsr_helpers as ah
    import splat_native as n
    torch.manual_seed(11)
    L, d = 256, 64
    mask = ao.causal_windowed_mask(L, 40)
    mask[5:9, :] = 0            # empty rows
    mask[100, :] = 0
    mask[100, 37] = 1           # one non-zero, not at column 0
    mask[255, :] = 0            # last row empty
    meta = ao.metadata_from_mask(mask, 16)
    acsr = ah.create_acsr(mask.tolist(), 16, 0)
    for dtype in (torch.float32, torch.bfloat16):
        q, k, v = (torch.randn(1, 2, L, d).to(dtype) for _ in range(3))
        ref = at.attention_acsr(q, k.transpose(2, 3), v, meta, meta["trailing_dim"], d ** -0.5)
        assert torch.count_nonzero(ref[:, :, 5:9]) == 0 and torch.count_nonzero(ref[:, :, 255]) == 0
        assert torch.equal(ref[:, :, 100], v[:, :, 0].float())
        for path in (n.PATH_GENERIC, n.PATH_AUTO):
            out = torch.full((1, 2, L, d), float("nan"), dtype=dtype, device="cuda")
            n.attention_fused(q.cuda(), k.cuda().transpose(2, 3), v.cuda(), out, acsr[2], acsr[3],
                              acsr[4], d ** -0.5, path)
            n.check_status_word(0)
            assert_close(out, ref, dtype, f"empty rows path={path} {dtype}")
    # zero heads: every entry point returns without a launch
    q0 = torch.empty(0, 2, L, d, device="cuda")
    out0 = torch.empty(0, 2, L, d, device="cuda")
    n.attention_fused(q0, q0.transpose(2, 3), q0, out0, acsr[2], acsr[3], acsr[4], 1.0, n.PATH_AUTO)
    s0 = torch.empty(0, 2, L, meta["trailing_dim"], device="cuda")
    T = meta["trailing_dim"]
    n.sddmm(q0, q0.transpose(2, 3), s0, acsr[2], acsr[3], acsr[4], T)
    n.softmax(s0, s0, acsr[4], T)
    n.spmm(s0, q0, out0, acsr[2], acsr[3], acsr[4], T)
    torch.cuda.synchronize()


def test_checked_index_mode_clamps_and_reports():
    """Checked-index mode of the CUDA-core kernels.  The metadata below names columns up to 110 while
    n_cols = 64 is passed in; K and V are allocated with 128 columns, so every address the kernels
    can form, clamped or not, lies inside the allocation.  With the mode on, columns >= n_cols must
    be read as column n_cols - 1 and the kernel's code must be left in the registered word; with it
    off the columns are used as they are and the word stays 0."""
    import ctypes
    import splat_native as n
    dev = torch.device("cuda", 0)
    rows, n_cols, n_alloc, d, T = 64, 64, 128, 32, 48
    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, 1, rows, d, generator=g).to(dev)
    k = torch.randn(1, 1, n_alloc, d, generator=g).to(dev)
    v = torch.randn(1, 1, n_alloc, d, generator=g).to(dev)
    p_in = torch.rand(1, 1, rows, T, generator=g).to(dev)
    lin = torch.ones(rows, device=dev)
    tr = torch.arange(rows, dtype=torch.float32, device=dev)          # start_i = i, stride 1
    nnzs = torch.full((rows,), float(T), device=dev)
    cols = torch.arange(rows, device=dev)[:, None] + torch.arange(T, device=dev)[None, :]   # up to 110
    word = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    f32 = n.dtype_code(torch.float32)
    scale = d ** -0.5

    def reference(c):
        s = torch.einsum("rd,rtd->rt", q[0, 0], k[0, 0][c])
        o_spmm = torch.einsum("rt,rtd->rd", p_in[0, 0], v[0, 0][c])
        o_fused = torch.einsum("rt,rtd->rd", torch.softmax(s * scale, dim=-1), v[0, 0][c])
        return s, o_spmm, o_fused

    def run():
        s_out = torch.empty(1, 1, rows, T, device=dev)
        o1 = torch.empty(1, 1, rows, d, device=dev)
        o2 = torch.empty(1, 1, rows, d, device=dev)
        results = []
        for call in ("sddmm", "spmm", "fused"):
            word.zero_()
            if call == "sddmm":
                rc = n._lib.splat_sddmm(q.data_ptr(), k.data_ptr(), n_alloc * d, d, 1, s_out.data_ptr(),
                                        lin.data_ptr(), tr.data_ptr(), nnzs.data_ptr(), 1, rows, n_cols, d, T,
                                        f32, st)
            elif call == "spmm":
                rc = n._lib.splat_spmm(p_in.data_ptr(), v.data_ptr(), o1.data_ptr(), lin.data_ptr(),
                                       tr.data_ptr(), nnzs.data_ptr(), 1, rows, n_cols, d, T, f32, st)
            else:
                rc = n._lib.splat_attention_fused(q.data_ptr(), k.data_ptr(), n_alloc * d, d, 1, v.data_ptr(),
                                                  o2.data_ptr(), lin.data_ptr(), tr.data_ptr(), nnzs.data_ptr(),
                                                  1, rows, n_cols, d, ctypes.c_float(scale), f32,
                                                  n.PATH_GENERIC, None, word.data_ptr(), st)
            assert rc == 0, (call, rc)
            torch.cuda.synchronize()
            results.append(int(word.item()))
        return s_out[0, 0], o1[0, 0], o2[0, 0], results

    try:
        assert n._lib.splat_debug_check_indices(word.data_ptr()) == 0
        s_c, o1_c, o2_c, codes = run()
    finally:
        assert n._lib.splat_debug_check_indices(None) == 0
    assert codes == [71, 72, 73], codes
    ref = reference(cols.clamp(max=n_cols - 1))
    for got, want, name in zip((s_c, o1_c, o2_c), ref, ("sddmm", "spmm", "fused")):
        assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), f"checked {name}: {(got - want).abs().max().item()}"
    s_u, o1_u, o2_u, codes = run()
    assert codes == [0, 0, 0], codes
    ref = reference(cols)
    for got, want, name in zip((s_u, o1_u, o2_u), ref, ("sddmm", "spmm", "fused")):
        assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), f"unchecked {name}: {(got - want).abs().max().item()}"
    assert (s_c - s_u).abs().max().item() > 1e-3   # the clamp changed what was read


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_fused_generic_log_sum_exp(golden_meta, dtype):
    """lse output of the CUDA-core fused kernel, including rows without non-zeros (-inf)."""
    import acsr_helpers as ah
    import r_attention
    import splat_native as n
    L, d = 192, 64
    mask = ah.create_windowed_mask(L, 20)
    attn = r_attention.RegularAttention(2, L, 2, d, mask, 16, 16, 0, dtype, scale=0.2, path=n.PATH_GENERIC, lse=True)
    # empty rows: zero their nnz
    attn.nnzs[5] = 0
    attn.nnzs[100] = 0
    torch.manual_seed(21)
    q, k, v = (torch.randn(2, 2, L, d).to(dtype) for _ in range(3))
    out = attn([q.cuda(), k.cuda().transpose(2, 3), v.cuda()])
    torch.cuda.synchronize()
    meta = ao.metadata_from_pattern(ao.PATTERN_WINDOWED, L, 20, 0, 16)
    meta = dict(meta)
    nn = np.array(meta["nnzs"], dtype=np.float32).copy(); nn[5] = 0; nn[100] = 0
    meta["nnzs"] = nn
    s = at.sddmm_acsr(q, k.transpose(2, 3), meta, meta["trailing_dim"])
    ref = at.lse_acsr(s, meta, 0.2)
    got = attn.lse.cpu()
    assert torch.isinf(got[:, :, 5]).all() and (got[:, :, 5] < 0).all()
    assert torch.isinf(got[:, :, 100]).all()
    keep = torch.isfinite(ref)
    tol = 1e-4 if dtype == torch.float32 else 5e-3
    assert (got[keep] - ref[keep]).abs().max().item() < tol
    assert_close(out, at.attention_acsr(q, k.transpose(2, 3), v, meta, meta["trailing_dim"], 0.2), dtype, "generic with lse")
