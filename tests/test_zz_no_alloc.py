"""GPU: splat_attention_noalloc, the entry point for callers that cannot allocate device memory
(host applications with a frozen memory pool, plug-ins that only receive input/output buffers,
callers that must not trigger cudaMalloc's device-wide synchronisation).  It runs the same three
kernels as splat_sddmm / splat_softmax / splat_spmm but keeps the (BH, L, trailing_dim) intermediate
in a fixed 64 MiB array inside the library.

Checked here, through the C ABI: its output equals the three existing entry points' output (same
kernels, so bit for bit) on two calls in a row of different shape -- the second call finds the
first call's leftovers in the shared array -- and a problem larger than the array is refused
without a launch.  This file sorts last on purpose so that a stop-at-first-failure run has already
executed every other test."""
import ctypes

import pytest
import torch

from oracle import acsr_oracle as ao

pytestmark = pytest.mark.gpu


def _three_entry_points(n, q, kt, v, acsr, scale):
    """Reference result from the existing entry points (splat_sddmm, splat_softmax, splat_spmm: the
    kernels the no-allocation variant chains) with caller-owned S and P buffers."""
    B, H, L, d = q.shape
    T = acsr[5]
    s = torch.empty((B, H, L, T), dtype=q.dtype, device=q.device)
    p = torch.empty_like(s)
    o = torch.empty_like(q)
    n.sddmm(q, kt, s, acsr[2], acsr[3], acsr[4], T, n.PATH_GENERIC)
    n.softmax(s, p, acsr[4], T, scale)
    n.spmm(p, v, o, acsr[2], acsr[3], acsr[4], T, n.PATH_GENERIC)
    return o


def _noalloc(n, q, kt, v, acsr, scale):
    B, H, L, d = q.shape
    o = torch.full_like(q, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    rc = n._lib.splat_attention_noalloc(
        q.data_ptr(), kt.data_ptr(), kt.stride(1), kt.stride(3), kt.stride(2), v.data_ptr(),
        o.data_ptr(), acsr[2].data_ptr(), acsr[3].data_ptr(), acsr[4].data_ptr(), B * H, L,
        kt.shape[3], d, acsr[5], ctypes.c_float(scale), n.dtype_code(q.dtype), stream)
    assert rc == 0, n.status_string(rc)
    return o


def test_noalloc_matches_existing_entry_points_twice_in_a_row():
    """Calls in a row of different shape and dtype: each finds the previous call's leftovers in the
    shared array.  The trailing dimensions are chosen so that the in-place softmax runs through
    each of its three kernels (201 and 17: the general loop; 256: short rows, two per warp; 512:
    rows held in registers).  Every result must equal the three existing entry points' bit for bit
    and agree with the CPU oracle within the library's tolerances."""
    import acsr_helpers as ah
    import splat_native as n
    from conftest import assert_close
    from oracle import attention_oracle as at
    torch.manual_seed(21)
    calls = [  # (pattern kind, L, p0, p1, dtype, B, H, d)
        (ao.PATTERN_CAUSAL_WINDOWED, 640, 200, 0, torch.bfloat16, 2, 3, 64),
        (ao.PATTERN_DILATED, 300, 17, 3, torch.float32, 1, 2, 32),
        (ao.PATTERN_CAUSAL_WINDOWED, 1024, 255, 0, torch.bfloat16, 1, 2, 64),
        (ao.PATTERN_CAUSAL_WINDOWED, 1024, 511, 0, torch.float16, 1, 2, 32),
    ]
    for kind, L, p0, p1, dtype, B, H, d in calls:
        acsr = ah.create_acsr(ah.PatternMask(kind, L, p0, p1), 16, 0)
        meta = ao.metadata_from_pattern(kind, L, p0, p1, 16)
        q, k, v = (torch.randn(B, H, L, d, device="cuda").to(dtype) for _ in range(3))
        kt = k.transpose(2, 3)
        scale = d ** -0.5
        expect = _three_entry_points(n, q, kt, v, acsr, scale)
        got = _noalloc(n, q, kt, v, acsr, scale)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, expect), f"max diff {(got.float() - expect.float()).abs().max().item()}"
        ref = at.attention_acsr(q.cpu(), kt.cpu(), v.cpu(), meta, meta["trailing_dim"], scale)
        assert_close(got, ref, dtype, f"no-alloc vs oracle, trailing_dim {acsr[5]}")


def test_noalloc_empty_problem_needs_no_buffers():
    """No (batch, head) pairs or no rows: nothing to do, null data pointers are fine."""
    import splat_native as n
    stream = torch.cuda.current_stream().cuda_stream
    for bh, rows in ((0, 128), (3, 0)):
        rc = n._lib.splat_attention_noalloc(None, None, 0, 64, 1, None, None, None, None, None, bh, rows,
                                            rows, 64, 16, ctypes.c_float(1.0),
                                            n.dtype_code(torch.bfloat16), stream)
        assert rc == 0, n.status_string(rc)
    torch.cuda.synchronize()


def test_noalloc_refuses_problems_beyond_its_fixed_buffer():
    import acsr_helpers as ah
    import splat_native as n
    L, d = 4096, 64
    acsr = ah.create_acsr(ah.create_causal_windowed_mask(L, 1023), 16, 0)   # trailing_dim 1024
    bh = n.NOALLOC_SCRATCH_BYTES // (L * 1024 * 2) + 1                     # one head too many
    dummy = torch.zeros(16, dtype=torch.bfloat16, device="cuda")           # never dereferenced
    rc = n._lib.splat_attention_noalloc(
        dummy.data_ptr(), dummy.data_ptr(), L * d, d, 1, dummy.data_ptr(), dummy.data_ptr(),
        acsr[2].data_ptr(), acsr[3].data_ptr(), acsr[4].data_ptr(), bh, L, L, d, acsr[5],
        ctypes.c_float(1.0), n.dtype_code(torch.bfloat16), torch.cuda.current_stream().cuda_stream)
    assert rc == -9 and "64 MiB" in n.status_string(rc)
    torch.cuda.synchronize()
