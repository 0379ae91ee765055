"""CPU: the C-ABI library loads and exports what include/splat_b200.h declares; host-side logic
(mask objects, sharding incl. a 2-rank gloo run, argument checking).  No kernel is launched."""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, SPLAT_DIR
from oracle import acsr_oracle as ao


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "splat_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(splat_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import splat_native as n
    lib = ctypes.CDLL(n.LIB_PATH)
    syms = _declared_symbols()
    assert len(syms) >= 12
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/splat_b200.h but not exported"
    # and the binding table covers the header
    assert set(syms) == set(n.SIGNATURES) | {"splat_status_string"}


def test_version_and_status_strings():
    import splat_native as n
    assert n.version() == 100
    assert n.status_string(0) == "ok"
    for code in range(-9, 0):
        assert n.status_string(code) not in ("ok", "unknown status")
    assert n.status_string(-99) == "unknown status"


def test_host_side_argument_errors_launch_nothing():
    """Bad arguments are rejected before any CUDA call (negative status, no launch)."""
    import splat_native as n
    lib = n._lib
    assert lib.splat_softmax(None, None, None, 1, 1, 1, 1.0, 0, None) == -1
    assert lib.splat_sddmm(None, None, 0, 0, 0, None, None, None, None, 1, 1, 1, 1, 1, 0, None) == -1
    assert lib.splat_pattern_row_summary(99, 10, 1, 0, ctypes.c_void_p(16), None) == -1
    assert lib.splat_pattern_row_summary(0, 10, 0, 0, ctypes.c_void_p(16), None) == -1


def test_cpu_device_is_rejected():
    import acsr_helpers as ah
    with pytest.raises(ValueError):
        ah.create_acsr(ah.create_blocked_mask(10, 2), 16, "cpu")


def test_pattern_mask_behaves_like_list_of_lists():
    import acsr_helpers as ah
    cases = [(ah.create_blocked_mask(37, 5), ao.blocked_mask(37, 5)),
             (ah.create_windowed_mask(50, 7), ao.windowed_mask(50, 7)),
             (ah.create_causal_windowed_mask(70, 9), ao.causal_windowed_mask(70, 9)),
             (ah.create_strided_mask(90, 8), ao.strided_mask(90, 8)),
             (ah.create_dilated_mask(77, 5, 3), ao.dilated_mask(77, 5, 3))]
    for pm, dense in cases:
        assert len(pm) == dense.shape[0] and len(pm[0]) == dense.shape[1]
        assert np.array_equal(np.asarray(pm.tolist()), dense)
        assert pm[3][2] == dense[3, 2] and pm[-1] == dense[-1].tolist()
        assert sum(1 for _ in pm) == dense.shape[0]
    with pytest.raises(IndexError):
        cases[0][0][37]
    with pytest.raises(ValueError):
        ah.create_blocked_mask(10, 0)


def test_shard_range_partitions():
    from sharding import shard_range
    for total in (0, 1, 2, 7, 64, 512):
        for world in (1, 2, 3, 4, 8):
            pieces = [shard_range(total, world, r) for r in range(world)]
            assert pieces[0][0] == 0 and pieces[-1][1] == total
            for (a0, a1), (b0, b1) in zip(pieces, pieces[1:]):
                assert a1 == b0 and a0 <= a1
            sizes = [b - a for a, b in pieces]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


_GLOO_WORKER = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
from sharding import shard_range
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
total = 13
b, e = shard_range(total, world, rank)
# every rank "processes" its heads: a deterministic per-head value, no data-path collective
local = torch.zeros(total)
local[b:e] = torch.arange(b, e, dtype=torch.float32) * 2 + 1
# test-only reduction to check the partition is exact and disjoint
dist.all_reduce(local)
assert torch.equal(local, torch.arange(total, dtype=torch.float32) * 2 + 1), local
t = torch.tensor([float(rank + 1)])
dist.all_reduce(t, op=dist.ReduceOp.MAX)   # the max-over-ranks timing reduction of the benchmark
assert t.item() == world
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
"""


def test_two_rank_gloo_sharding(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(script), SPLAT_DIR]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.count("ok") == 2
