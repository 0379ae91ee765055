"""Shared test plumbing: paths, the ``gpu`` marker, golden-fixture loaders and tolerances."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SPLAT_DIR = os.path.join(ROOT, "triton-fun_b200", "SPLAT")
GOLDEN = os.path.join(ROOT, "tests", "golden")
for p in (ROOT, SPLAT_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


META_KEYS = ("dTos_lin", "dTos_tr", "sTod_lin", "sTod_tr", "nnzs", "span_start", "span_end")


@pytest.fixture(scope="session")
def golden_meta():
    return np.load(os.path.join(GOLDEN, "acsr_metadata.npz"))


@pytest.fixture(scope="session")
def golden_meta_configs():
    return np.load(os.path.join(GOLDEN, "acsr_metadata_configs.npz"))


@pytest.fixture(scope="session")
def golden_reftests():
    return np.load(os.path.join(GOLDEN, "kernels_reftests.npz"))


@pytest.fixture(scope="session")
def golden_cfg1():
    return np.load(os.path.join(GOLDEN, "kernels_cfg1.npz"))


def golden_case(g, name):
    return {k: g[f"{name}/{k}"] for k in META_KEYS} | {"trailing_dim": int(g[f"{name}/trailing_dim"]),
                                                       "params": [int(v) for v in g[f"{name}/params"]]}


def bits_equal(a, b) -> bool:
    a = np.ascontiguousarray(np.asarray(a, dtype=np.float32))
    b = np.ascontiguousarray(np.asarray(b, dtype=np.float32))
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


# Tolerances of the parity contract: fp32 within 1e-4; fp16/bf16 within max-abs 2e-2 + max-rel 1e-2.
TOL = {torch.float32: dict(atol=1e-4, rtol=1e-4),
       torch.float16: dict(atol=2e-2, rtol=1e-2),
       torch.bfloat16: dict(atol=2e-2, rtol=1e-2)}


def assert_close(actual: torch.Tensor, expected: torch.Tensor, dtype, what=""):
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(e.shape)}"
    assert torch.isfinite(a).all(), f"{what}: non-finite values in the result"
    tol = TOL[dtype]
    err = (a - e).abs()
    bound = tol["atol"] + tol["rtol"] * e.abs()
    bad = err > bound
    if bad.any():
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.numel()} elements out of tolerance; "
                             f"max abs err {err.max().item():.4g}; first at {idx}: "
                             f"{a[tuple(idx)].item():.6g} vs {e[tuple(idx)].item():.6g}")
