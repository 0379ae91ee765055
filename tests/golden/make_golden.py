"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE ITSELF.

Usage (only where the reference checkout is available; it is not needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/reference [--configs]

The reference's Python modules are imported unmodified from ``<reference>/SPLAT`` and its Triton
kernels execute under the Triton interpreter (``TRITON_INTERPRET=1``, device ``'cpu'``).  Each
kernel is only recorded on the sub-domain where it computes what its own checker expects:

  * ``create_acsr`` / ``naive_block_mappings`` ...... everywhere (pure Python)
  * ``rsddmm_launcher`` ............................. rows whose affine stride is 1
  * ``rsoftmax_launcher`` ........................... with a BLOCK_SIZE_X=1 preamble, because the
                                                     launch grid is cdiv(L, BLOCK_SIZE_X) programs
                                                     of a one-row-per-program kernel
  * ``rspmm_launcher`` .............................. square problems (L == head_dim <= 128), the
                                                     shape its own tests use

Outputs (np.savez_compressed):
  acsr_metadata.npz          metadata + tile maps of 30-odd small masks
  acsr_metadata_configs.npz  metadata of the four large benchmark patterns (``--configs``; the
                             reference needs minutes for these, rows are fed lazily)
  kernels_reftests.npz       the reference's nine self-test shapes, integer-valued inputs
  kernels_cfg1.npz           B=1 H=2 L=256 d=32 fp32 causal window 32, N(0,1) inputs, seed 0
"""
import argparse
import os
import sys
import time

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import acsr_oracle as ao  # noqa: E402  (mask generators for the two added patterns)

META_KEYS = ("dTos_lin", "dTos_tr", "sTod_lin", "sTod_tr", "nnzs", "span_start", "span_end")


def ref_mask(ah, kind, s, p0, p1):
    """Reference generator where it has one, else the oracle's mask as list[list[int]]."""
    if kind == ao.PATTERN_BLOCKED:
        return ah.create_blocked_mask(s, p0)
    if kind == ao.PATTERN_WINDOWED:
        return ah.create_windowed_mask(s, p0)
    if kind == ao.PATTERN_CAUSAL_WINDOWED:
        return ah.create_causal_windowed_mask(s, p0)
    return ao.make_mask(kind, s, p0, p1).astype(int).tolist()


def acsr_to_dict(out):
    d = {k: out[i].numpy() for i, k in enumerate(("dTos_lin", "dTos_tr", "sTod_lin", "sTod_tr", "nnzs"))}
    d["trailing_dim"] = np.int64(out[5])
    d["span_start"] = out[6].numpy()
    d["span_end"] = out[7].numpy()
    return d


SMALL_CASES = [
    # (name, kind, s, p0, p1, block_height)
    *[(f"blocked_{n}_{p}", ao.PATTERN_BLOCKED, n, p, 0, 16)
      for n, p in [(10, 2), (10, 5), (10, 7), (16, 5), (16, 16), (32, 10), (32, 20), (32, 32),
                   (128, 57), (128, 16), (100, 7)]],
    ("blocked_64_16_bh8", ao.PATTERN_BLOCKED, 64, 16, 0, 8),
    ("blocked_10_2_bh2", ao.PATTERN_BLOCKED, 10, 2, 0, 2),
    ("windowed_100_7", ao.PATTERN_WINDOWED, 100, 7, 0, 16),
    ("windowed_64_3", ao.PATTERN_WINDOWED, 64, 3, 0, 16),
    ("windowed_256_40", ao.PATTERN_WINDOWED, 256, 40, 0, 16),
    ("windowed_33_0", ao.PATTERN_WINDOWED, 33, 0, 0, 16),
    ("causal_256_31", ao.PATTERN_CAUSAL_WINDOWED, 256, 31, 0, 16),
    ("causal_64_7", ao.PATTERN_CAUSAL_WINDOWED, 64, 7, 0, 16),
    ("causal_100_9", ao.PATTERN_CAUSAL_WINDOWED, 100, 9, 0, 16),
    ("causal_300_127", ao.PATTERN_CAUSAL_WINDOWED, 300, 127, 0, 16),
    ("causal_128_200", ao.PATTERN_CAUSAL_WINDOWED, 128, 200, 0, 32),
    ("strided_256_64", ao.PATTERN_STRIDED, 256, 64, 0, 16),
    ("strided_96_3", ao.PATTERN_STRIDED, 96, 3, 0, 16),
    ("strided_200_7", ao.PATTERN_STRIDED, 200, 7, 0, 16),
    ("strided_512_5", ao.PATTERN_STRIDED, 512, 5, 0, 16),
    ("dilated_256_8_2", ao.PATTERN_DILATED, 256, 8, 2, 16),
    ("dilated_128_16_3", ao.PATTERN_DILATED, 128, 16, 3, 16),
    ("dilated_250_6_11", ao.PATTERN_DILATED, 250, 6, 11, 16),
]


def gen_metadata(ah, r_sddmm, out_path):
    store = {}
    names = []
    for name, kind, s, p0, p1, bh in SMALL_CASES:
        mask = ref_mask(ah, kind, s, p0, p1)
        d = acsr_to_dict(ah.create_acsr(mask, bh, "cpu"))
        tx, ty = r_sddmm.naive_block_mappings(mask, bh, 16, "cpu")
        d["tb_x"], d["tb_y"] = tx.numpy(), ty.numpy()
        d["params"] = np.asarray([kind, s, p0, p1, bh], dtype=np.int64)
        for k, v in d.items():
            store[f"{name}/{k}"] = v
        names.append(name)
    store["names"] = np.asarray(names)
    np.savez_compressed(out_path, **store)
    print("wrote", out_path, len(names), "cases")


class LazyMask:
    """Feeds the reference one row at a time (it only uses len(mask), len(mask[0]), mask[row]
    and iteration), so that L=32768 does not need an L x L list of Python ints."""

    def __init__(self, kind, s, p0, p1):
        self.first, self.second, self.last, self.count = ao.pattern_rows(kind, s, p0, p1)
        self.s = s

    def __len__(self):
        return self.s

    def __getitem__(self, r):
        if r < 0 or r >= self.s:
            raise IndexError(r)
        row = [0] * self.s
        n = int(self.count[r])
        if n == 1:
            row[int(self.first[r])] = 1
        elif n > 1:
            a, b = int(self.first[r]), int(self.second[r])
            row[a:a + (n - 1) * (b - a) + 1:b - a] = [1] * n
        return row


CONFIG_CASES = [
    ("cfg2_causal_4096_255", ao.PATTERN_CAUSAL_WINDOWED, 4096, 255, 0, 16),
    ("cfg3_strided_8192_64", ao.PATTERN_STRIDED, 8192, 64, 0, 16),
    ("cfg4_dilated_16384_512_2", ao.PATTERN_DILATED, 16384, 512, 2, 16),
    ("cfg5_causal_32768_1023", ao.PATTERN_CAUSAL_WINDOWED, 32768, 1023, 0, 16),
]


def gen_config_metadata(ah, out_path):
    store = {}
    names = []
    for name, kind, s, p0, p1, bh in CONFIG_CASES:
        t = time.time()
        lazy = LazyMask(kind, s, p0, p1)
        # the lazy rows are checked against the dense generator on a small instance elsewhere
        d = acsr_to_dict(ah.create_acsr(lazy, bh, "cpu"))
        d["params"] = np.asarray([kind, s, p0, p1, bh], dtype=np.int64)
        for k, v in d.items():
            store[f"{name}/{k}"] = v
        names.append(name)
        print(name, "done in", round(time.time() - t, 1), "s", flush=True)
    store["names"] = np.asarray(names)
    np.savez_compressed(out_path, **store)
    print("wrote", out_path)


def run_sddmm(r_sddmm, mask, acsr, q, kt, dtype):
    B, H, L, _ = q.shape
    out, grid, tx, ty = r_sddmm.rsddmm_preamble(mask, (B, H, L, acsr[5]), 16, 16, "cpu", dtype)
    out.zero_()
    r_sddmm.rsddmm_launcher(q, kt, out, acsr[0], acsr[1], acsr[2], acsr[3], acsr[5], acsr[4],
                            grid, tx, ty, 16, 16)
    return out


def run_softmax(r_softmax, mask, acsr, x, dtype):
    B, H, L, T = x.shape
    grid, out, _shape, pow2 = r_softmax.rsoftmax_preamble(mask, (B, H, L, T), 1, "cpu", dtype)
    out.zero_()
    r_softmax.rsoftmax_launcher(x, out, acsr[0], acsr[1], acsr[2], acsr[3], T, pow2, acsr[4], grid, 1)
    return out


def run_spmm(r_spmm, mask, acsr, p, v, dtype):
    B, H, L, d = v.shape
    out, grid, T = r_spmm.rspmm_preamble(mask, (B, H, L, d), 16, 16, "cpu", dtype)
    out.zero_()
    r_spmm.rspmm_launcher(p, v, out, acsr[0], acsr[1], acsr[2], acsr[3], acsr[6], acsr[7], T,
                          acsr[4], grid, 16, 16)
    return out


def gen_reftests(ah, r_sddmm, r_softmax, r_spmm, out_path):
    """The reference's self-test shapes (SPLAT/r_sddmm.py:258-413 and the twin lists in
    r_softmax.py / r_spmm.py): blocked masks, m = n = k, batch = heads = 2, integer-valued fp32
    inputs in [0, 100) -- seeded here, unseeded there."""
    store = {}
    names = []
    g = torch.Generator().manual_seed(1234)
    for n, p in [(10, 2), (10, 5), (10, 7), (16, 5), (16, 16), (32, 10), (32, 20), (32, 32), (128, 57)]:
        name = f"blocked_{n}_{p}"
        mask = ah.create_blocked_mask(n, p)
        acsr = ah.create_acsr(mask, 16, "cpu")
        T = acsr[5]
        B = H = 2
        left = torch.randint(0, 100, (B, H, n, n), generator=g).float()
        right = torch.randint(0, 100, (B, H, n, n), generator=g).float()
        s = run_sddmm(r_sddmm, mask, acsr, left, right, torch.float32)
        x = torch.randint(0, 100, (B, H, n, T), generator=g).float()
        sm = run_softmax(r_softmax, mask, acsr, x, torch.float32)
        pl = torch.randint(0, 100, (B, H, n, T), generator=g).float()
        vr = torch.randint(0, 100, (B, H, n, n), generator=g).float()
        o = run_spmm(r_spmm, mask, acsr, pl, vr, torch.float32)
        for k, v in dict(sddmm_x=left, sddmm_y=right, sddmm_out=s, softmax_x=x, softmax_out=sm,
                         spmm_x=pl, spmm_y=vr, spmm_out=o).items():
            store[f"{name}/{k}"] = v.numpy()
        store[f"{name}/params"] = np.asarray([n, p, T], dtype=np.int64)
        names.append(name)
        print(name, "T", T, flush=True)
    store["names"] = np.asarray(names)
    np.savez_compressed(out_path, **store)
    print("wrote", out_path)


def gen_cfg1(ah, r_sddmm, r_softmax, r_spmm, out_path):
    """Benchmark configuration 1 through the three reference launchers.  SpMM is only recorded
    for rows < head_dim (the others are never written by the reference kernel)."""
    B, H, L, d, w = 1, 2, 256, 32, 32
    torch.manual_seed(0)
    q = torch.randn(B, H, L, d)
    k = torch.randn(B, H, L, d)
    v = torch.randn(B, H, L, d)
    kt = k.transpose(2, 3).contiguous()
    mask = ah.create_causal_windowed_mask(L, w - 1)
    acsr = ah.create_acsr(mask, 16, "cpu")
    s = run_sddmm(r_sddmm, mask, acsr, q, kt, torch.float32)
    p = run_softmax(r_softmax, mask, acsr, s, torch.float32)
    o = run_spmm(r_spmm, mask, acsr, p, v, torch.float32)
    # an fp16 SDDMM of the same problem (the interpreter handles fp16, not bf16)
    s16 = run_sddmm(r_sddmm, mask, acsr, q.half(), kt.half(), torch.float16)
    np.savez_compressed(out_path, q=q.numpy(), k=k.numpy(), v=v.numpy(), sddmm_out=s.numpy(),
                        softmax_out=p.numpy(), spmm_out_rows_lt_d=o[:, :, :d].numpy(),
                        sddmm_out_fp16=s16.numpy(), trailing_dim=np.int64(acsr[5]))
    print("wrote", out_path)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--configs", action="store_true", help="also the four large patterns (slow)")
    ap.add_argument("--only-configs", action="store_true")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "SPLAT"))
    import acsr_helpers as ah
    import r_sddmm
    import r_softmax
    import r_spmm
    if not args.only_configs:
        gen_metadata(ah, r_sddmm, os.path.join(HERE, "acsr_metadata.npz"))
        gen_reftests(ah, r_sddmm, r_softmax, r_spmm, os.path.join(HERE, "kernels_reftests.npz"))
        gen_cfg1(ah, r_sddmm, r_softmax, r_spmm, os.path.join(HERE, "kernels_cfg1.npz"))
    if args.configs or args.only_configs:
        gen_config_metadata(ah, os.path.join(HERE, "acsr_metadata_configs.npz"))


if __name__ == "__main__":
    main()
