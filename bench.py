"""Benchmark of the fused sparse attention (SDDMM + softmax + SpMM over ACSR).

    python bench.py --gpus N --steps K --warmup W            # this implementation
    python bench.py --impl reference --steps K --warmup W    # CPU restatement of the reference path

Workload (default --config 5): B=8, H=64, L=32768, d=128, bf16, causal sliding window 1024,
Q,K,V ~ N(0,1), softmax scale 1/sqrt(d); the 512 (batch, head) pairs are sharded over the ranks
(strong scaling, no data-path collective).  One step = one pass of the fused kernel over the
rank's heads.  Prints ONE JSON line on rank 0:

  value         nnz-effective TFLOP/s (4*nnz*d flops per head) with inputs resident in HBM,
                all ranks' work / max-over-ranks device time
  e2e           the same metric through RegularAttention.forward_host: pinned host operands,
                host->device and device->host copies inside the timed region
  roofline      the fused kernel against the measured dense bf16 peak
  cpu_baseline  the C restatement of the reference kernels on the host cores, bounded sample; plus
                (one GPU only) the dense-masked torch chain on configurations 1 and 2
  other_configs (one GPU only) the fused kernel on configurations 2, 3 and 4, each timed for at
                least half a second with its own clock record and roofline
  check         one head of the timed output against the CPU oracle (outside the timed region)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "triton-fun_b200", "SPLAT")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "nnz_effective_tflops_sddmm_softmax_spmm"
UNIT = "TFLOP/s"

#  cfg: (B, H, L, d, dtype name, pattern, p0, p1, input scale, seed, label)
CONFIGS = {
    1: (1, 2, 256, 32, "fp32", "causal_windowed", 31, 0, 1.0, 0, "cfg1 plumbing, causal window 32"),
    2: (4, 16, 4096, 64, "fp16", "causal_windowed", 255, 0, 1.0, 1, "cfg2 local causal window 256"),
    3: (2, 32, 8192, 128, "bf16", "strided", 64, 0, 1.0, 2, "cfg3 column stride 64"),
    4: (1, 32, 16384, 128, "bf16", "dilated", 512, 2, 0.5, 3, "cfg4 dilated window 512x2"),
    5: (8, 64, 32768, 128, "bf16", "causal_windowed", 1023, 0, 1.0, 4, "cfg5 long-context causal window 1024"),
}
KIND = {"blocked": 0, "windowed": 1, "causal_windowed": 2, "strided": 3, "dilated": 4}
TORCH_DTYPE = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def nnz_per_head(cfg) -> int:
    from oracle import acsr_oracle as ao  # integer arithmetic only; not on the measured path
    B, H, L, d, dt, pat, p0, p1, *_ = CONFIGS[cfg]
    return int(ao.pattern_rows(KIND[pat], L, p0, p1)[3].sum())


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"],
                "tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU.  The sampler is started early (nvidia-smi
    takes a while to produce its first row); ``mark()`` brackets the timed region and only rows
    whose host timestamp falls inside it are summarised."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_ms: int = 20):
        self.index, self.rows, self.proc, self.t0, self.t1 = index, [], None, None, None
        self.period_ms = period_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def mark_begin(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=5)

    def summary(self):
        sm, mx, pw, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ts, r in self.rows:
            if len(r) < 7 or self.t0 is None or self.t1 is None or not (self.t0 <= ts <= self.t1 + 0.05):
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1])); pw.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w": statistics.median(pw) if pw else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(cfg, begin, end, device, chunk=64):
    """Q, K, V for flat heads [begin, end); seeded per (config, 64-head chunk) so that the values do
    not depend on how many GPUs share the work."""
    B, H, L, d, dt, pat, p0, p1, spread, seed, _ = CONFIGS[cfg]
    dtype = TORCH_DTYPE[dt]
    outs = [torch.empty((1, end - begin, L, d), dtype=dtype, device=device) for _ in range(3)]
    c0 = begin // chunk
    while c0 * chunk < end:
        g = torch.Generator(device=device).manual_seed(seed * 100003 + c0)
        lo, hi = max(begin, c0 * chunk), min(end, (c0 + 1) * chunk)
        for t in outs:
            full = torch.randn((chunk, L, d), generator=g, device=device, dtype=torch.float32)
            t[0, lo - begin:hi - begin] = (full[lo - c0 * chunk:hi - c0 * chunk] * spread).to(dtype)
            del full
        c0 += 1
    return outs


def cpu_reference_sample(cfg, budget_s=20.0, max_heads=16):
    """Times the C restatement of the reference path (three kernels, S and P materialised) on the
    host cores over a bounded number of heads of the workload.  Returns (tflops, heads, seconds,
    threads)."""
    import numpy as np
    from oracle import acsr_oracle as ao
    from oracle import c_oracle
    B, H, L, d, dt, pat, p0, p1, spread, seed, _ = CONFIGS[cfg]
    meta = ao.metadata_from_pattern(KIND[pat], L, p0, p1, 16)
    T = meta["trailing_dim"]
    rng = np.random.default_rng(seed)
    one = [(rng.standard_normal((1, L, d), dtype=np.float32) * spread) for _ in range(3)]
    scale = d ** -0.5
    t0 = time.perf_counter()
    c_oracle.attention(*one, meta, T, scale)
    t1 = time.perf_counter() - t0
    heads = int(max(1, min(max_heads, budget_s / max(t1, 1e-3))))
    qkv = [np.repeat(x, heads, axis=0) for x in one] if heads > 1 else one
    t0 = time.perf_counter()
    c_oracle.attention(*qkv, meta, T, scale)
    dt_s = time.perf_counter() - t0
    flops = 4.0 * nnz_per_head(cfg) * d * heads
    return flops / dt_s / 1e12, heads, dt_s, c_oracle.num_threads()


def torch_dense_masked_baseline(cfgs=(1, 2), budget_s=12.0):
    """The dense-masked torch chain (einsum, mask, softmax, matmul: what the reference's own
    checker `truth` computes, SPLAT/r_sddmm.py:186-187) on the host cores, whole configurations."""
    from oracle import acsr_oracle as ao
    from oracle import attention_oracle as at
    out = []
    for cfg in cfgs:
        B, H, L, d, dt, pat, p0, p1, spread, seed, label = CONFIGS[cfg]
        meta = ao.metadata_from_pattern(KIND[pat], L, p0, p1, 16)
        g = torch.Generator().manual_seed(seed)
        q, k, v = ((torch.randn(B, H, L, d, generator=g) * spread).to(TORCH_DTYPE[dt]) for _ in range(3))
        t0 = time.perf_counter()
        at.attention_dense_masked(q, k.transpose(2, 3), v, meta, d ** -0.5)
        secs = time.perf_counter() - t0
        calls = 1
        while secs < 0.2 and calls < 64:      # tiny configurations: repeat for a stable figure
            t0 = time.perf_counter()
            for _ in range(calls * 2):
                at.attention_dense_masked(q, k.transpose(2, 3), v, meta, d ** -0.5)
            secs = (time.perf_counter() - t0) / (calls * 2)
            calls *= 2
            if secs * calls > 0.5:
                break
        flops = 4.0 * nnz_per_head(cfg) * d * B * H
        out.append({"workload": label, "ms_per_call": secs * 1e3, "value": flops / secs / 1e12, "unit": UNIT,
                    "threads": torch.get_num_threads()})
        budget_s -= secs
        if budget_s < 0:
            break
    return out


# fused band kernel by the library's SPLAT_B200_BAND_TILES switch (default: one Q tile per CTA)
BAND_KERNELS = {"1": "attention_band1_kernel", "2": "attention_band_kernel", "3": "attention_pair_kernel"}


def ncu_traffic(cfg, heads, path):
    """DRAM bytes per launch of the fused kernel from the ncu captures summarised under
    profiles/ (dram__bytes_read.sum + dram__bytes_write.sum), scaled by the head count, with the
    capture it came from.  None if the kernel sources changed after the capture."""
    meta_path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    if path != "band" or not os.path.exists(meta_path):
        return None, None
    if os.environ.get("SPLAT_B200_BAND_TILES", "1")[:1] != "1":
        return None, "the traffic record covers the default kernel only"
    with open(meta_path) as f:
        text = f.read()
    try:
        rec = json.loads(text.split("```json", 1)[1].split("```", 1)[0])
    except (IndexError, ValueError):
        return None, "profiles/dram_traffic.md holds no readable record"
    entry = rec["configs"].get(str(cfg))
    if entry is None:
        return None, None
    import hashlib
    h = hashlib.sha1()
    for name in rec["kernel_sources"]:
        with open(os.path.join(ROOT, name), "rb") as f:
            h.update(f.read())
    if h.hexdigest() != rec["kernel_sources_sha1"]:
        return None, "kernel sources changed since the capture of " + rec["captured"]
    return entry["bytes"] / entry["heads"] * heads, f"ncu capture of {rec['captured']}: {entry['what']}"


def time_config(cfg, dev, min_seconds=0.5, max_launches=20000):
    """The fused kernel on one of the smaller configurations, whole configuration on this GPU,
    launches repeated until the timed region spans min_seconds (clock samples every 20 ms)."""
    import r_attention
    import acsr_helpers as ah
    import splat_native as n
    B, H, L, d, dt, pat, p0, p1, spread, seed, label = CONFIGS[cfg]
    dtype = TORCH_DTYPE[dt]
    heads = B * H
    attn = r_attention.RegularAttention(1, L, heads, d, ah.PatternMask(KIND[pat], L, p0, p1), 16, 16, dev,
                                        dtype, scale=d ** -0.5, path=n.PATH_BAND)
    nnz = int(attn.nnzs.double().sum().item())
    q, k, v = make_inputs(cfg, 0, heads, dev)
    kt = k.transpose(2, 3)
    for _ in range(20):
        attn([q, kt, v])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(50):
        attn([q, kt, v])
    e1.record()
    torch.cuda.synchronize()
    est = e0.elapsed_time(e1) / 50
    launches = int(min(max_launches, max(200, min_seconds * 1e3 / est * 1.1)))
    clocks = ClockSampler(dev.index).start()
    time.sleep(0.3)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(launches + 1)]
    torch.cuda.synchronize()
    clocks.mark_begin()
    ev[0].record()
    for i in range(launches):
        attn([q, kt, v])
        ev[i + 1].record()
    torch.cuda.synchronize()
    clocks.mark_end()
    clocks.stop()
    attn.check_status()
    per = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(launches))
    mean_ms = ev[0].elapsed_time(ev[-1]) / launches
    peaks = measured_peaks()
    flops = 4.0 * nnz * d * heads
    bytes_alg = 4.0 * L * d * q.element_size() * heads
    t_flop, t_hbm = flops / (peaks["tflops"] * 1e12), bytes_alg / (peaks["hbm_gbs"] * 1e9)
    traffic, prov = ncu_traffic(cfg, heads, "band")
    if t_flop >= t_hbm:
        ach = flops / (mean_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"]}
    else:
        ach = bytes_alg / (mean_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"]}
    roof.update({"traffic": traffic, "traffic_source": prov, "peak_source": peaks["source"]})
    out = {"workload": label, "dtype": dt, "launches": launches, "ms": mean_ms, "ms_median": per[len(per) // 2],
           "ms_best": per[0], "value": flops / (mean_ms * 1e-3) / 1e12, "unit": UNIT, "roofline": roof,
           "clocks": clocks.summary(), "l2": "L2 flushed by the launch itself: inputs + outputs = %.0f MB per launch"
           % (bytes_alg / 1e6)}
    del attn, q, k, v
    torch.cuda.empty_cache()
    return out


def run_reference(args):
    """The reference arm: the reference's algorithm on the host cores (C restatement; the Python +
    Triton reference itself has no compiled form and is not present where this runs)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = args.config
    B, H, L, d, dt, pat, p0, p1, spread, seed, label = CONFIGS[cfg]
    budget = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    vals = []
    heads = threads = 0
    secs = 0.0
    for i in range(args.warmup + args.steps):
        v, heads, secs, threads = cpu_reference_sample(cfg, budget_s=budget)
        if i >= args.warmup:
            vals.append(v)
    value = statistics.median(vals)
    sample = f"{heads} of {B * H} heads per step ({secs:.2f} s), fp32, S and P materialised"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        # a step of this arm is a SAMPLE of heads; the step time is scaled to all heads
        "ms_per_step": secs * 1e3 * (B * H) / heads, "sample_heads": heads, "sample_ms": secs * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": label, "B": B, "H": H, "L": L, "d": d,
                                        "pattern": pat, "p0": p0, "p1": p1},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch.distributed as dist
    import r_attention
    import acsr_helpers as ah
    import splat_native as n
    from sharding import shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    cfg = args.config
    B, H, L, d, dt, pat, p0, p1, spread, seed, label = CONFIGS[cfg]
    dtype = TORCH_DTYPE[dt]
    total_heads = B * H if args.heads <= 0 else min(B * H, args.heads)
    begin, end = shard_range(total_heads, world, rank)
    heads = end - begin
    scale = d ** -0.5

    mask = ah.PatternMask(KIND[pat], L, p0, p1)
    t0 = time.perf_counter()
    unfused = args.path == "unfused"
    if unfused:
        args.no_e2e = True   # forward_host streams the fused kernel only
    attn = r_attention.RegularAttention(1, L, heads, d, mask, 16, 16, dev, dtype, scale=scale,
                                        fused=not unfused,
                                        path=n.PATH_BAND if args.path == "band" else
                                        (n.PATH_GENERIC if args.path == "generic" else n.PATH_AUTO))
    torch.cuda.synchronize()
    metadata_ms = (time.perf_counter() - t0) * 1e3
    nnz = int(attn.nnzs.double().sum().item())       # non-zeros per head, from the device metadata
    flops_per_head = 4.0 * nnz * d
    q, k, v = make_inputs(cfg, begin, end, dev)
    kt = k.transpose(2, 3)
    if args.kt == "contiguous":      # the reference's own layout: a contiguous (B,H,d,L) tensor
        kt = kt.contiguous()
        args.no_e2e = True           # forward_host streams row-major K

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- device-resident timing
    clocks = ClockSampler(local_rank).start()
    for _ in range(args.warmup):
        attn([q, kt, v])
    attn.check_status()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    clocks.mark_begin()
    ev[0].record()
    for i in range(args.steps):
        attn([q, kt, v])
        ev[i + 1].record()
    barrier()
    clocks.mark_end()
    clocks.stop()
    attn.check_status()
    per_launch = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps))
    ms_total = ev[0].elapsed_time(ev[-1])
    ms_step = ms_total / args.steps
    t = torch.tensor([ms_step], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step_max = float(t.item())
    value = flops_per_head * total_heads / (ms_step_max * 1e-3) / 1e12

    # ---------------------------------------------------------------- result check, one head
    check = None
    if rank == 0 and not args.no_check:
        from oracle import acsr_oracle as ao
        from oracle import attention_oracle as at
        out = attn([q, kt, v])
        torch.cuda.synchronize()
        meta = ao.metadata_from_pattern(KIND[pat], L, p0, p1, 16)
        hsel = heads - 1                                   # the last head of this rank's shard
        ref = at.attention_acsr(q[:, hsel:hsel + 1].cpu(), k[:, hsel:hsel + 1].cpu().transpose(2, 3),
                                v[:, hsel:hsel + 1].cpu(), meta, meta["trailing_dim"], scale)
        got = out[:, hsel:hsel + 1].float().cpu()
        err = (got - ref).abs()
        tol = {"fp32": (1e-4, 1e-4)}.get(dt, (2e-2, 1e-2))
        check = {"against": "oracle.attention_oracle.attention_acsr (fp32, CPU), one head of the timed output",
                 "head": begin + hsel, "max_abs_err": float(err.max()),
                 "within_tolerance": bool((err <= tol[0] + tol[1] * ref.abs()).all()),
                 "tolerance": f"abs {tol[0]} + rel {tol[1]}"}
        del out, ref, got, err

    # ---------------------------------------------------------------- end to end, host operands
    e2e = None
    if not args.no_e2e:
        import psutil
        need = 4 * heads * L * d * q.element_size()
        share_host = psutil.virtual_memory().available < 2.5 * need * max(1, world)
        h_heads = min(heads, 32) if share_host else heads
        host = [torch.empty((1, h_heads, L, d), dtype=dtype, pin_memory=True) for _ in range(4)]
        for hbuf, src in zip(host[:3], (q, k, v)):
            hbuf.copy_(src[:, :h_heads])
        torch.cuda.synchronize()

        def e2e_step():
            if share_host:   # host RAM too small for the whole shard: re-send the same pinned chunk
                for b in range(0, heads, h_heads):
                    attn.forward_host(host[0], host[1], host[2], host[3], chunk_heads=h_heads)
            else:
                attn.forward_host(host[0], host[1], host[2], host[3], chunk_heads=32)

        e2e_steps = max(1, min(args.steps, args.e2e_steps))
        for _ in range(min(args.warmup, 2)):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        attn.check_status()
        te = torch.tensor([e0.elapsed_time(e1) / e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        # result check of the host path on one head
        if rank == 0:
            q1, k1, v1 = (t[:, :1].contiguous() for t in (q, k, v))
            o1 = torch.empty_like(q1)
            n.attention_fused(q1, k1.transpose(2, 3), v1, o1, attn.sTod_linear_transformations,
                              attn.sTod_translations, attn.nnzs, scale, attn.path, attn.plan)
            assert torch.equal(o1.cpu(), host[3][:, :1]), "forward_host disagrees with forward"
        # what the copies alone cost: the same pinned buffers through the same staging, no kernel
        def copies_only():
            # the same traffic as one e2e step, host->device and device->host on their own
            # streams as forward_host runs them, without the kernels and their dependencies
            st = attn._host_stage
            c = st["chunk"]
            cur = torch.cuda.current_stream(dev)
            st["s_in"].wait_stream(cur)
            st["s_out"].wait_stream(cur)
            for i in range(-(-heads // c)):
                buf = st["bufs"][i % 2]
                with torch.cuda.stream(st["s_in"]):
                    for key, src in (("q", host[0]), ("k", host[1]), ("v", host[2])):
                        buf[key][:, :c].copy_(src[:, :c], non_blocking=True)
                with torch.cuda.stream(st["s_out"]):
                    host[3][:, :c].copy_(buf["o"][:, :c], non_blocking=True)
            cur.wait_stream(st["s_in"])
            cur.wait_stream(st["s_out"])
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        copies_only()
        c1.record()
        barrier()
        tc = torch.tensor([c0.elapsed_time(c1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tc, op=dist.ReduceOp.MAX)
        copy_bytes = 4 * heads * L * d * q.element_size() * world
        copy_gbs = copy_bytes / (float(tc.item()) * 1e-3) / 1e9
        e2e_gbs = copy_bytes / (float(te.item()) * 1e-3) / 1e9
        e2e = {"value": flops_per_head * total_heads / (float(te.item()) * 1e-3) / 1e12, "unit": UNIT,
               "copy_ceiling_gbs": copy_gbs, "achieved_copy_gbs": e2e_gbs,
               "frac_of_copy_ceiling": e2e_gbs / copy_gbs,
               "copy_ceiling": "the step's host->device and device->host copies alone (same pinned buffers, the "
                               "two directions on their own streams, no kernel), all ranks at once; aggregate "
                               "GB/s over both directions",
               "h2d_bytes_per_step": 3 * heads * L * d * q.element_size() * world,
               "d2h_bytes_per_step": heads * L * d * q.element_size() * world,
               "ms_per_step": float(te.item()), "steps": e2e_steps,
               "host_buffers": "one pinned 32-head chunk re-sent" if share_host else "whole shard pinned"}
        del host

    # ---------------------------------------------------------------- CPU baseline (rank 0, N=1)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        val, h, secs, threads = cpu_reference_sample(cfg, budget_s=args.cpu_budget)
        cpu = {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{h} of {total_heads} heads ({secs:.1f} s) of the same workload, fp32, "
                         "three kernels with S and P materialised",
               "host_cpus": os.cpu_count(),
               "torch_dense_masked": torch_dense_masked_baseline()}

    # ---------------------------------------------------------------- the smaller configurations
    other = None
    if rank == 0 and world == 1 and not args.no_other and cfg == 5 and args.path == "band":
        del q, k, v, kt
        torch.cuda.empty_cache()
        other = [time_config(c, dev) for c in (2, 3, 4)]
        q = torch.empty(1, dtype=dtype, device=dev)     # element size for the figures below

    if rank == 0:
        peaks = measured_peaks()
        launch_ms = statistics.mean(per_launch)
        launch_ms_median, launch_ms_best = per_launch[len(per_launch) // 2], per_launch[0]
        achieved = flops_per_head * heads / (launch_ms * 1e-3) / 1e12
        bytes_alg = 4.0 * L * d * q.element_size() * heads
        if unfused:   # S written and read, P written and read, on top of Q, K, V, O
            bytes_alg += 4.0 * L * int(attn.acsr_trailing_dim) * q.element_size() * heads
        t_flop = flops_per_head * heads / (peaks["tflops"] * 1e12)
        t_hbm = bytes_alg / (peaks["hbm_gbs"] * 1e9)
        tensor_bound = t_flop >= t_hbm and not unfused
        if tensor_bound:
            roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["tflops"]}
        else:
            gbs = bytes_alg / (launch_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"]}
        traffic, traffic_source = ncu_traffic(cfg, heads, args.path)
        roof.update({"traffic": traffic, "traffic_unit": "bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum, "
                                                         "ncu capture scaled by heads)",
                     "traffic_source": traffic_source,
                     "kernel": "sddmm + softmax + spmm (three launches)" if unfused else
                               (BAND_KERNELS.get(os.environ.get("SPLAT_B200_BAND_TILES", "1")[:1], "attention_band1_kernel")
                                if args.path == "band" else "attention_rows_kernel"),
                     "peak_source": peaks["source"],
                     "peak_kind": "burst", "launch_ms": launch_ms, "launch_ms_median": launch_ms_median,
                     "launch_ms_best": launch_ms_best,
                     "frac_of_sustained_peak": (achieved / peaks["tflops_sustained"])
                     if tensor_bound and peaks.get("tflops_sustained") else None,
                     "algorithmic_gflop_per_launch": flops_per_head * heads / 1e9,
                     "algorithmic_mb_per_launch": bytes_alg / 1e6})
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step_max, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": label, "B": B, "H": H, "L": L, "d": d, "pattern": pat, "p0": p0,
                       "p1": p1, "softmax_scale": "1/sqrt(d)", "heads_per_gpu": heads, "heads_total": total_heads,
                       "parallelism": f"(batch,head) sharded over {world} GPU(s), no collective",
                       "l2": "inputs larger than L2 (per-GPU Q+K+V = %.0f MB)" % (3 * heads * L * d * q.element_size() / 1e6),
                       "path": args.path, "kt_layout": args.kt},
            "ms_per_step_median": launch_ms_median, "ms_per_step_best": launch_ms_best,
            "e2e": e2e, "roofline": roof, "cpu_baseline": cpu, "clocks": clocks.summary(),
            "check": check, "other_configs": other,
            "gpu_launches": args.steps * world * (3 if unfused else 1), "metadata_build_ms": metadata_ms,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=5, choices=sorted(CONFIGS))
    ap.add_argument("--path", default="band", choices=["band", "generic", "auto", "unfused"],
                    help="fused kernel choice, or 'unfused': the reference's three launches (SDDMM, softmax, SpMM)")
    ap.add_argument("--kt", default="view", choices=["view", "contiguous"],
                    help="K^T operand: transposed view of a (B,H,L,d) tensor, or a contiguous (B,H,d,L) tensor")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the oracle comparison of one head")
    ap.add_argument("--no-other", action="store_true", help="skip configurations 2-4 (one GPU, configuration 5 only)")
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--heads", type=int, default=0,
                    help="profiling aid: run only the first N (batch, head) pairs of the workload")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
