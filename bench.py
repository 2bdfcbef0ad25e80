#!/usr/bin/env python
"""Benchmark of the mograd training hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A "step" is one full train step (forward, backward, gradient exchange when
N > 1, AdamW) on one batch of seeded synthetic data.  One JSON line is printed
by rank 0:

  value        whole-job tokens/s with the batch already resident in HBM
               (Model.step_resident(): the step's captured CUDA graphs are
               replayed), timed with CUDA events over exactly K steps, max
               over ranks
  e2e          the same metric through the host-facing call Model.step(): the
               batch comes from pinned host memory every step (the copy of the
               next batch is issued under the current step's kernels, and the
               next step is queued before this step's loss is waited for) and
               the loss is read back to the host every step
  gpu_launches kernels of this library run inside the timed K steps: those
               launched directly plus those recorded in each replayed graph
  dp           N > 1 only: a check that the overlapped bf16 bucket exchange
               gives the gradients a plain fp32 all-reduce gives, that the
               replicas hold identical parameters after the timed steps, and
               how long per step the main stream stood waiting for a bucket
  roofline     the dominant kernel of the step, timed live here with CUDA
               events on the launching stream
  kernels      the standalone kernels the metric names (flash-attention
               backward, LayerNorm backward, fused cross-entropy), N = 1 only
  cpu_baseline the CPU restatement of the reference's math (oracle/) timed on
               this box's host cores on a bounded sample, N = 1 only

`--impl reference` times only that CPU restatement (the reference itself is
Mojo on Modular MAX and cannot be built or run on this box).
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
sys.path.insert(0, ROOT)

WORKLOADS = {
    # the reference README's MLP
    "readme_mlp": dict(kind="mlp", dims=[4096, 4096, 4096, 10], batch=2048, tokens_per_step=2048,
                       desc="README MLP 4096-4096(ReLU)-LN-4096(ReLU)-10, batch 2048, bf16 (1 sample = 1 token)"),
    # the reference's char-level transformer example
    "char_transformer": dict(kind="tf", vocab=65, d_model=384, d_ff=1536, n_layers=6, n_heads=6, batch=64, seq=256,
                             tokens_per_step=64 * 256,
                             desc="char transformer vocab 65 ctx 256 L6 H6 d384, batch 64, bf16"),
    # GPT-2-small-shaped decoder (the configuration the tokens/s metric is quoted on)
    "gpt2_small": dict(kind="tf", vocab=50304, d_model=768, d_ff=3072, n_layers=12, n_heads=12, batch=16, seq=1024,
                       tokens_per_step=16 * 1024,
                       desc="GPT-2-small-shaped decoder L12 H12 d768 ctx 1024 vocab 50304, per-GPU batch 16, bf16"),
}
DEFAULT_WORKLOAD = "gpt2_small"
# DRAM bytes (read + write) of one launch of the roofline kernel: dram__bytes_read.sum + dram__bytes_write.sum of
# one profiler capture of that exact launch.  A stored figure, not something this run measures (a profiler cannot
# run inside a timed benchmark); the JSON line says so in roofline.traffic_source.
ROOFLINE_TRAFFIC = {"gpt2_small": 137.9e6 + 1596.0e6}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d["bf16_tflops"], tflops_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 6:
                continue
            try:
                clocks.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(clocks) if clocks else None, sm_max_mhz=mx, reasons=sorted(reasons),
                    samples=len(clocks))


# ----------------------------------------------------------------------------- model + data
def build_model(cfg, device, world, pg, seed, bucket_mb=64):
    import torch
    from mograd_b200.train import MLP, TinyTransformer

    if cfg["kind"] == "mlp":
        return MLP(cfg["dims"], cfg["batch"], dtype=torch.bfloat16, device=device, seed=seed, world_size=world,
                   process_group=pg, bucket_bytes=bucket_mb << 20)
    return TinyTransformer(cfg["vocab"], cfg["d_model"], cfg["d_ff"], cfg["n_layers"], cfg["n_heads"], cfg["batch"],
                           cfg["seq"], dtype=torch.bfloat16, device=device, seed=seed, world_size=world,
                           process_group=pg, bucket_bytes=bucket_mb << 20)


def make_batch(cfg, seed, pinned=True):
    """Seeded synthetic batch with the config's shapes and distributions, on the host."""
    import torch

    g = torch.Generator().manual_seed(seed)
    if cfg["kind"] == "mlp":
        x = torch.randn((cfg["batch"], cfg["dims"][0]), generator=g).to(torch.bfloat16)
        y = torch.randint(0, cfg["dims"][-1], (cfg["batch"],), generator=g, dtype=torch.int64)
    else:
        x = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq"]), generator=g, dtype=torch.int64)
        y = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq"]), generator=g, dtype=torch.int64)
    if pinned:
        x, y = x.pin_memory(), y.pin_memory()
    return x, y


# ----------------------------------------------------------------------------- kernel micro-benchmarks
def time_launches(fn, reps, flush=None):
    """Average device time of fn() in ms, CUDA events on the current stream, L2 flushed before each launch.

    The flush doubles as a head start for the host: it is repeated until it keeps the GPU busy for about 150 us,
    so the start event, the launch and the stop event are all queued before the GPU reaches them.  (With a
    shorter flush the GPU passes the start event and then idles until the host has prepared the launch, which
    adds the host's 15-20 us of launch preparation to every kernel shorter than that.)"""
    import torch

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    repeat = 1 if flush is None else max(1, int((1 << 30) // max(1, flush.numel() * flush.element_size())))
    total = 0.0
    for _ in range(reps):
        if flush is not None:
            for _ in range(repeat):
                flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        total += e0.elapsed_time(e1)
    return total / reps


def dominant_gemm_roofline(cfg, peaks, device):
    """Times the step's largest matmul_bias_bt launch; returns the roofline object."""
    import torch
    from mograd_b200 import dispatch as K

    if cfg["kind"] == "mlp":
        M, N, Kd = cfg["batch"], cfg["dims"][1], cfg["dims"][0]
    else:
        M, N, Kd = cfg["batch"] * cfg["seq"], cfg["vocab"], cfg["d_model"]
    g = torch.Generator(device=device).manual_seed(1)
    a = torch.randn((M, Kd), generator=g, device=device).bfloat16()
    w = (torch.randn((N, Kd), generator=g, device=device) / Kd ** 0.5).bfloat16()
    ldy = (N + 7) // 8 * 8
    out = torch.empty((M, ldy), dtype=torch.bfloat16, device=device)[:, :N]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    ms = time_launches(lambda: K.matmul_bias_strided(a, w, None, out=out), 10, flush)
    flops = 2.0 * M * N * Kd
    ach = flops / (ms * 1e-3) / 1e12
    return dict(bound="tensor", kernel=f"gemm_tc2_kernel (matmul_bias_bt {M}x{N}x{Kd})", achieved=round(ach, 1),
                peak=peaks["tflops"], unit="TFLOP/s", frac=round(ach / peaks["tflops"], 4), traffic=ROOFLINE_TRAFFIC.get(cfg.get("name")),
                algorithmic_flops=flops, algorithmic_bytes=2.0 * (M * Kd + N * Kd + M * N),
                peak_source=peaks["source"], ms_per_launch=round(ms, 4),
                traffic_source="stored profiler capture of this launch (dram read + write bytes), not measured by this run")


def standalone_kernels(peaks, device):
    """The standalone kernels the metric names, at their standalone shapes."""
    import torch
    from mograd_b200 import dispatch as K

    out = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    g = torch.Generator(device=device).manual_seed(3)
    # fused softmax-cross-entropy fwd+bwd, (16384 x 50304) bf16, index labels
    N, C = 16384, 50304
    x = (torch.randn((N, C), generator=g, device=device) * 2).bfloat16()
    idx = torch.randint(0, C, (N,), generator=g, device=device)
    dl = torch.empty_like(x)

    def ce():
        from mograd_b200.dispatch import call, _ptr, _stream, scratch_take, query
        ws = scratch_take(query("mograd_b200_softmax_xent_workspace_bytes", N, C, 0), device)
        call("mograd_b200_softmax_xent_fwd_bwd", _ptr(x), _ptr(idx), _ptr(loss), _ptr(dl), N, C, C, C, 1.0, 0,
             _ptr(ws), ws.numel(), _stream())

    loss = torch.empty((), dtype=torch.float32, device=device)
    ms = time_launches(ce, 10, flush)
    nbytes = 2.0 * N * C * 2 + 8 * N + 4
    out["softmax_xent_fwd_bwd_16384x50304_bf16"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1),
                                                         frac_hbm=round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4),
                                                         algorithmic_bytes=nbytes)
    del x, dl
    # LayerNorm backward
    for rows, cols in ((16384, 768), (131072, 768), (65536, 4096)):
        xx = torch.randn((rows, cols), generator=g, device=device).bfloat16()
        dy = torch.randn((rows, cols), generator=g, device=device).bfloat16()
        gm = torch.ones(cols, device=device).bfloat16()
        dx, dg, db = torch.empty_like(xx), torch.empty_like(gm), torch.empty_like(gm)
        ms = time_launches(lambda: K.layer_norm_bwd_dispatch(dy, xx, gm, dx_out=dx, dgamma_out=dg, dbeta_out=db), 10,
                           flush)
        nbytes = (3.0 * rows * cols + 3 * cols) * 2
        out[f"layer_norm_bwd_{rows}x{cols}_bf16"] = dict(ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1),
                                                         frac_hbm=round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4),
                                                         algorithmic_bytes=nbytes)
        del xx, dy, dx
    # flash-attention forward / backward, causal: the standalone shape and the train step's own shape
    for B, S, H, D in ((4, 4096, 16, 128), (16, 1024, 12, 64)):
        try:
            q, k, v = (torch.randn((B, S, H, D), generator=g, device=device).bfloat16() for _ in range(3))
            do = torch.randn((B, H, S, D), generator=g, device=device).bfloat16()
            o, lse = K.flash_attn_fwd_dispatch(q, k, v, None, None, True, False)
            outs = (torch.empty_like(q), torch.empty_like(q), torch.empty_like(q))
            ms_f = time_launches(lambda: K.flash_attn_fwd_dispatch(q, k, v, None, None, True, False, out=o, lse_out=lse),
                                 10, flush)
            ms_b = time_launches(lambda: K.flash_attn_bwd_dispatch(do, o, q, k, v, None, lse, None, True, False,
                                                                   out=outs), 10, flush)
            ff, fb = 2.0 * B * H * S * S * D, 5.0 * B * H * S * S * D
            tag = f"B{B}_H{H}_S{S}_D{D}_causal"
            out[f"flash_attn_fwd_{tag}"] = dict(ms=round(ms_f, 4), tflops=round(ff / ms_f / 1e9, 1),
                                                frac_tensor=round(ff / ms_f / 1e9 / peaks["tflops"], 4))
            out[f"flash_attn_bwd_{tag}"] = dict(ms=round(ms_b, 4), tflops=round(fb / ms_b / 1e9, 1),
                                                frac_tensor=round(fb / ms_b / 1e9 / peaks["tflops"], 4))
            del q, k, v, do, o, outs
        except Exception as e:  # reported, never hidden
            out[f"flash_attn_B{B}_S{S}"] = dict(error=str(e)[:200])
    return out


def profile_case(name, reps, device):
    """Runs one kernel a few times on a small case (inputs > L2, < 2 GB) so a profiler capture stays short."""
    import torch
    from mograd_b200 import dispatch as K

    g = torch.Generator(device=device).manual_seed(5)
    if name == "xent":
        N, C = 4096, 50304
        x = (torch.randn((N, C), generator=g, device=device) * 2).bfloat16()
        idx = torch.randint(0, C, (N,), generator=g, device=device)
        fn = lambda: K.softmax_xent_fwd_bwd(x, idx)
    elif name == "ln_bwd":
        rows, cols = 16384, 4096
        xx = torch.randn((rows, cols), generator=g, device=device).bfloat16()
        dy = torch.randn((rows, cols), generator=g, device=device).bfloat16()
        gm = torch.ones(cols, device=device).bfloat16()
        fn = lambda: K.layer_norm_bwd_dispatch(dy, xx, gm)
    elif name == "ln_bwd_768":
        rows, cols = 131072, 768
        xx = torch.randn((rows, cols), generator=g, device=device).bfloat16()
        dy = torch.randn((rows, cols), generator=g, device=device).bfloat16()
        gm = torch.ones(cols, device=device).bfloat16()
        fn = lambda: K.layer_norm_bwd_dispatch(dy, xx, gm)
    elif name == "gemm":
        a = torch.randn((8192, 4096), generator=g, device=device).bfloat16()
        w = (torch.randn((4096, 4096), generator=g, device=device) / 64).bfloat16()
        fn = lambda: K.matmul_bias_strided(a, w)
    elif name == "gemm_lm_head":
        a = torch.randn((16384, 768), generator=g, device=device).bfloat16()
        w = (torch.randn((50304, 768), generator=g, device=device) / 28).bfloat16()
        fn = lambda: K.matmul_bias_strided(a, w)
    elif name in ("flash_fwd", "flash_bwd", "flash_fwd_d64", "flash_bwd_d64"):
        # D = 128: one batch element of the attention benchmark; D = 64: the train step's own shape
        B, S, H, D = (16, 1024, 12, 64) if name.endswith("d64") else (1, 4096, 16, 128)
        q, k, v = (torch.randn((B, S, H, D), generator=g, device=device).bfloat16() for _ in range(3))
        do = torch.randn((B, H, S, D), generator=g, device=device).bfloat16()
        o, lse = K.flash_attn_fwd_dispatch(q, k, v, None, None, True, False)
        if name.startswith("flash_fwd"):
            fn = lambda: K.flash_attn_fwd_dispatch(q, k, v, None, None, True, False)
        else:
            fn = lambda: K.flash_attn_bwd_dispatch(do, o, q, k, v, None, lse, None, True, False)
    else:
        raise SystemExit(f"unknown case {name}")
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    print(json.dumps(dict(case=name, reps=reps, status="ok")), flush=True)


# ----------------------------------------------------------------------------- in-step timeline
def step_timeline(cfg, device, steps=14):
    """Device timeline of one train step from the CUDA activity records (torch.profiler / CUPTI, no kernel
    replay): per kernel its launches and its EXCLUSIVE time inside the step, i.e. the part of each launch that does
    not overlap the kernels before it (programmatic dependent launch lets a kernel's set-up run under its
    predecessor's tail, so plain durations add up to more than the step).  Prints a table to stderr and returns
    the rows; the numbers are of a real step (the last of `steps` consecutive ones, so that the GPU has settled at
    the clocks its power cap allows), unlike per-launch times under a replaying profiler."""
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile

    model = build_model(cfg, device, 1, None, seed=0)
    bx, by = make_batch(cfg, seed=100)
    model.d_inputs.copy_(bx)
    model.d_targets.copy_(by)
    for _ in range(5):
        model.step_device()
    # the same kernel-by-kernel step timed with CUDA events over 20 steps, for comparison with the span below
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        model.step_device()
    e1.record()
    torch.cuda.synchronize()
    print(f"20 steps launched kernel by kernel, CUDA events: {e0.elapsed_time(e1) / 20:.3f} ms per step", file=sys.stderr)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            model.step_device()
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                key=lambda e: e.time_range.start)
    marks = [i for i, e in enumerate(ev) if "adamw" in e.name]  # the optimizer kernel closes a step
    if len(marks) < 2:
        raise SystemExit("timeline: fewer than two optimizer launches recorded")
    # the last complete step: the profiler starts after an idle moment, and the first steps behind it run above the
    # clocks the GPU settles at under its power cap
    step = ev[marks[-2] + 1:marks[-1] + 1]
    t0 = step[0].time_range.start
    agg, prev_end = collections.OrderedDict(), t0
    for e in step:
        s0, s1 = e.time_range.start, e.time_range.end
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").replace("mgb::", "")
        depth = 0
        for ci, ch in enumerate(name):
            depth += (ch == "<") - (ch == ">")
            if ch == "(" and depth == 0:
                name = name[:ci]
                break
        a = agg.setdefault(name[:72], [0, 0.0, 0.0])
        a[0] += 1
        a[1] += max(0.0, s1 - max(s0, prev_end))
        a[2] += s1 - s0
        prev_end = max(prev_end, s1)
    span = (prev_end - t0) / 1e3
    rows = sorted(agg.items(), key=lambda kv: -kv[1][1])
    print(f"one train step: span {span:.3f} ms, {len(step)} launches, exclusive times sum "
          f"{sum(a[1] for _, a in rows) / 1e3:.3f} ms", file=sys.stderr)
    print(f"{'launches':>8} {'exclusive ms':>13} {'share':>6} {'avg us':>8} {'avg duration us':>16}  kernel", file=sys.stderr)
    tot = sum(a[1] for _, a in rows)
    for name, (n, ex, du) in rows:
        print(f"{n:8d} {ex / 1e3:13.3f} {100 * ex / tot:5.1f}% {ex / n:8.1f} {du / n:16.1f}  {name}", file=sys.stderr)
    return dict(span_ms=round(span, 3), launches=len(step),
                kernels={k: dict(launches=n, exclusive_ms=round(ex / 1e3, 4)) for k, (n, ex, du) in rows})


# ----------------------------------------------------------------------------- CPU baseline (oracle)
def cpu_baseline(cfg, budget_s=20.0):
    """Times the CPU restatement of the same train step on a bounded sample of the batch."""
    import numpy as np
    import oracle
    from oracle import ref_model

    oracle.build()
    cores = int(os.environ.get("OMP_NUM_THREADS", "0")) or (os.cpu_count() or 1)
    rng = np.random.default_rng(0)
    if cfg["kind"] == "mlp":
        dims = cfg["dims"]
        params = {}
        for i in range(len(dims) - 1):
            b = 1.0 / dims[i] ** 0.5
            params[f"W{i}"] = rng.uniform(-b, b, (dims[i + 1], dims[i])).astype(np.float32)
            params[f"b{i}"] = rng.uniform(-b, b, dims[i + 1]).astype(np.float32)
        params["ln_g"] = np.ones(dims[1], np.float32)
        params["ln_b"] = np.zeros(dims[1], np.float32)
        n = 16
        while True:
            x = rng.standard_normal((n, dims[0])).astype(np.float32)
            y = rng.integers(0, dims[-1], n)
            t0 = time.perf_counter()
            ref_model.mlp_step(params, x, y)
            dt = time.perf_counter() - t0
            if dt > budget_s / 4 or n >= cfg["batch"]:
                break
            n = min(cfg["batch"], n * 4)
        return dict(value=round(n / dt, 2), unit="tokens/s", cores=cores, kind="port",
                    sample=f"{n} of {cfg['batch']} samples, one full fwd+bwd train step in {dt:.2f} s (OpenMP, f64 math)")
    V, d = cfg["vocab"], cfg["d_model"]
    params = {"embed": (rng.standard_normal((V, d)) * 0.02).astype(np.float32),
              "lm_head": (rng.standard_normal((V, d)) * 0.02).astype(np.float32)}
    for l in range(cfg["n_layers"]):
        for nm in ("Wq", "Wk", "Wv", "Wo"):
            params[f"{nm}{l}"] = (rng.standard_normal((d, d)) * 0.02).astype(np.float32)
        params[f"W1_{l}"] = (rng.standard_normal((cfg["d_ff"], d)) * 0.02).astype(np.float32)
        params[f"b1_{l}"] = np.zeros(cfg["d_ff"], np.float32)
        params[f"W2_{l}"] = (rng.standard_normal((d, cfg["d_ff"])) * 0.02).astype(np.float32)
        for nm in ("g1", "g2"):
            params[f"{nm}_{l}"] = np.ones(d, np.float32)
        for nm in ("be1", "be2"):
            params[f"{nm}_{l}"] = np.zeros(d, np.float32)
    def run(nb, S):
        tok = rng.integers(0, V, (nb, S))
        tgt = rng.integers(0, V, (nb, S))
        t0 = time.perf_counter()
        ref_model.transformer_step(params, tok, tgt, cfg["n_layers"], cfg["n_heads"])
        return time.perf_counter() - t0

    # calibrate on one short sequence, then size the sample to the time budget
    S = min(cfg["seq"], 128)
    nb = 1
    dt = run(nb, S)
    want = int(S * budget_s / max(dt, 1e-3))
    if want >= 2 * S:
        S = min(cfg["seq"], want // 128 * 128)
        nb = max(1, min(cfg["batch"], want // S))
        dt = run(nb, S)
    return dict(value=round(nb * S / dt, 2), unit="tokens/s", cores=cores, kind="port",
                sample=f"{nb} sequence(s) of {S} tokens (of {cfg['batch']}x{cfg['seq']}), one full fwd+bwd step in "
                       f"{dt:.2f} s (OpenMP on {cores} threads, f64 accumulation)")


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-kernels", action="store_true", help="skip the standalone kernel section")
    ap.add_argument("--case", default=None, help="run one small kernel case --reps times and exit (for profiling)")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--timeline", action="store_true",
                    help="print the per-kernel exclusive-time table of one train step (1 GPU) and exit")
    ap.add_argument("--bucket-mb", type=int, default=64, help="gradient all-reduce bucket size (N > 1)")
    ap.add_argument("--batches", type=int, default=8,
                    help="distinct seeded batches per rank, used in rotation (with one or two the model memorises "
                         "them within the run, its gradients shrink and the GPU clocks higher under its power cap)")
    args = ap.parse_args()
    # Libraries (NCCL's version banner, for one) write to stdout; the contract is one JSON line there.  Everything
    # but that line goes to stderr: fd 1 is pointed at fd 2 until emit() restores it.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)

    if args.case:
        import torch
        import mograd_b200

        mograd_b200.load()
        profile_case(args.case, args.reps, torch.device("cuda", 0))
        return 0
    cfg = dict(WORKLOADS[args.workload], name=args.workload)
    if args.timeline:
        import torch
        import mograd_b200

        mograd_b200.load()
        emit(dict(timeline=step_timeline(cfg, torch.device("cuda", 0)), workload=args.workload))
        return 0
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    base = dict(metric="train_step_tokens_per_s", unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                data="synthetic",
                config=dict(workload=args.workload, description=cfg["desc"], per_gpu_tokens=cfg["tokens_per_step"],
                            parallelism=f"dp{args.gpus}", l2="working set (weights, grads, AdamW state, activations) "
                                                             "exceeds the 126 MB L2 every step"))

    # the CPU legs use every host core (torchrun presets OMP_NUM_THREADS=1; the OpenMP runtime reads it when the
    # oracle library is first loaded, which happens after this line)
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    if args.impl == "reference":
        if rank != 0:
            return 0
        t0 = time.perf_counter()
        vals = []
        cb = None
        for _ in range(max(1, min(args.steps, 3))):
            cb = cpu_baseline(cfg, budget_s=15.0)
            vals.append(cb["value"])
            if time.perf_counter() - t0 > 120:
                break
        v = statistics.median(vals)
        cb["value"] = v
        line = dict(base, impl="reference", value=v, ms_per_step=round(1e3 * cfg["tokens_per_step"] / v, 1),
                    dtype="f32", cpu_baseline=cb, gpu_launches=0,
                    e2e=dict(value=v, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                    note="reference = CPU restatement of mograd's math (oracle/); mograd itself is Mojo/MAX and has no "
                         "CPU runtime; ms_per_step extrapolates the sample to the full batch")
        emit(line)
        return 0

    import torch
    import torch.distributed as dist
    import mograd_b200

    lib = mograd_b200.load()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    pg = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        pg = dist.group.WORLD
    peaks = load_peaks()
    model = build_model(cfg, device, world, pg, seed=0, bucket_mb=args.bucket_mb)
    # several different batches per rank, used in rotation: pinned on the host for the end-to-end loop, resident in
    # HBM for the device-timed loop (a step copies its batch device-to-device into the input slot it reads)
    nb = max(2, args.batches)
    batches = [make_batch(cfg, seed=100 + 7000 * j + rank) for j in range(nb)]
    resident = [(bx.to(device), by.to(device)) for bx, by in batches]

    def resident_step(i):
        k = i & 1
        model.use_slot(k)
        model.d_inputs.copy_(resident[i % nb][0])
        model.d_targets.copy_(resident[i % nb][1])
        return model.step_resident(k)

    resident_step(0)  # (also gives check_data_parallel below a batch to work on)
    torch.cuda.synchronize()
    hx, hy = batches[0]
    dp = None
    if world > 1:
        # the overlapped bf16 bucket exchange against a plain fp32 all-reduce of the same local gradients
        err = model.check_data_parallel()
        dp = dict(grad_exchange_max_rel_err=round(err, 6), grad_exchange_ok=bool(err <= 2e-2))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # Resident-input steps go through Model.step_resident(), which replays the step's captured CUDA graph(s)
    # (captured during the warm-up: two steps launched kernel by kernel, then one capture per input slot; with
    # several GPUs the capture is cut where a gradient bucket is complete and the all-reduces run between the cuts).
    for i in range(max(3, args.warmup) + 3):
        resident_step(i)
    barrier()
    l0 = lib.mograd_b200_launch_count()
    replayed = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = resident_step(i)
        replayed += model.graph_launches[i & 1] if model._graphs[i & 1] is not None else 0
    e1.record()
    barrier()
    # kernels of this library run inside the timed region: launched directly, plus those recorded in a replayed graph
    launches = lib.mograd_b200_launch_count() - l0 + replayed
    from mograd_b200 import _lib as _abi

    _abi.check_device_status("bench: timed steps")  # a bounded device-side wait that gave up voids the run
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    ms_per_step = ms / args.steps
    value = cfg["tokens_per_step"] * world / (ms_per_step * 1e-3)

    # end to end through the host-facing call: host batch in, loss out, every step
    # (untimed: two eager steps, then the steps in which Model.step() captures its two CUDA graphs, one per slot)
    # Every call copies its successor's batch to the device while its own step runs and (launch_next) queues that
    # successor before it waits for its own loss; the last call of each loop queues nothing, so the timed region
    # holds exactly --steps steps.
    for i in range(6):
        model.step(*batches[i % nb], prefetch=batches[(i + 1) % nb], launch_next=i < 5)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        last = model.step(*batches[i % nb], prefetch=batches[(i + 1) % nb], launch_next=i + 1 < args.steps)
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = t.item()
    clocks = sampler.stop() if rank == 0 else None  # samples span warm-up, the timed steps and the end-to-end steps
    if world > 1:
        # how long the main stream stands waiting for each bucket's all-reduce (CUDA events around every wait)
        model.time_exposed = True
        for i in range(4):
            model.use_slot(i & 1)
            model.step_device()
        torch.cuda.synchronize()
        model.time_exposed = False
        per_step = [[b.elapsed_time(a) for _, _, b, a in marks] for marks in model.exposed_events[1:]]
        tot = torch.tensor([sum(map(sum, per_step)) / max(1, len(per_step)),
                            sum(p[-1] for p in per_step if p) / max(1, len(per_step))], device=device)
        dist.all_reduce(tot, op=dist.ReduceOp.MAX)
        dp.update(allreduce_exposed_ms_per_step=round(float(tot[0]), 4),
                  last_bucket_exposed_ms_per_step=round(float(tot[1]), 4), buckets=len(model.buckets),
                  in_sync=model.replicas_in_sync(),
                  note="exposed = time the main stream waited on a bucket's all-reduce before its AdamW launch, max "
                       "over ranks; the last bucket holds the embedding gradient, final only when backward ends")
    e2e_val = cfg["tokens_per_step"] * world * args.steps / e2e_s
    h2d = hx.numel() * hx.element_size() + hy.numel() * hy.element_size()

    if rank == 0:
        line = dict(base, value=round(value, 1), ms_per_step=round(ms_per_step, 4), clocks=clocks,
                    e2e=dict(value=round(e2e_val, 1), unit="tokens/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=4),
                    gpu_launches=int(launches), loss=round(float(last), 4))
        line["config"]["batches"] = f"{nb} seeded batches per rank, used in rotation"
        line["config"]["launch"] = ("kernel by kernel" if model._graphs[0] is None else
                                    "one captured CUDA graph per step, replayed" if world == 1 else
                                    "captured CUDA graphs cut at the gradient-bucket boundaries, replayed, with the "
                                    "NCCL all-reduces issued between them")
        if dp is not None:
            line["dp"] = dp
            line["dp_in_sync"] = dp["in_sync"]
            line["allreduce_exposed_ms"] = dp["allreduce_exposed_ms_per_step"]
        line["roofline"] = dominant_gemm_roofline(cfg, peaks, device)
        if world == 1:
            if not args.no_kernels:
                line["kernels"] = standalone_kernels(peaks, device)
            line["cpu_baseline"] = cpu_baseline(cfg)
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
