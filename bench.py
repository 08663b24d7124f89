#!/usr/bin/env python
"""Benchmark of the quantised decode path.

Workload (one GPU): the Large-class decoder of the benchmark spec (32 layers,
d_model 4096, 32 query / 8 KV heads, head_dim 128, SwiGLU hidden 14336, vocab
32000), random N(0, 0.02) weights quantised to group-128 INT4 (bf16 scale, u4
zero point), INT8 KV cache, a 512-token random prompt, then greedy decode at
batch 1.  A step is one decode step (one new token per sequence).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

Prints one JSON line (rank 0).  `value` is decode tokens/s with everything
resident on the GPU (graph-replayed steps, on-device greedy sampling); `e2e` is
the same loop through the host API with the token ids crossing PCIe both ways
every step; `roofline` is for the fused dequant-GEMV kernel; `cpu_baseline` is
the oracle's dense f32 decoder (the reference's CPU path restated in C) on the
host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LARGE = dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn_hidden=14336,
             vocab=32000, max_seq=1024)
PROMPT, NEW_TOKENS = 512, 256
LINEARS = ["wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down"]


def linear_shapes(c, tp=1):
    qd, kd = c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]
    return {"wq": (qd, c["d_model"]), "wk": (kd, c["d_model"]), "wv": (kd, c["d_model"]),
            "wo": (c["d_model"], qd), "w_gate": (c["ffn_hidden"], c["d_model"]),
            "w_up": (c["ffn_hidden"], c["d_model"]), "w_down": (c["d_model"], c["ffn_hidden"])}


def w4_bytes(n, k, g=128):
    """Algorithmic bytes of one group-wise INT4 weight: codes + bf16 scale + u4 zero per group."""
    return n * k // 2 + (k // g) * n * 2 + (k // g) * n // 2


def step_weight_bytes(c):
    per_layer = sum(w4_bytes(n, k) for n, k in linear_shapes(c).values())
    return c["n_layers"] * per_layer + w4_bytes(c["vocab"], c["d_model"])


def kv_bytes_per_token(c):
    """INT8 K and V of one cached token in every layer, with their f32 scales."""
    return c["n_layers"] * (2 * c["n_kv_heads"] * c["head_dim"] + 2 * c["n_kv_heads"] * 4)


# dram__bytes_read.sum + dram__bytes_write.sum of gemv_w4a16_m1_kernel divided by its
# algorithmic bytes, from one ncu capture on a 4096 x 128256 weight with one token
# (profiles/gemv_w4a16_m1_kernel__k4096_n128256_m1.md).  The kernel streams every
# weight block exactly once whatever the shape, so traffic grows in proportion to the bytes.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 283.18 / 279.4


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi.  The process is
    started ahead of the warm-up (its start-up takes longer than a short timed
    region); only rows that arrive between begin() and end() count."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.rows, self.proc, self.gpu = [], None, gpu_index
        self.windows, self._t0 = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [x.strip() for x in line.split(",")]))

    def begin(self):
        deadline = time.monotonic() + 5.0
        while self.proc and not self.rows and time.monotonic() < deadline:
            time.sleep(0.01)
        self._t0 = time.monotonic()

    def end(self):
        self.windows.append((self._t0, time.monotonic() + 0.06))

    def __enter__(self):
        self.begin()
        return self

    def __exit__(self, *exc):
        self.end()

    def close(self):
        if self.proc:
            time.sleep(0.08)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.proc = None

    def summary(self):
        self.close()
        rows = [r for t, r in self.rows if any(a <= t <= b for a, b in self.windows) and len(r) >= 9]
        sm = sorted(int(r[1]) for r in rows if r[1].isdigit())
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mx = [int(r[2]) for r in rows if r[2].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_large(pkg, torch, cfg, seed=0, tp_rank=0, tp_world=1):
    """Random N(0, 0.02) weights, quantised on the GPU to group-128 INT4.  Under
    tensor parallelism every rank draws the same full weights and keeps its shard."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    weights = {}

    def make(name, n, k):
        w = torch.randn((n, k), generator=gen, device="cuda", dtype=torch.float32) * 0.02
        return pkg.QuantLinear.quantise(pkg.parallel.shard_weight(name, w, tp_rank, tp_world), "w4a16", 128)

    weights["embedding"] = make("embedding", cfg["vocab"], cfg["d_model"])
    weights["lm_head"] = make("lm_head", cfg["vocab"], cfg["d_model"])
    weights["final_norm"] = torch.ones(cfg["d_model"], device="cuda")
    for l in range(cfg["n_layers"]):
        for name, (n, k) in linear_shapes(cfg).items():
            weights[f"layers.{l}.{name}"] = make(f"layers.{l}.{name}", n, k)
        weights[f"layers.{l}.norm1"] = torch.ones(cfg["d_model"], device="cuda")
        weights[f"layers.{l}.norm2"] = torch.ones(cfg["d_model"], device="cuda")
    mc = pkg.ModelConfig(cfg["n_layers"], cfg["d_model"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"],
                         cfg["ffn_hidden"], cfg["vocab"], cfg["max_seq"], 1e-5, 10000.0, False)
    if tp_world > 1:
        mc = pkg.parallel.shard_config(mc, tp_world)
    return mc, weights


def time_gemv_only(pkg, torch, weights, cfg, steps, stream):
    """Average duration of the dequant-GEMV launches of one decode step (the four
    fused projections of each layer and the LM head), timed with CUDA events on
    the launching stream over graph replays.  Returns (seconds per launch,
    launches per step, algorithmic bytes per launch)."""
    from aarambh_ai_b200._lib import lib, check
    import ctypes as C
    d, hd = cfg["d_model"], cfg["head_dim"]
    fused = []
    keep = []
    for l in range(cfg["n_layers"]):
        def cat(names):
            parts = (C.c_void_p * len(names))(*[weights[f"layers.{l}.{n}"]._h for n in names])
            h = C.c_void_p()
            check(lib.ab2_qweight_concat_rows(C.byref(h), parts, len(names)))
            q = pkg.QuantLinear(h.value)
            keep.append(q)
            return q
        fused += [cat(["wq", "wk", "wv"]), weights[f"layers.{l}.wo"], cat(["w_gate", "w_up"]),
                  weights[f"layers.{l}.w_down"]]
    fused.append(weights["lm_head"])
    xs = {k: torch.randn(1, k, device="cuda").to(torch.bfloat16) for k in {w.in_features for w in fused}}
    with torch.cuda.stream(stream):
        for w in fused:
            w(xs[w.in_features])
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for w in fused:
                w(xs[w.in_features])
        g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
            g.replay()
        b.record(stream)
        stream.synchronize()
    sec = a.elapsed_time(b) * 1e-3 / (steps * len(fused))
    alg = sum(w4_bytes(w.out_features, w.in_features) + 2 * (w.in_features + w.out_features) for w in fused)
    del keep
    return sec, len(fused), alg / len(fused)


def cpu_decode_baseline(pkg, torch, weights, cfg, steps, warmup, ctx):
    """The oracle's dense f32 decoder (the reference's CPU path: weights
    dequantised once at load, f32 GEMV per token, f32 KV) timed on the host
    cores for `steps` decode tokens at context `ctx`."""
    import numpy as np
    from oracle import oracle as orc
    dense = {}
    for name, w in weights.items():
        dense[name] = (w.dequantise(torch.float32) if hasattr(w, "dequantise") else w.float()).cpu().numpy()
    c = dict(cfg, eps=1e-5, rope_theta=10000.0)
    orc.use_all_cores()  # torchrun exports OMP_NUM_THREADS=1 to its workers
    model = orc.DenseModel(c, dense, 1, ctx + steps + warmup + 1)
    model.fill_cache(0, ctx, 1)
    tok = np.array([[17]], np.uint32)
    for i in range(warmup):
        tok = np.array([[orc.argmax(model.forward(tok, [ctx + i])[0, 0])]], np.uint32)
    t0 = time.perf_counter()
    for i in range(steps):
        tok = np.array([[orc.argmax(model.forward(tok, [ctx + warmup + i])[0, 0])]], np.uint32)
    dt = time.perf_counter() - t0
    return steps / dt, orc.num_threads(), dt


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--cpu-steps", type=int, default=12)
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline (profiling runs)")
    args = ap.parse_args()

    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and rank != 0:
        return 0
    torch.cuda.set_device(local_rank)
    from __graft_entry__ import import_package
    pkg = import_package()
    cfg = LARGE
    B = args.batch
    workload = f"large_decode_b{B}_ctx{PROMPT}"

    if args.impl == "reference":
        mc, weights = build_large(pkg, torch, cfg)
        K = max(1, min(args.steps, 40))
        W = max(1, min(args.warmup, 3))
        tok_s, cores, dt = cpu_decode_baseline(pkg, torch, weights, cfg, K, W, PROMPT)
        line = {"impl": "reference", "metric": "INT4 decode tok/s", "value": round(tok_s, 4), "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": round(1e3 / tok_s, 3),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": "large_decode_b1_ctx512", "path": "oracle port of the reference CPU path: "
                           "weights dequantised to dense f32 at load, f32 GEMV per token, f32 KV cache"},
                "cpu_baseline": {"value": round(tok_s, 4), "unit": "tokens/s", "cores": cores, "kind": "port",
                                 "sample": f"{K} decode steps at batch 1, context {PROMPT} (cache pre-filled), all 32 layers"},
                "e2e": {"value": round(tok_s, 4), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    tp = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        tp = pkg.TensorParallel.from_torch_distributed()
    mc, weights = build_large(pkg, torch, cfg, tp_rank=rank, tp_world=world)
    model = pkg.AarambhModel(mc, weights, dtype=torch.bfloat16, max_tokens=max(PROMPT, B), tp=tp)
    cache = model.empty_kv_cache_with_capacity(PROMPT + NEW_TOKENS + args.warmup + args.steps + 8, batch=B, dtype="int8")
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg["vocab"], (B, PROMPT), generator=gen)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for b in range(B):
            logits = model.forward_with_cache(prompt[b:b + 1], 0, cache, row=b, last_only=True)
        first = pkg.dispatch.argmax(logits.view(1, -1)).repeat(B)
        bufs = [first.clone(), torch.empty(B, dtype=torch.int32, device="cuda")]
        step_no = 0

        def step():
            nonlocal step_no
            model.decode_step(bufs[step_no % 2], cache, None, bufs[(step_no + 1) % 2])
            step_no += 1

        clocks = ClockSampler(local_rank)
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        a, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with clocks:
            a.record(stream)
            for _ in range(args.steps):
                step()
            b_ev.record(stream)
            stream.synchronize()
        dev_ms = a.elapsed_time(b_ev)
        if world > 1:
            t = torch.tensor([dev_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dev_ms = float(t[0])
        ms_per_step = dev_ms / args.steps

        # end to end through the host API: token ids cross PCIe both ways every step
        ids_host = torch.empty(B, dtype=torch.int32).pin_memory()
        out_host = torch.empty(B, dtype=torch.int32).pin_memory()
        ids_dev = torch.empty(B, dtype=torch.int32, device="cuda")
        out_dev = torch.empty(B, dtype=torch.int32, device="cuda")
        ids_host.copy_(bufs[step_no % 2].cpu())
        e2e_steps = max(8, args.steps // 4)

        def host_step():
            ids_dev.copy_(ids_host, non_blocking=True)
            model.decode_step(ids_dev, cache, None, out_dev)
            out_host.copy_(out_dev, non_blocking=True)
            stream.synchronize()
            ids_host.copy_(out_host)

        for _ in range(3):
            host_step()
        with clocks:
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                host_step()
            e2e_s = (time.perf_counter() - t0) / e2e_steps

    local_cfg = dict(cfg, n_heads=cfg["n_heads"] // world, n_kv_heads=cfg["n_kv_heads"] // world,
                     ffn_hidden=cfg["ffn_hidden"] // world)
    gemv_s, gemv_launches, gemv_bytes = time_gemv_only(pkg, torch, weights, local_cfg, max(8, args.steps // 4), stream)
    status = pkg.device_status()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = gemv_bytes / gemv_s / 1e9
    ctx_mid = PROMPT + max(args.warmup, 3) + args.steps // 2
    # per GPU: a rank reads its 1/world share of the layer weights, head and KV
    step_bytes = (step_weight_bytes(cfg) + B * ctx_mid * kv_bytes_per_token(cfg)) // world
    # embedding, per layer {norm+qkv, attention, o, norm+gate|up+SwiGLU, down} (tensor parallel: the same five,
    # the partial sums travel in the projections' epilogues and the next GEMV's prologue), norm+head, argmax,
    # commit; NCCL's all-gather of the logits shards is not counted
    launches_per_step = (1 + cfg["n_layers"] * 5 + 3) if B == 1 else None

    line = {
        "metric": "INT4 decode tok/s", "value": round(B * 1e3 / ms_per_step, 2), "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 activations, f32 accumulate, u4 weights, i8 KV", "data": "synthetic",
        "config": {"workload": workload, "batch": B, "prompt": PROMPT, "weights": "W4A16 g128 (bf16 scale, u4 zero)",
                   "kv": "int8 per token per head", "parallelism": f"tp{world}",
                   "l2": "weights (3.7 GB per step) exceed the 126 MB L2"},
        "step_bytes": step_bytes,
        "step_hbm_frac": round(step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak, 4),
        "roofline": {"bound": "hbm", "kernel": "gemv_w4a16_m1_kernel (gemv_w4a16_warp_kernel where K > 8192)", "achieved": round(achieved, 1),
                     "peak": hbm_peak, "unit": "GB/s", "frac": round(achieved / hbm_peak, 4),
                     "traffic": round(gemv_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE),
                     "traffic_source": "ncu dram read+write of this kernel on a 4096 x 128256 weight, one token "
                                       "(283.18 MB for 279.4 MB algorithmic), scaled by the bytes one launch streams",
                     "peak_source": "measured" if peaks else "fallback",
                     "launches_per_step": gemv_launches, "bytes_per_launch": round(gemv_bytes)},
        "e2e": {"value": round(B / e2e_s, 2), "unit": "tokens/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 4 * B},
        "gpu_launches": (launches_per_step if launches_per_step else 1 + cfg["n_layers"] * 7 + 4) * args.steps,
        "clocks": clocks.summary(),
        "device_status": status,
    }
    if rank == 0 and world == 1 and not args.skip_cpu:
        tok_s, cores, dt = cpu_decode_baseline(pkg, torch, weights, cfg, args.cpu_steps, 2, PROMPT)
        line["cpu_baseline"] = {"value": round(tok_s, 4), "unit": "tokens/s", "cores": cores, "kind": "port",
                                "sample": f"{args.cpu_steps} decode steps at batch 1, context {PROMPT} (cache pre-filled), all 32 layers"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
