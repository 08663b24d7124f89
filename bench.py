#!/usr/bin/env python
"""Benchmark of the quantised decode path.

Workload (one GPU): the Large-class decoder of the benchmark spec (32 layers,
d_model 4096, 32 query / 8 KV heads, head_dim 128, SwiGLU hidden 14336, vocab
32000), random N(0, 0.02) weights quantised to group-128 INT4 (bf16 scale, u4
zero point), INT8 KV cache, a 512-token random prompt, then greedy decode at
batch 1.  A step is one decode step (one new token per sequence).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

Prints one JSON line (rank 0).  `value` is decode tokens/s with everything
resident on the GPU (graph-replayed steps, on-device greedy sampling): the median
of BLOCKS timed blocks of --steps steps, each block starting at context 512;
`e2e` is the same loop through the host API with the token ids crossing PCIe
both ways every step; `roofline` is for the fused dequant-GEMV kernel;
`cpu_baseline` is the oracle's dense f32 decoder (the reference's CPU path
restated in C) on the host cores; `batch32` and `prefill` are the benchmark
spec's other two measurements of this model, taken outside the timed region.
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
BLOCKS = 5   # timed blocks of --steps steps; the median block is reported
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
# algorithmic bytes, from ncu captures of the kernel on one token: 283.10 MB against 279.4 MB on
# a 4096 x 128256 weight, and the in-step gate|up shape (4096 x 28672).  The kernel streams
# every weight block exactly once whatever the shape, so traffic grows in proportion to the bytes.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 283.10 / 279.4


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


def cpu_dense_weights(cfg, seed=0):
    """Dense f32 weights for the CPU arm, made without the GPU library: one N(0, 0.02) tensor
    per projection shape, shared by all layers (the reference dequantises to dense f32 at load;
    the timing does not depend on the values, and 0.9 GB per layer is far beyond any cache, so
    sharing the buffers between layers changes nothing in what is streamed from memory)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    dense = {}
    shared = {name: (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
              for name, shape in linear_shapes(cfg).items()}
    head = rng.standard_normal((cfg["vocab"], cfg["d_model"]), dtype=np.float32) * np.float32(0.02)
    dense["embedding"] = head
    dense["lm_head"] = head
    dense["final_norm"] = np.ones(cfg["d_model"], np.float32)
    for l in range(cfg["n_layers"]):
        for name in LINEARS:
            dense[f"layers.{l}.{name}"] = shared[name]
        dense[f"layers.{l}.norm1"] = np.ones(cfg["d_model"], np.float32)
        dense[f"layers.{l}.norm2"] = np.ones(cfg["d_model"], np.float32)
    return dense


def cpu_decode_baseline(dense, cfg, steps, warmup, ctx, simd_order):
    """The oracle's dense f32 decoder (the reference's CPU path: weights dequantised once at
    load, f32 GEMV per token, f32 KV) timed on the host cores for `steps` decode tokens at
    context `ctx`.  simd_order False: the strict-order scalar GEMV that defines parity; True:
    the 32-lane SIMD order a vectorised GEMM library would use."""
    import numpy as np
    from oracle import oracle as orc
    c = dict(cfg, eps=1e-5, rope_theta=10000.0)
    orc.use_all_cores()  # torchrun exports OMP_NUM_THREADS=1 to its workers
    model = orc.DenseModel(c, dense, 1, ctx + steps + warmup + 1)
    model.set_linear_order(simd_order)
    model.fill_cache(0, ctx, 1)
    tok = np.array([[17]], np.uint32)
    for i in range(warmup):
        tok = np.array([[orc.argmax(model.forward(tok, [ctx + i])[0, 0])]], np.uint32)
    t0 = time.perf_counter()
    for i in range(steps):
        tok = np.array([[orc.argmax(model.forward(tok, [ctx + warmup + i])[0, 0])]], np.uint32)
    dt = time.perf_counter() - t0
    return steps / dt, orc.num_threads(), dt


def cpu_baseline_record(cfg, steps, warmup):
    dense = cpu_dense_weights(cfg)
    strict, cores, _ = cpu_decode_baseline(dense, cfg, steps, warmup, PROMPT, False)
    simd, _, _ = cpu_decode_baseline(dense, cfg, steps, warmup, PROMPT, True)
    return {"value": round(strict, 4), "unit": "tokens/s", "cores": cores, "kind": "port",
            "order": "strict-order scalar GEMV (one running sum per output: the oracle's parity definition)",
            "value_simd_order": round(simd, 4),
            "simd_order": "the same decoder with 32-lane SIMD partial sums per output, as a vectorised GEMM "
                          "library would run it (the reference calls Candle's matmul -> gemm crate); brackets the "
                          "speed of the reference's CPU path from above",
            "sample": f"{steps} decode steps at batch 1, context {PROMPT} (cache pre-filled), all 32 layers, "
                      "dense f32 weights as the reference holds them after load"}


def cpu_ops_record():
    """Per-operator CPU legs of the microbenchmark configurations (`--cpu-ops`): the oracle's
    restatement of what the reference's CPU path does per call, on all host cores.  Weight-only
    quantised linear: the reference dequantises to dense f32 at load, so a call is a dense f32
    product (strict-order scalar sums, the oracle's parity definition) - W4A16 shapes at 1, 4 and 16
    tokens, 2048 tokens on the smallest shape only.  Decode attention: f32 KV cache, one task per
    (sequence, head), for 1 and 8 sequences of 4096 and 16384 cached tokens.  The other corners of
    the sweeps are listed as skipped: they take minutes on a CPU."""
    import numpy as np
    from oracle import oracle as orc
    orc.use_all_cores()
    rng = np.random.default_rng(2)
    ops = []

    def timed(fn, budget_s=1.5):
        fn()
        n, t0 = 0, time.perf_counter()
        while True:
            fn()
            n += 1
            dt = time.perf_counter() - t0
            if dt > budget_s or n >= 20:
                return dt / n

    for K, N in [(4096, 4096), (4096, 14336), (14336, 4096), (4096, 128256)]:
        w = rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
        for M in (1, 4, 16, 2048):
            if M == 2048 and (K, N) != (4096, 4096):
                ops.append({"op": "linear", "K": K, "N": N, "tokens": M, "skipped": "too slow on a CPU"})
                continue
            x = rng.standard_normal((M, K), dtype=np.float32)
            dt = timed(lambda: orc.linear(x, w))
            ops.append({"op": "linear", "K": K, "N": N, "tokens": M, "ms": round(dt * 1e3, 3),
                        "dense_f32_GBs": round(N * K * 4 / dt / 1e9, 1), "GFLOPs": round(2.0 * M * N * K / dt / 1e9, 1)})
        del w
    h, kvh, hd = 32, 8, 128
    for B in (1, 8, 64):
        for ctx in (4096, 16384, 32768):
            if B > 8 or ctx > 16384:
                ops.append({"op": "decode attention", "sequences": B, "context": ctx, "skipped": "too slow on a CPU"})
                continue
            q = rng.standard_normal((B, h, hd), dtype=np.float32)
            kc = rng.standard_normal((B, ctx, kvh, hd), dtype=np.float32)
            vc = rng.standard_normal((B, ctx, kvh, hd), dtype=np.float32)
            lens = np.full(B, ctx, np.int32)
            dt = timed(lambda: orc.attention_decode_gqa(q, kc, vc, lens, 1.0 / np.sqrt(hd)))
            ops.append({"op": "decode attention", "sequences": B, "context": ctx, "ms": round(dt * 1e3, 3),
                        "f32_kv_GBs": round(2.0 * B * ctx * kvh * hd * 4 / dt / 1e9, 1)})
            del kc, vc
    return {"cpu_ops": ops, "cores": orc.num_threads(), "kind": "port",
            "what": "oracle restatement of the reference's CPU path per call: dense f32 product after load-time "
                    "dequantisation, f32 KV decode attention"}


def decode_timer(torch, model, cache, pkg, B, stream, dist, world):
    """Returns (step, time_block): `step` runs one graph-replayed decode step with on-device
    sampling; `time_block(k)` times k steps with CUDA events on the launching stream, bracketed
    by a barrier and a synchronize, and returns the maximum over ranks in ms."""
    state = {"n": 0, "bufs": None}

    def start(first_tokens):
        state["bufs"] = [first_tokens.clone(), torch.empty(B, dtype=torch.int32, device="cuda")]
        state["n"] = 0

    def step():
        n = state["n"]
        model.decode_step(state["bufs"][n % 2], cache, None, state["bufs"][(n + 1) % 2])
        state["n"] = n + 1

    def time_block(k):
        stream.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(k):
            step()
        b.record(stream)
        stream.synchronize()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        return ms

    return start, step, time_block, state


def prefill_rows(torch, model, cache, prompt, B):
    logits = None
    for b in range(B):
        logits = model.forward_with_cache(prompt[b:b + 1], 0, cache, row=b, last_only=True)
    return logits


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--cpu-steps", type=int, default=12)
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline (profiling runs)")
    ap.add_argument("--skip-extra", action="store_true", help="omit the batch-32 and prefill sub-records")
    ap.add_argument("--cpu-ops", action="store_true",
                    help="time the CPU legs of the per-operator microbenchmarks (no GPU) and print them as one JSON line")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = LARGE
    B = args.batch

    if args.cpu_ops:
        if rank == 0:
            print(json.dumps(cpu_ops_record()))
        return 0

    if args.impl == "reference":
        # The reference's CPU path, restated (oracle/): no GPU, none of this repository's kernels.
        if rank != 0:
            return 0
        K = max(1, min(args.steps, 40))
        W = max(1, min(args.warmup, 3))
        dense = cpu_dense_weights(cfg)
        tok_s, cores, dt = cpu_decode_baseline(dense, cfg, K, W, PROMPT, True)
        strict, _, _ = cpu_decode_baseline(dense, cfg, min(K, 12), 1, PROMPT, False)
        sample = (f"{K} decode steps at batch 1, context {PROMPT} (cache pre-filled), all 32 layers, dense f32 "
                  "weights, 32-lane SIMD summation order (the faster of the two orders the port has)")
        line = {"impl": "reference", "metric": "INT4 decode tok/s", "value": round(tok_s, 4), "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": round(1e3 / tok_s, 3),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": "large_decode_b1_ctx512", "path": "oracle port of the reference CPU path: "
                           "weights dequantised to dense f32 at load, f32 GEMV per token, f32 KV cache"},
                "cpu_baseline": {"value": round(tok_s, 4), "unit": "tokens/s", "cores": cores, "kind": "port",
                                 "sample": sample, "value_strict_order": round(strict, 4)},
                "e2e": {"value": round(tok_s, 4), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    import torch
    torch.cuda.set_device(local_rank)
    from __graft_entry__ import import_package
    pkg = import_package()
    workload = f"large_decode_b{B}_ctx{PROMPT}"
    dist = None
    tp = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        tp = pkg.TensorParallel.from_torch_distributed()
    mc, weights = build_large(pkg, torch, cfg, tp_rank=rank, tp_world=world)
    model = pkg.AarambhModel(mc, weights, dtype=torch.bfloat16, max_tokens=max(PROMPT, B, 32), tp=tp)
    e2e_steps = max(32, args.steps // 2)
    capacity = PROMPT + max(max(args.warmup, 3) + args.steps, 3 + e2e_steps) + 16
    cache = model.empty_kv_cache_with_capacity(capacity, batch=B, dtype="int8")
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg["vocab"], (B, PROMPT), generator=gen)
    stream = torch.cuda.Stream()
    warm = max(args.warmup, 3)
    with torch.cuda.stream(stream):
        logits = prefill_rows(torch, model, cache, prompt, B)
        first = pkg.dispatch.argmax(logits.view(1, -1)).repeat(B)
        start, step, time_block, state = decode_timer(torch, model, cache, pkg, B, stream, dist, world)
        start(first)
        clocks = ClockSampler(local_rank)
        for _ in range(warm):
            step()
        # BLOCKS blocks of --steps steps; every block starts from the prompt's context again
        block_ms = []
        with clocks:
            for _ in range(BLOCKS):
                stream.synchronize()
                for b in range(B):
                    cache.truncate(PROMPT, b)
                block_ms.append(time_block(args.steps))
        block_ms.sort()
        dev_ms = block_ms[len(block_ms) // 2]
        ms_per_step = dev_ms / args.steps

        # end to end through the host API: token ids cross PCIe both ways every step
        host_ids = [torch.empty(B, dtype=torch.int32).pin_memory() for _ in range(2)]
        host_ids[0].copy_(state["bufs"][state["n"] % 2].cpu())
        for b in range(B):
            cache.truncate(PROMPT, b)
        host_n = [0]

        def host_step():
            # one call of the host API: ids cross to the device, the step replays, the greedy tokens
            # cross back, the call returns when they have arrived; they are the next step's ids
            i = host_n[0] & 1
            model.decode_step_host(host_ids[i], cache, host_ids[i ^ 1])
            host_n[0] += 1

        for _ in range(3):
            host_step()
        with clocks:
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                host_step()
            e2e_s = (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([e2e_s], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t[0])

    local_cfg = dict(cfg, n_heads=cfg["n_heads"] // world, n_kv_heads=cfg["n_kv_heads"] // world,
                     ffn_hidden=cfg["ffn_hidden"] // world)
    gemv_s, gemv_launches, gemv_bytes = time_gemv_only(pkg, torch, weights, local_cfg, max(8, args.steps // 4), stream)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = gemv_bytes / gemv_s / 1e9
    ctx_mid = PROMPT + args.steps // 2
    # per GPU: a rank reads its 1/world share of the layer weights, head and KV
    step_bytes = (step_weight_bytes(cfg) + B * ctx_mid * kv_bytes_per_token(cfg)) // world
    # embedding, per layer {norm+qkv, attention, o, norm+gate|up+SwiGLU, down} (tensor parallel: the same five,
    # the partial sums travel in the projections' epilogues and the next GEMV's prologue), norm+head, argmax,
    # commit; NCCL's all-gather of the logits shards is not counted
    launches_per_step = (1 + cfg["n_layers"] * 5 + 3) if B == 1 else (1 + cfg["n_layers"] * 7 + 4)

    line = {
        "metric": "INT4 decode tok/s", "value": round(B * 1e3 / ms_per_step, 2), "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": warm,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 activations, f32 accumulate, u4 weights, i8 KV", "data": "synthetic",
        "config": {"workload": workload, "batch": B, "prompt": PROMPT, "weights": "W4A16 g128 (bf16 scale, u4 zero)",
                   "kv": "int8 per token per head", "parallelism": f"tp{world}",
                   "l2": "weights (3.7 GB per step) exceed the 126 MB L2"},
        "blocks": {"n": BLOCKS, "steps_each": args.steps, "reported": "median",
                   "ms_per_step_min": round(block_ms[0] / args.steps, 4),
                   "ms_per_step_max": round(block_ms[-1] / args.steps, 4)},
        "step_bytes": step_bytes,
        "step_hbm_frac": round(step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak, 4),
        "roofline": {"bound": "hbm", "kernel": "gemv_w4a16_m1_kernel (gemv_w4a16_warp_kernel where K > 8192)", "achieved": round(achieved, 1),
                     "peak": hbm_peak, "unit": "GB/s", "frac": round(achieved / hbm_peak, 4),
                     "traffic": round(gemv_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE),
                     "traffic_source": "ncu dram read+write of this kernel on one token, divided by its algorithmic "
                                       "bytes (ratio 1.013), times the bytes an average launch of the step streams",
                     "peak_source": "measured" if peaks else "fallback",
                     "launches_per_step": gemv_launches, "bytes_per_launch": round(gemv_bytes)},
        "e2e": {"value": round(B / e2e_s, 2), "unit": "tokens/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 4 * B},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
    }

    if world > 1:
        line["tp_check"] = tp_check(pkg, torch, dist, cfg, model, mc, rank, world, stream)
    if not args.skip_extra and world == 1 and B == 1:
        del cache
        line["prefill"] = prefill_record(pkg, torch, cfg, model, stream)
        line["batch32"] = batch32_record(pkg, torch, cfg, model, stream, hbm_peak, min(args.steps, 64))
    line["device_status"] = pkg.device_status()
    if rank == 0 and world == 1 and not args.skip_cpu:
        del model, weights
        torch.cuda.empty_cache()
        line["cpu_baseline"] = cpu_baseline_record(cfg, args.cpu_steps, 2)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def prefill_record(pkg, torch, cfg, model, stream):
    """The 512-token prompt of the decode workload through the prefill path (tcgen05 GEMMs, causal
    attention), timed on its own: median of five passes over a fresh cache row."""
    cache = model.empty_kv_cache_with_capacity(PROMPT + 8, batch=1, dtype="int8")
    prompt = torch.randint(0, cfg["vocab"], (1, PROMPT), generator=torch.Generator().manual_seed(2))
    times = []
    with torch.cuda.stream(stream):
        for i in range(7):
            cache.truncate(0, 0)
            stream.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            model.forward_with_cache(prompt, 0, cache, row=0, last_only=True)
            b.record(stream)
            stream.synchronize()
            if i >= 2:
                times.append(a.elapsed_time(b))
    times.sort()
    ms = times[len(times) // 2]
    params = sum(n * k for n, k in linear_shapes(cfg).values()) * cfg["n_layers"]
    flops = 2.0 * PROMPT * params + 2.0 * cfg["vocab"] * cfg["d_model"]          # linears (+ the head on the last token)
    flops += cfg["n_layers"] * 2.0 * 2.0 * cfg["n_heads"] * cfg["head_dim"] * PROMPT * (PROMPT + 1) / 2   # causal QK^T and PV
    return {"tokens": PROMPT, "ms": round(ms, 3), "tok_s": round(PROMPT * 1e3 / ms, 1), "tflops": round(flops / ms / 1e9, 1),
            "note": "one sequence, INT8 KV written as it goes; timed apart from the decode steps"}


def batch32_record(pkg, torch, cfg, model, stream, hbm_peak, steps):
    """The benchmark spec's second decode workload: 32 sequences of a 512-token prompt each, one
    graph-replayed step for all of them (median of three blocks)."""
    B = 32
    cache = model.empty_kv_cache_with_capacity(PROMPT + steps + 24, batch=B, dtype="int8")
    prompt = torch.randint(0, cfg["vocab"], (B, PROMPT), generator=torch.Generator().manual_seed(3))
    with torch.cuda.stream(stream):
        logits = prefill_rows(torch, model, cache, prompt, B)
        first = pkg.dispatch.argmax(logits.view(1, -1)).repeat(B)
        start, step, time_block, _ = decode_timer(torch, model, cache, pkg, B, stream, None, 1)
        start(first)
        for _ in range(4):
            step()
        blocks = []
        for _ in range(3):
            stream.synchronize()
            for b in range(B):
                cache.truncate(PROMPT, b)
            blocks.append(time_block(steps) / steps)
    blocks.sort()
    ms = blocks[1]
    byt = step_weight_bytes(cfg) + B * (PROMPT + steps // 2) * kv_bytes_per_token(cfg)
    return {"batch": B, "steps": steps, "ms_per_step": round(ms, 4), "tok_s": round(B * 1e3 / ms, 1),
            "step_bytes": byt, "step_hbm_frac": round(byt / (ms * 1e-3) / 1e9 / hbm_peak, 4)}


def tp_check(pkg, torch, dist, cfg, model, mc, rank, world, stream):
    """Correctness evidence for the sharded run, at the benchmark's own shapes.
    (1) The first two blocks of the model (same seeded weights, sharded exactly as the full
    model) decode 32 greedy tokens from a 48-token prompt on all ranks and alone on rank 0:
    logits must agree within 1e-2 relative (`ok`) - two blocks keep the comparison free of the
    compounding bf16 rounding noise of a deep random-weight model.  Tokens are compared too;
    where the streams part, the margin between the two candidates (single-GPU logits, relative
    to the largest logit) shows whether it was a near tie of a random-weight model.
    (2) The full 32-block model does the same; its equal prefix and logit error are reported
    for information (after 32 random-weight blocks in bf16 a different f32 summation order is
    enough to flip near-tied tokens; the error floor of that depth is reported beside it: the
    single-GPU model against itself through its other kernel path, prefill GEMMs against
    decode GEMVs)."""
    steps, plen = 32, 48
    prompt = torch.randint(0, cfg["vocab"], (1, plen), generator=torch.Generator().manual_seed(7))

    def run(m):
        cache = m.empty_kv_cache_with_capacity(plen + steps + 4, batch=1, dtype="int8")
        toks, lgs = [], []
        with torch.cuda.stream(stream):
            lg = m.forward_with_cache(prompt, 0, cache, row=0, last_only=True).view(1, -1)
            for i in range(steps):
                lgs.append(lg.float().clone())
                t = pkg.dispatch.argmax(lg)
                toks.append(int(t[0]))
                lg = m.forward_decode_batch(t.view(1, 1).cpu(), [plen + i], cache).view(1, -1)
            stream.synchronize()
        return toks, torch.cat(lgs)

    def compare(a, b):
        (ta, la), (tb, lb) = a, b
        n_same = 0
        for x, y in zip(ta, tb):
            if x != y:
                break
            n_same += 1
        upto = max(1, min(n_same + 1, steps))   # after a first difference the inputs differ
        err = float((la[:upto] - lb[:upto]).abs().amax() / lb[:upto].abs().amax())
        margin = None
        if n_same < steps:   # the two tokens chosen at the first difference, on the reference logits
            row = lb[n_same]
            margin = float((row[tb[n_same]] - row[ta[n_same]]).abs() / row.abs().amax())
        return n_same, err, margin

    tp = model.tp
    small = dict(cfg, n_layers=2)
    mc2, w2 = build_large(pkg, torch, small, tp_rank=rank, tp_world=world)
    sharded2 = pkg.AarambhModel(mc2, w2, dtype=torch.bfloat16, max_tokens=64, tp=tp)
    got2 = run(sharded2)
    got_full = run(model)
    out = None
    dist.barrier()
    if rank == 0:
        mc1, w1 = build_large(pkg, torch, small)
        single2 = pkg.AarambhModel(mc1, w1, dtype=torch.bfloat16, max_tokens=64)
        n2, e2, m2 = compare(got2, run(single2))
        del single2, w1
        mcf, wf = build_large(pkg, torch, cfg)
        single = pkg.AarambhModel(mcf, wf, dtype=torch.bfloat16, max_tokens=128)
        ref_full = run(single)
        nf, ef, mf = compare(got_full, ref_full)
        # the error floor of the depth: the same tokens through the prefill path in one pass
        seq = torch.cat([prompt[0], torch.tensor(ref_full[0][:-1])]).view(1, -1)
        cache = single.empty_kv_cache_with_capacity(plen + steps + 4, batch=1, dtype="int8")
        with torch.cuda.stream(stream):
            lg_all = single.forward_with_cache(seq, 0, cache, row=0)[0, plen - 1:].float()
            stream.synchronize()
        floor = float((lg_all - ref_full[1]).abs().amax() / ref_full[1].abs().amax())
        out = {"blocks": 2, "tokens": steps, "tokens_equal": n2 == steps, "equal_prefix": n2,
               "max_rel_logit_err": round(e2, 5), "tolerance": 1e-2, "ok": bool(e2 < 1e-2),
               "margin_at_first_difference": None if m2 is None else round(m2, 5),
               "full_model": {"blocks": cfg["n_layers"], "equal_prefix": nf, "max_rel_logit_err": round(ef, 5),
                              "margin_at_first_difference": None if mf is None else round(mf, 5),
                              "single_gpu_error_floor": round(floor, 5)}}
        del single, wf
        torch.cuda.empty_cache()
    dist.barrier()
    return out


if __name__ == "__main__":
    sys.exit(main())
