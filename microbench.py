#!/usr/bin/env python
"""Micro-benchmarks of the three hot kernels on synthetic inputs of the
benchmark specification's shapes.  Timing is with CUDA events on the launching
stream after warm-up; weights / caches larger than L2 are cycled so every timed
launch reads from HBM.

    python microbench.py gemv      [--m 1,4,16]      W4A16 dequant-GEMV (HBM GB/s)
    python microbench.py gemm      [--m 512,2048]    W4A16 tcgen05 GEMM (TFLOP/s)
    python microbench.py attention [--cases 8x16384] INT8-KV flash-decode (HBM GB/s)
    python microbench.py prefill_attention [--cases 1x512] causal attention of a prompt over the INT8 cache
    python microbench.py gemv|gemm --fmt int8             the same two for INT8 per-channel weights
    python microbench.py gemv --fmt q4km                  the GEMV over Q4_K_M-style blocks
    python microbench.py step      [--layers 2] [--ctx 512] one-token decoder step of a short
                                                   Large-shaped stack (a few hundred MB on the device: the
                                                   case to capture the step's kernels under a profiler)

``--profile`` runs three launches of the first case only (for ncu captures).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import import_package  # noqa: E402

SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096), (4096, 128256)]   # (K, N)


def peak_hbm() -> float:
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6650.0


def peak_tflops() -> float:
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except (OSError, KeyError, ValueError):
        return 1590.0


def random_w4a16(pkg, N, K, seed):
    """Uniform random packed ints, bf16 scales in [0.005, 0.02], zero points 0..15."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    qw = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, device="cuda", generator=g)
    sc = (torch.rand(N, K // 128, device="cuda", generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    qz = torch.randint(-2**31, 2**31 - 1, (N, (K // 128 + 7) // 8), dtype=torch.int32, device="cuda", generator=g)
    return pkg.QuantLinear.from_w4a16_gptq(qw, sc.view(torch.int16), qz, N, K, 128)


def w4_bytes(N, K):
    return K * N // 2 + (K // 128) * N * 2 + (K // 128) * N // 2


def time_graph(fn, reps, stream):
    """Captures `fn` in a CUDA graph and returns seconds per replay (launch overhead of the host excluded)."""
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            g.replay()
        b.record(stream)
        stream.synchronize()
    return a.elapsed_time(b) * 1e-3 / reps


def w4a16_kernel_name(M, N):
    """The kernel the library's dispatch takes for M tokens on a W4A16 weight of N rows (chunks of 32 tokens)."""
    if M == 1:
        return "gemv_w4a16_m1_kernel"
    if M <= 8:
        return "gemv_w4a16_warp_kernel"
    if M <= 24 or (M <= 32 and N >= 24576):
        return "gemv_w4a16_strip_kernel"
    return "gemv_w4a16_tc_kernel" if M <= 32 else "gemv_w4a16_tc_kernel / strip / warp per 32-token chunk"


def bench_gemv(pkg, args):
    stream = torch.cuda.Stream()
    for K, N in SHAPES:
        copies = 1 if args.profile else max(2, math.ceil(400e6 / w4_bytes(N, K)))
        lins = [random_w4a16(pkg, N, K, 2 + i) for i in range(copies)]
        for M in args.m:
            x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            if args.profile:
                for _ in range(3):
                    lins[0](x)
                torch.cuda.synchronize()
                print("profiled case", K, N, M)
                return
            t = time_graph(lambda: [lin(x) for lin in lins], 5, stream) / copies
            byt = w4_bytes(N, K) + 2 * M * (K + N)
            print(json.dumps({"kernel": w4a16_kernel_name(M, N), "K": K, "N": N, "M": M, "us": round(t * 1e6, 2),
                              "GBs": round(byt / t / 1e9, 1), "frac_of_measured_hbm": round(byt / t / 1e9 / peak_hbm(), 3)}),
                  flush=True)
        del lins


def random_int8(pkg, N, K, seed):
    """N(0, 0.02) weights quantised to INT8 with one absmax scale per output channel."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn((N, K), generator=g, device="cuda") * 0.02
    return pkg.QuantLinear.quantise(w, "int8_channel")


def random_q4km(pkg, N, K, seed):
    """N(0, 0.02) weights quantised to Q4_K_M-style blocks of 256."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn((N, K), generator=g, device="cuda") * 0.02
    return pkg.QuantLinear.quantise(w, "q4_k_m")


def bench_gemv_int8(pkg, args):
    stream = torch.cuda.Stream()
    q4 = args.fmt == "q4km"
    for K, N in SHAPES:
        if q4 and K % 256:
            continue
        wbytes = K * N // 2 + 4 * N * (K // 256) if q4 else K * N + 4 * N
        copies = 1 if args.profile else max(2, math.ceil(400e6 / wbytes))
        lins = [(random_q4km if q4 else random_int8)(pkg, N, K, 2 + i) for i in range(copies)]
        for M in args.m:
            x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            if args.profile:
                for _ in range(3):
                    lins[0](x)
                torch.cuda.synchronize()
                print("profiled case", K, N, M)
                return
            t = time_graph(lambda: [lin(x) for lin in lins], 5, stream) / copies
            byt = wbytes + 2 * M * (K + N)
            name = ("gemv_q4km_stream_kernel" if M <= 8 else "gemv_generic_kernel") if q4 else \
                   ("gemv_i8_stream_kernel" if M <= 8 else "gemm_i8_tc_kernel")
            print(json.dumps({"kernel": name, "K": K, "N": N, "M": M,
                              "us": round(t * 1e6, 2), "GBs": round(byt / t / 1e9, 1),
                              "frac_of_measured_hbm": round(byt / t / 1e9 / peak_hbm(), 3)}), flush=True)
        del lins


def bench_gemm(pkg, args):
    int8 = getattr(args, "fmt", "w4a16") == "int8"
    for K, N in (SHAPES if args.shape else SHAPES[:3]):
        lin = random_int8(pkg, N, K, 2) if int8 else random_w4a16(pkg, N, K, 2)
        dense = lin.dequantise(torch.bfloat16)
        for M in args.m:
            x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            for _ in range(3):
                y = lin(x)
            torch.cuda.synchronize()
            if args.profile:
                print("profiled case", K, N, M)
                return
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                y = lin(x)
            b.record()
            torch.cuda.synchronize()
            t = a.elapsed_time(b) * 1e-3 / 10
            ref = x @ dense.T
            err = ((y.float() - ref.float()).abs().max() / ref.float().abs().max()).item()
            fl = 2.0 * M * K * N
            print(json.dumps({"kernel": "gemm_i8_tc_kernel" if int8 else "gemm_w4a16_tc_kernel", "K": K, "N": N, "M": M, "us": round(t * 1e6, 1),
                              "TFLOPs": round(fl / t / 1e12, 1), "frac_of_measured_bf16": round(fl / t / 1e12 / peak_tflops(), 3),
                              "rel_err_vs_dense_bf16": err}), flush=True)


def bench_attention(pkg, args):
    h, kvh, hd = 32, 8, 128
    for B, ctx in args.cases:
        cache = pkg.KVCache(ctx, kvh, hd, h, batch=B, dtype="int8")
        g = torch.Generator(device="cuda").manual_seed(3)
        for b in range(B):
            for s0 in range(0, ctx, 4096):
                n = min(4096, ctx - s0)
                k = torch.randn((1, n, kvh, hd), generator=g, device="cuda", dtype=torch.bfloat16)
                cache.update(k, k, row0=b)
        q = torch.randn((B, h, hd), generator=g, device="cuda").to(torch.bfloat16)
        scale = 1 / math.sqrt(hd)
        for _ in range(3):
            pkg.dispatch.attention_decode(cache, q, scale)
        torch.cuda.synchronize()
        if args.profile:
            print("profiled case", B, ctx)
            return
        reps = 20 if B * ctx < 1e6 else 8
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            pkg.dispatch.attention_decode(cache, q, scale)
        b_.record()
        torch.cuda.synchronize()
        t = a.elapsed_time(b_) * 1e-3 / reps
        byt = B * (ctx * (2 * kvh * hd + 2 * kvh * 4) + 2 * h * hd * 2)
        print(json.dumps({"kernel": "attn_decode_mma_kernel", "B": B, "ctx": ctx, "us": round(t * 1e6, 1),
                          "GBs": round(byt / t / 1e9, 1), "frac_of_measured_hbm": round(byt / t / 1e9 / peak_hbm(), 3)}),
              flush=True)
        del cache


def bench_prefill_attention(pkg, args):
    """Causal attention of S new queries over an INT8 cache that ends with their own keys (32 / 8 heads of
    128): the prefill kernel on its own, per layer of the Large config."""
    h, kvh, hd = 32, 8, 128
    for B, S in args.cases:
        cache = pkg.KVCache(S, kvh, hd, h, batch=B, dtype="int8")
        g = torch.Generator(device="cuda").manual_seed(3)
        for b in range(B):
            k = torch.randn((1, S, kvh, hd), generator=g, device="cuda", dtype=torch.bfloat16)
            cache.update(k, k, row0=b)
        q = torch.randn((B, S, h, hd), generator=g, device="cuda").to(torch.bfloat16)
        scale = 1 / math.sqrt(hd)
        for _ in range(3):
            pkg.dispatch.attention_cached(cache, q, scale)
        torch.cuda.synchronize()
        if args.profile:
            print("profiled case", B, S)
            return
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            pkg.dispatch.attention_cached(cache, q, scale)
        b_.record()
        torch.cuda.synchronize()
        t = a.elapsed_time(b_) * 1e-3 / 10
        fl = B * 2.0 * 2.0 * h * hd * S * (S + 1) / 2
        print(json.dumps({"kernel": "attn_prefill_mma_kernel", "B": B, "S": S, "us": round(t * 1e6, 1),
                          "TFLOPs": round(fl / t / 1e12, 1)}), flush=True)


def bench_step(pkg, args):
    """Decode steps of an n-layer stack with the Large block shapes (d 4096, 32 / 8 heads of 128, hidden 14336,
    vocab 32000; W4A16 g128, INT8 KV, bf16), context `ctx`.  Prints the step time; with --profile runs 4 steps."""
    L, d, h, kvh, hd, ffn, vocab = args.layers, 4096, 32, 8, 128, 14336, 32000
    gen = torch.Generator(device="cuda").manual_seed(0)
    weights = {}

    def make(name, n, k):
        w = torch.randn((n, k), generator=gen, device="cuda", dtype=torch.float32) * 0.02
        weights[name] = pkg.QuantLinear.quantise(w, "w4a16", 128)

    for l in range(L):
        for nm, (n, k) in {"wq": (h * hd, d), "wk": (kvh * hd, d), "wv": (kvh * hd, d), "wo": (d, h * hd),
                           "w_gate": (ffn, d), "w_up": (ffn, d), "w_down": (d, ffn)}.items():
            make(f"layers.{l}.{nm}", n, k)
        weights[f"layers.{l}.norm1"] = torch.ones(d, device="cuda")
        weights[f"layers.{l}.norm2"] = torch.ones(d, device="cuda")
    weights["final_norm"] = torch.ones(d, device="cuda")
    make("embedding", vocab, d)
    make("lm_head", vocab, d)
    cfg = pkg.ModelConfig(L, d, h, kvh, hd, ffn, vocab, args.ctx + 64, 1e-5, 10000.0, False)
    B = args.batch
    model = pkg.AarambhModel(cfg, weights, dtype=torch.bfloat16, max_tokens=max(args.ctx, B))
    cache = model.empty_kv_cache_with_capacity(args.ctx + 48, batch=B, dtype="int8")
    prompt = torch.randint(0, vocab, (B, args.ctx), generator=torch.Generator().manual_seed(1))
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        first = [model.forward_with_cache(prompt[b:b + 1], 0, cache, row=b, last_only=True).view(1, -1) for b in range(B)]
        bufs = [pkg.dispatch.argmax(torch.cat(first)).clone(), torch.empty(B, dtype=torch.int32, device="cuda")]
        n = 0

        def step():
            nonlocal n
            model.decode_step(bufs[n % 2], cache, None, bufs[(n + 1) % 2])
            n += 1

        for _ in range(4):
            step()
        stream.synchronize()
        if args.profile:
            print("profiled case", L, args.ctx, B)
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(32):
            step()
        b.record(stream)
        stream.synchronize()
    print(json.dumps({"workload": f"decode step, {L} Large-shaped layers, context {args.ctx}, batch {B}",
                      "us_per_step": round(a.elapsed_time(b) * 1e3 / 32, 2)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv", "gemm", "attention", "prefill_attention", "step"])
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--batch", type=int, default=1, help="step: sequences decoded together")
    ap.add_argument("--m", default=None)
    ap.add_argument("--cases", default=None)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--shape", default=None, help="K,N: restrict gemv / gemm to one weight shape")
    ap.add_argument("--fmt", default="w4a16", choices=["w4a16", "int8", "q4km"], help="weight format of gemv (gemm: w4a16, int8)")
    args = ap.parse_args()
    pkg = import_package()
    torch.cuda.set_device(0)
    if args.shape:
        k, n = (int(v) for v in args.shape.split(","))
        SHAPES[:] = [(k, n)]
    if args.what == "gemv":
        args.m = [int(v) for v in (args.m or "1,4,16").split(",")]
        (bench_gemv_int8 if args.fmt in ("int8", "q4km") else bench_gemv)(pkg, args)
    elif args.what == "gemm":
        args.m = [int(v) for v in (args.m or "512,2048,8192").split(",")]
        bench_gemm(pkg, args)
    elif args.what == "step":
        bench_step(pkg, args)
    elif args.what == "prefill_attention":
        args.cases = [tuple(int(v) for v in c.split("x")) for c in (args.cases or "1x512,1x2048,4x512").split(",")]
        bench_prefill_attention(pkg, args)
    else:
        default = "1x4096,1x16384,1x32768,8x4096,8x16384,8x32768,64x4096,64x16384,64x32768"
        args.cases = [tuple(int(v) for v in c.split("x")) for c in (args.cases or default).split(",")]
        bench_attention(pkg, args)
    print(json.dumps({"device_status": pkg.device_status()}))


if __name__ == "__main__":
    main()
