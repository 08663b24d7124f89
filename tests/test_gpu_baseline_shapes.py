"""Parity on the shapes the benchmark configurations name, not scaled-down stand-ins:
which kernel serves a call depends on K, N, the token count and the context length,
so every shape the measurements quote is compared with the oracle here.

 * W4A16 g128 linears (K x N): 4096 x 4096, 4096 x 14336, 14336 x 4096, 4096 x 128256
   at 1, 4, 16, 32 tokens and 2048 tokens (sampled rows), GPTQ order; AWQ order and
   INT8 per-channel at 512 / 2048 / 8192 tokens (sampled rows)
   -- QatLinear::forward, crates/aarambh-studio-quant/src/qat.rs:315-348.
 * INT8-KV decode attention, 32 / 8 heads, head_dim 128, context 16384 and 32768,
   8 and 64 sequences -- GroupedQueryAttention::forward_decode_batch,
   crates/aarambh-studio-nn/src/attention.rs:228-288.
 * A 2-layer stack of the Large-class block (d 4096, 32 / 8 heads, hidden 14336,
   vocab 32000), INT8 KV, graph-replayed decode steps at 1 and 32 rows.

Tolerances: 1e-2 relative (max |diff| / max |ref|) for linear and attention outputs and
2e-2 for the logits of one block.  The logits of the two-block stack are held to 5e-2:
they carry the error of the formats themselves (a bf16 residual stream of 4096 values
rounded after every projection, and an INT8 cache) against an oracle that keeps f32
activations and an f32 cache; measured 2.1e-2 to 2.7e-2.
"""
import math

import numpy as np
import pytest
import torch

from helpers import pkg, rel_err
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-2
STACK_TOL = 5e-2
SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096), (4096, 128256)]   # K, N


def _w4a16(K, N, awq=False, seed=2):
    """Uniform packed ints, bf16 scales in [0.005, 0.02], u4 zero points (packed words)."""
    rng = np.random.default_rng(seed)
    G = K // 128
    qw = rng.integers(0, 2**32, (N, K // 8), dtype=np.uint32)
    scales = orc.bf16_bits(rng.uniform(0.005, 0.02, (N, G)).astype(np.float32))
    qz = rng.integers(0, 2**32, (N, -(-G // 8)), dtype=np.uint32)
    make = pkg().QuantLinear.from_w4a16_awq if awq else pkg().QuantLinear.from_w4a16_gptq
    lin = make(qw, scales, qz, N, K, 128)
    dense = orc.dequant_w4a16(qw, scales, qz, N, K, 128, awq_order=awq)
    return lin, dense, rng


@pytest.fixture(scope="module", params=SHAPES, ids=lambda s: f"K{s[0]}xN{s[1]}")
def gptq(request):
    K, N = request.param
    lin, dense, rng = _w4a16(K, N)
    got = lin.dequantise(torch.float32).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), dense.view(np.uint32)), "dequantised weights differ"
    return K, N, lin, dense, rng


@pytest.mark.parametrize("M", [1, 4, 16, 32])
def test_w4a16_gptq_decode_tokens(gptq, M):
    K, N, lin, dense, _ = gptq
    rng = np.random.default_rng(100 + M)
    x = orc.round_bf16(rng.standard_normal((M, K)).astype(np.float32))
    got = lin(torch.from_numpy(x).cuda().to(torch.bfloat16)).float().cpu().numpy()
    again = lin(torch.from_numpy(x).cuda().to(torch.bfloat16)).float().cpu().numpy()
    assert pkg().device_status() == 0
    assert rel_err(got, orc.linear(x, dense)) < TOL
    assert np.array_equal(got, again)


def _sampled(lin, dense, K, M, seed, rows=3):
    """M tokens through the GPU path; `rows` of them through the oracle."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    y = lin(x)
    assert pkg().device_status() == 0
    pick = sorted({0, min(M - 1, M // 2 + 1), M - 1})[:rows]
    xs = x[pick].float().cpu().numpy()
    ref = orc.linear(xs, dense)
    return rel_err(y[pick].float().cpu().numpy(), ref)


def test_w4a16_gptq_prefill_2048_tokens(gptq):
    K, N, lin, dense, _ = gptq
    assert _sampled(lin, dense, K, 2048, 7) < TOL


@pytest.mark.parametrize("K,N,Ms", [(4096, 4096, [512, 2048, 8192]), (4096, 14336, [512, 2048, 8192]),
                                    (14336, 4096, [512, 2048, 8192]), (4096, 128256, [512])])
def test_w4a16_awq_order_prefill(K, N, Ms):
    lin, dense, _ = _w4a16(K, N, awq=True, seed=3)
    got = lin.dequantise(torch.float32).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), dense.view(np.uint32))
    for M in Ms:
        assert _sampled(lin, dense, K, M, 11 + M) < TOL, M
    # the same weight at decode token counts (one token, the tensor-memory decode GEMM)
    for M in (1, 24):
        assert _sampled(lin, dense, K, M, 5 + M) < TOL, M


@pytest.mark.parametrize("K,N,Ms", [(4096, 4096, [1, 4, 16, 512, 2048, 8192]), (4096, 14336, [1, 16, 512, 2048, 8192]),
                                    (14336, 4096, [1, 16, 512, 2048, 8192]), (4096, 128256, [1, 512])])
def test_int8_per_channel_decode_and_prefill(K, N, Ms):
    """INT8 symmetric per-output-channel absmax (qat.rs:140-169): codes and scales from the
    device quantiser (bit-exact with the oracle, checked on a slice), then the linear."""
    g = torch.Generator(device="cuda").manual_seed(4)
    w = torch.randn((N, K), generator=g, device="cuda") * 0.02
    lin = pkg().QuantLinear.quantise(w, "int8_channel")
    dense = lin.dequantise().cpu().numpy()
    head = w[:64].cpu().numpy()
    codes, scales = orc.quantise_absmax_i8_rows(head)
    assert np.array_equal(dense[:64], orc.dequantise_i8_rows(codes, scales))
    del w
    for M in Ms:
        assert _sampled(lin, dense, K, M, 13 + M) < TOL, M


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 14336), (1024, 400)])
def test_q4km_blocks_decode_gemv(K, N):
    """Q4_K_M-style blocks (gguf_quant.rs:39-49), bf16 activations, 1..8 tokens: the streaming GEMV over
    the code and parameter planes; the dequantised weight is bit-exact with the oracle on a slice."""
    g = torch.Generator(device="cuda").manual_seed(5)
    w = torch.randn((N, K), generator=g, device="cuda") * 0.02
    lin = pkg().QuantLinear.quantise(w, "q4_k_m")
    dense = lin.dequantise().cpu().numpy()
    head = w[:16].cpu().numpy()
    assert np.array_equal(dense[:16], orc.decode_q4km_tensor(orc.encode_q4km_tensor(head), (16, K)))
    del w
    for M in (1, 3, 8):
        assert _sampled(lin, dense, K, M, 21 + M) < TOL, M
    assert pkg().device_status() == 0


# ---------------------------------------------------------------------------
# INT8-KV decode attention at long contexts
# ---------------------------------------------------------------------------
def _fill_rows(cache, lens, kvh, hd, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    for b, n in enumerate(lens):
        k = torch.randn((1, n, kvh, hd), generator=g, device="cuda")
        v = torch.randn((1, n, kvh, hd), generator=g, device="cuda")
        cache.update(k, v, row0=b)


@pytest.mark.parametrize("B", [8, 64])
@pytest.mark.parametrize("ctx", [16384, 32768])
def test_int8_kv_decode_attention_long_context(B, ctx):
    h, kvh, hd = 32, 8, 128
    p = pkg()
    # ragged: a full row, rows a little shorter, and one short row (its later splits are empty)
    lens = [ctx - (37 * b) % 900 for b in range(B)]
    lens[B // 2] = 200
    cache = p.KVCache(ctx, kvh, hd, h, batch=B, dtype="int8")
    _fill_rows(cache, lens, kvh, hd, 3)
    g = torch.Generator(device="cuda").manual_seed(9)
    q = torch.randn((B, h, hd), generator=g, device="cuda").to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    got = p.dispatch.attention_decode(cache, q, scale).float().cpu().numpy()
    assert p.device_status() == 0
    for b in (0, B // 2, B - 1):
        k, v = [t.cpu().numpy()[None] for t in cache.read(b)]
        ref = orc.attention_decode_gqa(q[b:b + 1].float().cpu().numpy(), k, v, np.array([lens[b]], np.int32), scale)
        assert rel_err(got[b], ref[0]) < TOL, (B, ctx, b)


# ---------------------------------------------------------------------------
# Large-class block stack
# ---------------------------------------------------------------------------
LARGE2 = dict(n_layers=2, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn_hidden=14336, vocab=32000,
              max_seq=1024, eps=1e-5, rope_theta=10000.0)


@pytest.fixture(scope="module")
def large2():
    """Two Large-class blocks: N(0, 0.02) weights (seed 0), W4A16 g128 on the GPU, the
    dequantised weights in the oracle's dense f32 model."""
    p = pkg()
    c = LARGE2
    g = torch.Generator(device="cuda").manual_seed(0)
    qd, kd = c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]
    shapes = {"wq": (qd, c["d_model"]), "wk": (kd, c["d_model"]), "wv": (kd, c["d_model"]),
              "wo": (c["d_model"], qd), "w_gate": (c["ffn_hidden"], c["d_model"]),
              "w_up": (c["ffn_hidden"], c["d_model"]), "w_down": (c["d_model"], c["ffn_hidden"])}
    packed, deq = {}, {}

    def add(name, shape):
        w = torch.randn(shape, generator=g, device="cuda") * 0.02
        packed[name] = p.QuantLinear.quantise(w, "w4a16", 128)
        deq[name] = packed[name].dequantise().cpu().numpy()

    add("embedding", (c["vocab"], c["d_model"]))
    add("lm_head", (c["vocab"], c["d_model"]))
    for l in range(c["n_layers"]):
        for name, shp in shapes.items():
            add(f"layers.{l}.{name}", shp)
        for n in ("norm1", "norm2"):
            packed[f"layers.{l}.{n}"] = torch.ones(c["d_model"], device="cuda")
            deq[f"layers.{l}.{n}"] = np.ones(c["d_model"], np.float32)
    packed["final_norm"] = torch.ones(c["d_model"], device="cuda")
    deq["final_norm"] = np.ones(c["d_model"], np.float32)
    cfg = p.ModelConfig(c["n_layers"], c["d_model"], c["n_heads"], c["n_kv_heads"], c["head_dim"],
                        c["ffn_hidden"], c["vocab"], c["max_seq"], c["eps"], c["rope_theta"], False)
    gpu = p.AarambhModel(cfg, packed, dtype=torch.bfloat16, max_tokens=512)
    return gpu, packed, deq


def _decode_steps(gpu, cache, tokens_per_step, B):
    """Graph-replayed steps on a side stream; returns the logits of every step."""
    side = torch.cuda.Stream()
    logits = torch.empty((B, LARGE2["vocab"]), dtype=torch.bfloat16, device="cuda")
    tok = torch.empty(B, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    out = []
    for ids in tokens_per_step:
        with torch.cuda.stream(side):
            tok.copy_(torch.tensor(ids, dtype=torch.int32))
            gpu.decode_step(tok, cache, logits, None)
            side.synchronize()
        out.append(logits.float().cpu().numpy().copy())
    return out


def test_large_block_stack_decode_one_row_context_512(large2):
    gpu, _, deq = large2
    P, steps = 510, 4          # the steps cross 512 cached tokens, where the step graph is captured anew
    ids = np.random.default_rng(1).integers(0, LARGE2["vocab"], P + steps)
    cpu = orc.DenseModel(LARGE2, deq, 1, P + steps + 2)
    ref = cpu.forward(ids[None], [0])[0]
    cache = gpu.empty_kv_cache_with_capacity(768, dtype="int8")
    lg = gpu.forward_with_cache(ids[None, :P], 0, cache, last_only=True).float().cpu().numpy()
    assert rel_err(lg[0, 0], ref[P - 1]) < STACK_TOL
    got = _decode_steps(gpu, cache, [[int(ids[P + s])] for s in range(steps)], 1)
    assert pkg().device_status() == 0
    for s in range(steps):
        assert rel_err(got[s][0], ref[P + s]) < STACK_TOL, s


def test_large_block_stack_decode_32_rows(large2):
    gpu, _, deq = large2
    B, steps = 32, 2
    lens = [12 + (5 * b) % 9 for b in range(B)]
    lens[3] = 300              # one long row among short ones
    rng = np.random.default_rng(5)
    seqs = [rng.integers(0, LARGE2["vocab"], n + steps) for n in lens]
    cpu = orc.DenseModel(LARGE2, deq, B, max(lens) + steps + 2)
    refs = [cpu.forward(s[None], [0], row0=b)[0] for b, s in enumerate(seqs)]
    cache = gpu.empty_kv_cache_with_capacity(512, batch=B, dtype="int8")
    for b in range(B):
        gpu.forward_with_cache(seqs[b][None, :lens[b]], 0, cache, row=b, last_only=True)
    got = _decode_steps(gpu, cache, [[int(seqs[b][lens[b] + s]) for b in range(B)] for s in range(steps)], B)
    assert pkg().device_status() == 0
    for s in range(steps):
        for b in range(B):
            assert rel_err(got[s][b], refs[b][lens[b] + s]) < STACK_TOL, (s, b)


def test_decode_step_attention_over_long_int8_context(large2):
    """The attention route of the batched decode step (rotation + append, then the
    tensor-core flash-decode over the appended but uncommitted token) at 8 rows of about
    16384 cached tokens: one Large-class block with a narrow feed-forward, the cache
    filled directly, and the step rebuilt from the oracle's operators over what the
    cache holds."""
    p = pkg()
    _, packed, deq = large2
    c = dict(LARGE2, n_layers=1, ffn_hidden=1024, vocab=1024, max_seq=16640)
    g = torch.Generator(device="cuda").manual_seed(21)
    w, d = dict(packed), dict(deq)
    for name, shape in (("embedding", (1024, 4096)), ("lm_head", (1024, 4096)), ("layers.0.w_gate", (1024, 4096)),
                        ("layers.0.w_up", (1024, 4096)), ("layers.0.w_down", (4096, 1024))):
        t = torch.randn(shape, generator=g, device="cuda") * 0.02
        w[name] = p.QuantLinear.quantise(t, "w4a16", 128)
        d[name] = w[name].dequantise().cpu().numpy()
    cfg = p.ModelConfig(1, 4096, 32, 8, 128, 1024, 1024, c["max_seq"], 1e-5, 10000.0, False)
    gpu = p.AarambhModel(cfg, w, dtype=torch.bfloat16, max_tokens=8)
    B, ctx = 8, 16384
    lens = [ctx - 61 * b for b in range(B)]
    lens[5] = 100
    cache = gpu.empty_kv_cache_with_capacity(ctx + 8, batch=B, dtype="int8")
    _fill_rows(cache, lens, 8, 128, 23)
    before = {b: [t.cpu().numpy() for t in cache.read(b)] for b in (0, 5, 7)}
    ids = [3, 77, 500, 9, 1023, 64, 640, 31]
    side = torch.cuda.Stream()
    logits = torch.empty((B, 1024), dtype=torch.bfloat16, device="cuda")
    tok = torch.tensor(ids, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        gpu.decode_step(tok, cache, logits, None)
        side.synchronize()
    assert p.device_status() == 0
    got = logits.float().cpu().numpy()
    cos, sin = orc.rope_tables(c["max_seq"], 128)
    ones = np.ones(4096, np.float32)
    scale = 1.0 / math.sqrt(128)
    for b in (0, 5, 7):
        n = lens[b]
        x = d["embedding"][ids[b]][None]
        xn = orc.rms_norm(x, ones, 1e-5)
        q = orc.linear(xn, d["layers.0.wq"]).reshape(1, 1, 32, 128)
        k = orc.linear(xn, d["layers.0.wk"]).reshape(1, 1, 8, 128)
        v = orc.linear(xn, d["layers.0.wv"]).reshape(1, 1, 8, 128)
        q = orc.rope_apply(q, cos, sin, n)
        k = orc.rope_apply(k, cos, sin, n)
        ck, sk = orc.quantise_kv_rows(k[0]); cv, sv = orc.quantise_kv_rows(v[0])
        kc = np.concatenate([before[b][0], ck.astype(np.float32) * sk[..., None]])[None]
        vc = np.concatenate([before[b][1], cv.astype(np.float32) * sv[..., None]])[None]
        att = orc.attention_decode_gqa(q[:, 0], kc, vc, np.array([n + 1], np.int32), scale).reshape(1, 4096)
        x = x + orc.linear(att, d["layers.0.wo"])
        xn = orc.rms_norm(x, ones, 1e-5)
        hid = orc.swiglu(orc.linear(xn, d["layers.0.w_gate"]), orc.linear(xn, d["layers.0.w_up"]))
        x = x + orc.linear(hid, d["layers.0.w_down"])
        ref = orc.linear(orc.rms_norm(x, ones, 1e-5), d["lm_head"])[0]
        assert rel_err(got[b], ref) < 2e-2, b
        assert cache.seq_len(b) == n + 1
