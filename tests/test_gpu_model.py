"""Decoder parity: logits against the oracle's dense f32 model and the greedy
token stream of the Tiny-class workload (32-token prompt, 128 new tokens)."""
import numpy as np
import pytest
import torch

from helpers import pkg, rel_err
from model_fixtures import SMALL, TINY, build_pair
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def prompt(vocab, n=32, seed=1):
    return np.random.default_rng(seed).integers(0, vocab, n)


@pytest.mark.parametrize("method", ["int8", "int8_channel", "int4", "q4_k_m"])
def test_prefill_and_decode_logits_match_oracle(method):
    gpu, cpu, _ = build_pair(SMALL, method, capacity=32)
    ids = prompt(SMALL["vocab"], 9)
    cache = gpu.empty_kv_cache_with_capacity(32)
    lg = gpu.forward_with_cache(ids[None], 0, cache).cpu().numpy()
    ref = cpu.forward(ids[None], [0])
    assert lg.shape == ref.shape == (1, 9, SMALL["vocab"])
    assert rel_err(lg, ref) < 1e-4
    nxt = np.array([[orc.argmax(ref[0, -1])]])
    lg2 = gpu.forward_decode_batch(nxt, [9], cache).cpu().numpy()
    ref2 = cpu.forward(nxt, [9])
    assert rel_err(lg2, ref2) < 1e-4
    assert cache.seq_len() == 10 == cpu.seq_len()


def test_cached_forward_equals_full_forward():
    # crates/aarambh-studio-model/tests/model_tests.rs:177-202 (max abs diff < 1e-4)
    gpu, _, _ = build_pair(SMALL, "int8", capacity=32)
    ids = prompt(SMALL["vocab"], 12)
    full = gpu.forward_with_cache(ids[None], 0, gpu.empty_kv_cache_with_capacity(32)).cpu().numpy()
    cache = gpu.empty_kv_cache_with_capacity(32)
    a = gpu.forward_with_cache(ids[None, :7], 0, cache).cpu().numpy()
    b = gpu.forward_with_cache(ids[None, 7:], 7, cache).cpu().numpy()
    assert np.abs(np.concatenate([a, b], 1) - full).max() < 1e-4


def test_batched_decode_equals_independent_sequences():
    # crates/aarambh-studio-inference/src/engine.rs:1296-1373: ragged rows do not interact
    gpu, _, _ = build_pair(SMALL, "int8_channel", capacity=32)
    pa, pb = prompt(SMALL["vocab"], 5, 2), prompt(SMALL["vocab"], 11, 3)
    cache = gpu.empty_kv_cache_with_capacity(32, batch=2)
    gpu.forward_with_cache(pa[None], 0, cache, row=0)
    gpu.forward_with_cache(pb[None], 0, cache, row=1)
    both = gpu.forward_decode_batch(np.array([[7], [9]]), [5, 11], cache).cpu().numpy()
    for row, (pr, tok) in enumerate([(pa, 7), (pb, 9)]):
        solo = gpu.empty_kv_cache_with_capacity(32)
        gpu.forward_with_cache(pr[None], 0, solo)
        one = gpu.forward_decode_batch(np.array([[tok]]), [len(pr)], solo).cpu().numpy()
        assert np.abs(one[0] - both[row]).max() < 1e-5


def test_capacity_and_max_seq_errors():
    p = pkg()
    gpu, _, _ = build_pair(SMALL, "int8", capacity=8)
    cache = gpu.empty_kv_cache_with_capacity(8)
    with pytest.raises(p.Ab2Error) as e:
        gpu.forward_with_cache(prompt(SMALL["vocab"], 9)[None], 0, cache)
    assert e.value.status == -4
    with pytest.raises(p.Ab2Error) as e:
        gpu.forward_decode_batch(np.array([[1]]), [SMALL["max_seq"]], cache)
    assert e.value.status == -1
    with pytest.raises(p.Ab2Error):
        gpu.forward_decode_batch(np.array([[SMALL["vocab"]]]), [0], cache)


@pytest.mark.parametrize("method", ["int8_channel", "int8"])
def test_tiny_greedy_token_stream_is_identical(method):
    """Tiny-class decoder, INT8 weights, f32 activations and KV: 32-token prompt
    (seed 1), 128 greedy tokens, token-for-token equal to the oracle."""
    gpu, cpu, _ = build_pair(TINY, method, capacity=160)
    ids = prompt(TINY["vocab"], 32, seed=1)
    out = pkg().InferenceEngine(gpu).generate_from_token_ids(ids, 128)
    # oracle: prefill then one token at a time, argmax = last maximum
    logits = cpu.forward(ids[None], [0])[0, -1]
    ref, margins = [], []
    for step in range(128):
        tok = orc.argmax(logits)
        top2 = np.partition(logits, -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
        ref.append(tok)
        if step < 127:
            logits = cpu.forward(np.array([[tok]]), [32 + step])[0, 0]
    assert out["token_ids"] == ref, f"first mismatch at {next(i for i,(a,b) in enumerate(zip(out['token_ids'], ref)) if a != b)}; min margin {min(margins):.3e}"
    # the host-sampled path (logits to the host each step) gives the same stream
    out2 = pkg().InferenceEngine(gpu).generate_from_token_ids(ids, 128, on_device_sampling=False)
    assert out2["token_ids"] == ref
    print(f"min top-1/top-2 logit margin over 128 steps: {min(margins):.3e}; engine would stop at step {out['eos_step']}")


def test_bf16_int8kv_model_close_to_oracle():
    """bf16 activations + INT8 KV on the W4A16 path: logits within 1e-2 relative
    of the dense f32 oracle over the same dequantised weights (d_model must be a
    multiple of 128 for group-128 weights)."""
    cfg = dict(SMALL)
    gpu, cpu, _ = build_pair(cfg, "w4a16", dtype=torch.bfloat16, capacity=32)
    ids = prompt(cfg["vocab"], 10)
    cache = gpu.empty_kv_cache_with_capacity(32, dtype="int8")
    lg = gpu.forward_with_cache(ids[None], 0, cache).float().cpu().numpy()
    ref = cpu.forward(ids[None], [0])
    assert rel_err(lg, ref) < 2e-2


def test_fused_epilogue_path_matches_unfused_operators():
    """Large-class block shapes scaled down: the decoder's fused projection
    epilogues (residual add, SwiGLU) against the same step assembled from the
    unfused operators of the C ABI."""
    import math
    p = pkg()
    cfg = dict(SMALL, d_model=512, ffn_hidden=1024, n_heads=4, n_kv_heads=2, head_dim=128, n_layers=1)
    gpu, _, packed = build_pair(cfg, "w4a16", dtype=torch.bfloat16, capacity=32)
    ids = torch.tensor([[5, 9, 200, 17]])
    cache = gpu.empty_kv_cache_with_capacity(32, dtype="bf16")
    got = gpu.forward_with_cache(ids, 0, cache).float()
    D = p.dispatch
    bf = torch.bfloat16
    x = D.embedding_forward(packed["embedding"], ids.cuda(), bf)[0]
    cos, sin = [torch.from_numpy(a).cuda() for a in orc.rope_tables(cfg["max_seq"], 128)]
    ones = torch.ones(512, device="cuda")
    xn = D.rms_norm(x, ones, 1e-5)
    q = packed["layers.0.wq"](xn).view(1, 4, 4, 128); k = packed["layers.0.wk"](xn).view(1, 4, 2, 128)
    v = packed["layers.0.wv"](xn).view(1, 4, 2, 128)
    q = D.fused_rope_apply(q, cos, sin, 0); k = D.fused_rope_apply(k, cos, sin, 0)
    c2 = p.KVCache(32, 2, 128, 4, dtype="bf16")
    c2.update(k, v)
    att = D.attention_cached(c2, q, 1 / math.sqrt(128)).view(4, 512)
    x = x + packed["layers.0.wo"](att)
    xn = D.rms_norm(x, ones, 1e-5)
    hid = D.fused_swiglu(packed["layers.0.w_gate"](xn), packed["layers.0.w_up"](xn))
    x = x + packed["layers.0.w_down"](hid)
    ref = packed["embedding"](D.rms_norm(x, ones, 1e-5)).float()
    assert rel_err(got[0].cpu().numpy(), ref.cpu().numpy()) < 1e-2


@pytest.mark.parametrize("prompt_len", [5, 120, 150, 300, 510, 600])
def test_decode_step_head_dim_128_int8_kv_matches_oracle(prompt_len):
    """The one-token step on the Large-class block shapes scaled down (head_dim
    128, grouped queries, INT8 KV, W4A16 weights, bf16): graph-replayed decode
    steps (cluster attention over 1, 2, 4 and 8 context splits, with 4, 2 and 1 lanes per cached token, RMSNorm fused into
    the one-token GEMV) against the dense f32 oracle run over the whole sequence,
    and against the plain-launch decode of the same tokens.  From 510 cached tokens the
    steps cross a power of two of the context length, where the step graph is captured anew."""
    cfg = dict(SMALL, d_model=512, ffn_hidden=1024, n_heads=4, n_kv_heads=2, head_dim=128, n_layers=2,
               max_seq=1024)
    gpu, cpu, _ = build_pair(cfg, "w4a16", dtype=torch.bfloat16, max_tokens=640, capacity=640)
    steps = 4
    ids = prompt(cfg["vocab"], prompt_len + steps, 7)
    ref = cpu.forward(ids[None], [0])[0]                       # [S, vocab]
    cache = gpu.empty_kv_cache_with_capacity(prompt_len + steps + 2, dtype="int8")
    cache2 = gpu.empty_kv_cache_with_capacity(prompt_len + steps + 2, dtype="int8")
    gpu.forward_with_cache(ids[None, :prompt_len], 0, cache)
    gpu.forward_with_cache(ids[None, :prompt_len], 0, cache2)
    side = torch.cuda.Stream()
    logits = torch.empty((1, cfg["vocab"]), dtype=torch.bfloat16, device="cuda")
    tok = torch.empty(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    for s in range(steps):
        pos = prompt_len + s
        with torch.cuda.stream(side):
            tok.fill_(int(ids[pos]))
            gpu.decode_step(tok, cache, logits, None)
            side.synchronize()
        got = logits.float().cpu().numpy()[0]
        assert rel_err(got, ref[pos]) < 2e-2, (prompt_len, s)
        plain = gpu.forward_decode_batch(np.array([[int(ids[pos])]]), [pos], cache2).float().cpu().numpy()[0, 0]
        assert rel_err(got, plain) < 1e-2, (prompt_len, s)
    assert pkg().device_status() == 0


@pytest.mark.parametrize("B", [1, 3])
def test_decode_step_with_host_tokens_equals_the_device_step(B):
    """ab2_model_decode_step_host (ids and greedy tokens in pinned host memory, one call
    per step, each step's tokens fed to the next) against the device-side step on a second
    cache: the same token stream, and both equal to the argmax of the oracle's logits over
    the sequence generated so far."""
    cfg = dict(SMALL, d_model=512, ffn_hidden=1024, n_heads=4, n_kv_heads=2, head_dim=128, n_layers=2,
               max_seq=256)
    gpu, cpu, _ = build_pair(cfg, "w4a16", dtype=torch.bfloat16, max_tokens=64, batch=B, capacity=64)
    P, steps = 9, 5
    prompts = np.stack([prompt(cfg["vocab"], P, 40 + b) for b in range(B)])
    host_cache = gpu.empty_kv_cache_with_capacity(P + steps + 2, batch=B, dtype="int8")
    dev_cache = gpu.empty_kv_cache_with_capacity(P + steps + 2, batch=B, dtype="int8")
    for b in range(B):
        gpu.forward_with_cache(prompts[b:b + 1, :P - 1], 0, host_cache, row=b)
        gpu.forward_with_cache(prompts[b:b + 1, :P - 1], 0, dev_cache, row=b)
    bufs = [torch.empty(B, dtype=torch.int32).pin_memory() for _ in range(2)]
    bufs[0].copy_(torch.from_numpy(prompts[:, P - 1].astype(np.int32)))
    dev = [torch.empty(B, dtype=torch.int32, device="cuda") for _ in range(2)]
    side = torch.cuda.Stream()
    seqs = [list(prompts[b]) for b in range(B)]
    with torch.cuda.stream(side):
        dev[0].copy_(bufs[0])
        for s in range(steps):
            gpu.decode_step_host(bufs[s & 1], host_cache, bufs[(s + 1) & 1])
            gpu.decode_step(dev[s & 1], dev_cache, None, dev[(s + 1) & 1])
            side.synchronize()
            got = bufs[(s + 1) & 1].numpy().copy()
            assert np.array_equal(got, dev[(s + 1) & 1].cpu().numpy()), s
            for b in range(B):
                ref = cpu.forward(np.asarray(seqs[b])[None], [0], row0=b)[0][-1]
                top = np.sort(ref)[-2:]
                if top[1] - top[0] > 2e-2 * np.abs(ref).max():  # a clear winner: the tokens must agree
                    assert int(got[b]) == int(np.argmax(ref)), (s, b)
                seqs[b].append(int(got[b]))
    assert pkg().device_status() == 0
    with pytest.raises(pkg().Ab2Error):
        gpu.decode_step_host(dev[0], host_cache, bufs[0])


def test_batched_decode_rows_match_single_row_decode_on_the_w4a16_path():
    """20 sequences decoded together (tensor-memory decode GEMM, one attention launch
    for all rows) and 12 together (warp kernel with the residual and SwiGLU
    epilogues) against each sequence decoded alone."""
    cfg = dict(SMALL, d_model=512, ffn_hidden=1024, n_heads=4, n_kv_heads=2, head_dim=128, n_layers=2,
               max_seq=128)
    gpu, _, _ = build_pair(cfg, "w4a16", dtype=torch.bfloat16, max_tokens=64, capacity=64)
    for B in (12, 20):
        _batched_vs_single(gpu, cfg, B)


def _batched_vs_single(gpu, cfg, B):
    P, steps = 6, 3
    rng = np.random.default_rng(21)
    prompts = rng.integers(0, cfg["vocab"], (B, P))
    nxt = rng.integers(0, cfg["vocab"], (steps, B))
    together = gpu.empty_kv_cache_with_capacity(32, batch=B, dtype="int8")
    for b in range(B):
        gpu.forward_with_cache(prompts[b:b + 1], 0, together, row=b)
    alone = [gpu.empty_kv_cache_with_capacity(32, dtype="int8") for _ in range(B)]
    for b in range(B):
        gpu.forward_with_cache(prompts[b:b + 1], 0, alone[b])
    for s in range(steps):
        lg = gpu.forward_decode_batch(nxt[s][:, None], [P + s] * B, together).float().cpu().numpy()
        for b in range(B):
            one = gpu.forward_decode_batch(nxt[s][b:b + 1, None], [P + s], alone[b]).float().cpu().numpy()
            assert rel_err(lg[b], one[0]) < 2e-2, (s, b)
    assert pkg().device_status() == 0


def test_batched_decode_step_over_ragged_long_rows_matches_oracle():
    """Four rows of 300, 257, 64 and 290 cached tokens decoded together: enough cached
    tokens per step that attention runs as rotation + append + the tensor-core
    flash-decode over uncommitted tokens (context splits, one of them empty for the
    short row) + merge.  Graph-replayed steps against the dense f32 oracle of each
    sequence."""
    cfg = dict(SMALL, d_model=512, ffn_hidden=1024, n_heads=4, n_kv_heads=2, head_dim=128, n_layers=2,
               max_seq=512)
    lens, steps = [300, 257, 64, 290], 3
    B = len(lens)
    gpu, cpu, _ = build_pair(cfg, "w4a16", dtype=torch.bfloat16, max_tokens=320, batch=B, capacity=320)
    seqs = [prompt(cfg["vocab"], n + steps, 31 + i) for i, n in enumerate(lens)]
    refs = [cpu.forward(s[None], [0], row0=i)[0] for i, s in enumerate(seqs)]   # [S, vocab] each
    cache = gpu.empty_kv_cache_with_capacity(max(lens) + steps + 2, batch=B, dtype="int8")
    for b in range(B):
        gpu.forward_with_cache(seqs[b][None, :lens[b]], 0, cache, row=b)
    side = torch.cuda.Stream()
    logits = torch.empty((B, cfg["vocab"]), dtype=torch.bfloat16, device="cuda")
    tok = torch.empty(B, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    for s in range(steps):
        with torch.cuda.stream(side):
            tok.copy_(torch.tensor([int(seqs[b][lens[b] + s]) for b in range(B)], dtype=torch.int32))
            gpu.decode_step(tok, cache, logits, None)
            side.synchronize()
        got = logits.float().cpu().numpy()
        for b in range(B):
            assert rel_err(got[b], refs[b][lens[b] + s]) < 2e-2, (s, b)
    assert pkg().device_status() == 0


@pytest.mark.parametrize("prompt_len", [5, 300, 510])
def test_persistent_decode_step_matches_oracle(prompt_len, monkeypatch):
    """The opt-in form of the one-row decode step (AB2_PERSISTENT_STEP=1 when the model is
    finalised): one cooperative kernel for the whole step.  Same comparison as the
    graph-replayed step: logits against the dense f32 oracle over the whole sequence, the
    greedy token against the argmax of the returned logits, the cache length advanced on
    the device; without AB2_PS_TRACE the phase trace is refused."""
    p = pkg()
    monkeypatch.setenv("AB2_PERSISTENT_STEP", "1")
    cfg = dict(SMALL, d_model=512, ffn_hidden=1024, n_heads=4, n_kv_heads=2, head_dim=128, n_layers=2,
               max_seq=1024)
    gpu, cpu, _ = build_pair(cfg, "w4a16", dtype=torch.bfloat16, max_tokens=640, capacity=640)
    steps = 4
    ids = prompt(cfg["vocab"], prompt_len + steps, 7)
    ref = cpu.forward(ids[None], [0])[0]
    cache = gpu.empty_kv_cache_with_capacity(prompt_len + steps + 2, dtype="int8")
    gpu.forward_with_cache(ids[None, :prompt_len], 0, cache)
    side = torch.cuda.Stream()
    logits = torch.empty((1, cfg["vocab"]), dtype=torch.bfloat16, device="cuda")
    tok = torch.empty(1, dtype=torch.int32, device="cuda")
    out = torch.empty(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    for s in range(steps):
        pos = prompt_len + s
        with torch.cuda.stream(side):
            tok.fill_(int(ids[pos]))
            gpu.decode_step(tok, cache, logits, out)
            side.synchronize()
        got = logits.float().cpu().numpy()[0]
        assert rel_err(got, ref[pos]) < 2e-2, (prompt_len, s)
        assert int(out[0]) == orc.argmax(got)
        assert cache.seq_len() == pos + 1
    assert p.device_status() == 0
    with pytest.raises(p.Ab2Error) as e:
        gpu.step_trace()
    assert e.value.status == -8
