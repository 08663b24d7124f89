"""KV cache semantics and grouped-query attention against the oracle.
Attention tolerance: 1e-2 relative for bf16 / INT8-KV outputs (the bar stated
for attention outputs), 1e-5 for f32 (summation order only); an INT8 cache
with f32 queries is held to 1e-3, because the tensor-core path rounds the
queries and probabilities to fp16 before its MMAs."""
import math

import numpy as np
import pytest
import torch

from helpers import bits, pkg, rel_err
from oracle import oracle as orc
from test_oracle_golden import patterned_values

pytestmark = pytest.mark.gpu


def cuda(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dtype)


def vals(v):
    return cuda(np.array(v, np.float32).reshape(1, len(v), 1, 1).repeat(32, axis=3))


def test_preallocated_cache_truncates_and_regrows():
    # crates/aarambh-studio-nn/src/kvcache.rs:399-420
    p = pkg()
    cache = p.KVCache.with_capacity(4, 1, 32, 1)
    cache.update(vals([1.0, 2.0]), vals([3.0, 4.0]))
    cache.truncate(1)
    keys, values = cache.update(vals([9.0]), vals([8.0]))
    assert cache.seq_len() == 2 and cache.capacity() == 4
    assert keys[:, 0, 0].cpu().tolist() == [1.0, 9.0]
    assert values[:, 0, 0].cpu().tolist() == [3.0, 8.0]
    with pytest.raises(p.Ab2Error) as e:
        p.KVCache.with_capacity(4, 1, 32, 1).truncate(1)     # cannot grow
    assert e.value.status == -4
    with pytest.raises(p.Ab2Error) as e:
        cache.update(vals([1.0, 2.0, 3.0]), vals([1.0, 2.0, 3.0]))  # exceeds capacity
    assert e.value.status == -4
    cache.clear()
    assert cache.seq_len() == 0


def test_snapshot_and_restore():
    # crates/aarambh-studio-inference/src/kvcache.rs:57-64
    p = pkg()
    cache = p.KVCache.with_capacity(8, 1, 32, 1)
    cache.update(vals([1.0, 2.0]), vals([3.0, 4.0]))
    snap = cache.snapshot()
    cache.update(vals([5.0]), vals([6.0]))
    assert cache.seq_len() == 3 and snap.seq_len() == 2
    cache.restore(snap)
    assert cache.seq_len() == 2
    assert cache.read()[0][:, 0, 0].cpu().tolist() == [1.0, 2.0]


@pytest.mark.parametrize("dtype", ["f32", "bf16", "int8"])
def test_update_stores_what_the_oracle_stores(dtype):
    rng = np.random.default_rng(30)
    B, S, kvh, hd = 2, 5, 2, 64
    k = rng.standard_normal((B, S, kvh, hd)).astype(np.float32)
    v = rng.standard_normal((B, S, kvh, hd)).astype(np.float32)
    k[0, 1, 0] = 0.0  # degenerate vector -> scale 1.0 (absmax.rs:10-14)
    cache = pkg().KVCache(16, kvh, hd, 4, batch=B, dtype=dtype)
    cache.update(cuda(k), cuda(v))
    for b in range(B):
        gk, gv = [t.cpu().numpy() for t in cache.read(b)]
        if dtype == "f32":
            ek, ev = k[b], v[b]
        elif dtype == "bf16":
            ek, ev = orc.round_bf16(k[b]), orc.round_bf16(v[b])
        else:
            ck, sk = orc.quantise_kv_rows(k[b]); cv, sv = orc.quantise_kv_rows(v[b])
            ek = ck.astype(np.float32) * sk[..., None]; ev = cv.astype(np.float32) * sv[..., None]
        assert np.array_equal(bits(gk), bits(ek.astype(np.float32)))
        assert np.array_equal(bits(gv), bits(ev.astype(np.float32)))


def test_append_with_rope_matches_oracle_rotation():
    rng = np.random.default_rng(31)
    kvh, hd = 2, 64
    cos, sin = orc.rope_tables(32, hd)
    cache = pkg().KVCache(16, kvh, hd, 4)
    k1 = rng.standard_normal((1, 3, kvh, hd)).astype(np.float32)
    cache.append(0, cuda(k1), cuda(k1), cos=cuda(cos), sin=cuda(sin), max_seq=32); cache.commit(3)
    k2 = rng.standard_normal((1, 2, kvh, hd)).astype(np.float32)
    cache.append(0, cuda(k2), cuda(k2), cos=cuda(cos), sin=cuda(sin), max_seq=32); cache.commit(2)
    gk, gv = [t.cpu().numpy() for t in cache.read()]
    ek = np.concatenate([orc.rope_apply(k1, cos, sin, 0)[0], orc.rope_apply(k2, cos, sin, 3)[0]])
    assert np.array_equal(bits(gk), bits(ek))
    assert np.array_equal(bits(gv), bits(np.concatenate([k1[0], k2[0]])))


def _fill(cache, k, v, lens):
    """k, v [B, cap, kvh, hd]; fills row b with its first lens[b] tokens."""
    for b, n in enumerate(lens):
        cache.update(cuda(k[b:b + 1, :n]), cuda(v[b:b + 1, :n]), row0=b)


@pytest.mark.parametrize("kv_dtype,act,tol", [("f32", torch.float32, 1e-5), ("bf16", torch.bfloat16, 1e-2),
                                              ("int8", torch.bfloat16, 1e-2), ("int8", torch.float32, 1e-3)])
@pytest.mark.parametrize("h,kvh,hd,lens", [(32, 8, 128, [1000, 37]), (6, 2, 64, [160, 1, 33]),
                                           (8, 8, 128, [300]), (16, 2, 128, [2049, 512])])
def test_decode_attention_matches_oracle(kv_dtype, act, tol, h, kvh, hd, lens):
    rng = np.random.default_rng(3)
    B, cap = len(lens), max(lens)
    k = rng.standard_normal((B, cap, kvh, hd)).astype(np.float32)
    v = rng.standard_normal((B, cap, kvh, hd)).astype(np.float32)
    q = rng.standard_normal((B, h, hd)).astype(np.float32)
    if act == torch.bfloat16:
        q = orc.round_bf16(q)
    p = pkg()
    cache = p.KVCache(cap, kvh, hd, h, batch=B, dtype=kv_dtype)
    _fill(cache, k, v, lens)
    scale = 1.0 / math.sqrt(hd)
    got = p.dispatch.attention_decode(cache, cuda(q, act), scale).float().cpu().numpy()
    # the oracle attends over exactly what the cache holds
    kd = np.zeros_like(k); vd = np.zeros_like(v)
    for b, n in enumerate(lens):
        a, c = cache.read(b)
        kd[b, :n] = a.cpu().numpy(); vd[b, :n] = c.cpu().numpy()
    ref = orc.attention_decode_gqa(q, kd, vd, np.array(lens, np.int32), scale)
    assert rel_err(got, ref) < tol


def test_int8_kv_attention_against_unquantised_reference():
    """The microbenchmark's comparison (INT8 KV against dequant + softmax
    attention): the kernel stays within 1e-2 relative of the oracle run over the
    same quantised cache; what separates both from the unquantised f32 attention
    is the quantisation error itself, which this test bounds separately."""
    rng = np.random.default_rng(3)
    h, kvh, hd, n = 32, 8, 128, 4096
    k = rng.standard_normal((1, n, kvh, hd)).astype(np.float32)
    v = rng.standard_normal((1, n, kvh, hd)).astype(np.float32)
    q = orc.round_bf16(rng.standard_normal((1, h, hd)).astype(np.float32))
    p = pkg()
    cache = p.KVCache(n, kvh, hd, h, dtype="int8")
    cache.update(cuda(k), cuda(v))
    scale = 1 / math.sqrt(hd)
    got = p.dispatch.attention_decode(cache, cuda(q, torch.bfloat16), scale).float().cpu().numpy()
    ck, sk = orc.quantise_kv_rows(k); cv, sv = orc.quantise_kv_rows(v)
    kq = ck.astype(np.float32) * sk[..., None]; vq = cv.astype(np.float32) * sv[..., None]
    lens = np.array([n], np.int32)
    ref_q = orc.attention_decode_gqa(q, kq, vq, lens, scale)
    ref = orc.attention_decode_gqa(q, k, v, lens, scale)
    assert rel_err(got, ref_q) < 1e-2
    assert rel_err(ref_q, ref) < 3e-2      # quantisation error of the format, oracle against oracle
    assert rel_err(got, ref) < 3e-2


@pytest.mark.parametrize("kv_dtype", ["f32", "int8"])
def test_prefill_attention_is_causal(kv_dtype):
    rng = np.random.default_rng(32)
    h, kvh, hd, old, S = 6, 2, 64, 7, 9
    k = rng.standard_normal((1, old + S, kvh, hd)).astype(np.float32)
    v = rng.standard_normal((1, old + S, kvh, hd)).astype(np.float32)
    q = rng.standard_normal((1, S, h, hd)).astype(np.float32)
    p = pkg()
    cache = p.KVCache(32, kvh, hd, h, dtype=kv_dtype)
    cache.update(cuda(k), cuda(v))
    got = p.dispatch.attention_cached(cache, cuda(q), 0.125).cpu().numpy()
    kd, vd = [t.cpu().numpy() for t in cache.read()]
    kr = np.repeat(kd[None], h // kvh, axis=2).transpose(0, 2, 1, 3)
    vr = np.repeat(vd[None], h // kvh, axis=2).transpose(0, 2, 1, 3)
    ref = orc.attention(q.transpose(0, 2, 1, 3), kr, vr, 0.125, causal=True).transpose(0, 2, 1, 3)
    assert rel_err(got, ref) < 1e-5


def test_attention_forward_causal_reference_shapes():
    # shapes and patterned inputs of crates/aarambh-studio-kernel/tests/kernel_tests.rs:91-120,
    # through the causal entry point (dispatch.rs:145-160)
    q = patterned_values(2 * 3 * 5 * 16, 0.015).reshape(2, 3, 5, 16)
    k = patterned_values(2 * 3 * 7 * 16, 0.012).reshape(2, 3, 7, 16)
    v = patterned_values(2 * 3 * 7 * 16, 0.01).reshape(2, 3, 7, 16)
    scale = 1.0 / math.sqrt(16.0)
    got = pkg().dispatch.attention_forward_causal(cuda(q), cuda(k), cuda(v), scale).cpu().numpy()
    assert np.abs(got - orc.attention(q, k, v, scale, causal=True)).max() < 1e-6


def test_attention_forward_causal_gqa_fast_path():
    rng = np.random.default_rng(33)
    b, h, kvh, ql, kl, hd = 2, 8, 2, 5, 40, 128
    q = rng.standard_normal((b, h, ql, hd)).astype(np.float32)
    k = rng.standard_normal((b, kvh, kl, hd)).astype(np.float32)
    v = rng.standard_normal((b, kvh, kl, hd)).astype(np.float32)
    got = pkg().dispatch.attention_forward_causal(cuda(q), cuda(k), cuda(v), 0.09).cpu().numpy()
    ref = orc.attention(q, np.repeat(k, h // kvh, 1), np.repeat(v, h // kvh, 1), 0.09, causal=True)
    assert rel_err(got, ref) < 1e-5


def test_attention_errors():
    p = pkg()
    cache = p.KVCache(8, 2, 64, 4)
    with pytest.raises(p.Ab2Error):   # empty cache: kv_seq must be non-zero
        p.dispatch.attention_decode(cache, torch.zeros(1, 4, 64, device="cuda"), 1.0)
    with pytest.raises(p.Ab2Error):
        p.KVCache(8, 3, 64, 4)        # heads not divisible
    with pytest.raises(p.Ab2Error):
        p.dispatch.attention_forward_causal(torch.zeros(1, 2, 3, 16, device="cuda"),
                                            torch.zeros(2, 2, 3, 16, device="cuda"),
                                            torch.zeros(2, 2, 3, 16, device="cuda"), 1.0)


@pytest.mark.parametrize("lens,S,h,kvh", [([512], 512, 32, 8), ([82, 45], 45, 8, 2), ([317, 600], 17, 4, 4),
                                          ([2, 40], 2, 32, 8), ([1030], 129, 16, 8)])
def test_prefill_attention_over_int8_cache_on_tensor_cores(lens, S, h, kvh):
    """S > 1 queries per sequence over an INT8 cache, head_dim 128 (prefill chunks, speculative
    verification): the tensor-core causal kernel against the oracle's causal attention over
    exactly what the cache holds.  Covers the 512-token prompt of the decode benchmark at
    32 / 8 heads, chunks that are not multiples of the 16-query tile, a cached prefix, ragged
    rows and every heads-per-KV-head ratio the kernel serves (1, 2, 4)."""
    rng = np.random.default_rng(34)
    hd, B = 128, len(lens)
    p = pkg()
    cache = p.KVCache(max(lens), kvh, hd, h, batch=B, dtype="int8")
    k = rng.standard_normal((B, max(lens), kvh, hd)).astype(np.float32)
    v = rng.standard_normal((B, max(lens), kvh, hd)).astype(np.float32)
    _fill(cache, k, v, lens)
    q = orc.round_bf16(rng.standard_normal((B, S, h, hd)).astype(np.float32))
    scale = 1.0 / math.sqrt(hd)
    got = p.dispatch.attention_cached(cache, cuda(q, torch.bfloat16), scale).float().cpu().numpy()
    assert p.device_status() == 0
    for b, n in enumerate(lens):
        kd, vd = [t.cpu().numpy() for t in cache.read(b)]          # [n, kvh, hd], dequantised
        kr = np.repeat(kd[None], h // kvh, axis=2).transpose(0, 2, 1, 3)
        vr = np.repeat(vd[None], h // kvh, axis=2).transpose(0, 2, 1, 3)
        ref = orc.attention(q[b:b + 1].transpose(0, 2, 1, 3), kr, vr, scale, causal=True).transpose(0, 2, 1, 3)
        assert rel_err(got[b], ref[0]) < 1e-2, (b, n)
