"""Pins the CPU oracle to the known-answer vectors held by the reference's own
unit tests (cited per test).  These run without a GPU."""
import math

import numpy as np
import pytest

from oracle import oracle as orc


def sin_vector(n=256):
    # crates/aarambh-studio-quant/src/qat.rs:442-446
    i = np.arange(n, dtype=np.float32)
    return (np.sin((i * np.float32(0.117)).astype(np.float32)).astype(np.float32)
            * np.float32(1.7) - np.float32(0.13)).astype(np.float32)


def sin_vector_rust(n=256):
    """Same vector with libm sinf on f32 inputs, as Rust's f32::sin computes it."""
    import ctypes
    libm = ctypes.CDLL("libm.so.6")
    libm.sinf.argtypes = [ctypes.c_float]
    libm.sinf.restype = ctypes.c_float
    out = np.empty(n, np.float32)
    for i in range(n):
        x = np.float32(np.float32(i) * np.float32(0.117))
        out[i] = np.float32(np.float32(libm.sinf(float(x))) * np.float32(1.7)) - np.float32(0.13)
    return out


def patterned_values(n, scale):
    # crates/aarambh-studio-kernel/tests/kernel_tests.rs:27-34
    idx = np.arange(n)
    return (((idx % 31).astype(np.float32) - np.float32(15.0)) * np.float32(scale)).astype(np.float32)


def test_nibble_roundtrip_odd_count():
    # crates/aarambh-studio-quant/src/int4.rs:98-103
    values = np.array([0, 1, 15, 7, 9], np.uint8)
    packed = orc.pack_i4(values)
    assert packed.tolist() == [0x10, 0x7F, 0x09]
    assert orc.unpack_i4(packed, 5).tolist() == values.tolist()


def test_int4_ramp_roundtrip_error():
    # crates/aarambh-studio-quant/src/int4.rs:105-121
    values = (np.arange(31, dtype=np.float32) * np.float32(0.03) - np.float32(0.5)).astype(np.float32)
    packed, scales, zeros = orc.quantise_affine_i4(values, 8)
    assert scales.shape == (4,) and packed.shape == (16,)
    dq = orc.dequantise_i4(packed, 31, 8, scales, zeros)
    assert np.abs(values - dq).max() < 0.04
    # independent numpy statement of int4.rs:17-33 for the same vector
    for g in range(4):
        chunk = values[g * 8:(g + 1) * 8]
        s = np.float32((chunk.max() - chunk.min()) / np.float32(15.0))
        assert scales[g] == s
        z = np.float32(math.floor(abs(float(-chunk.min() / s)) + 0.5) * (1 if -chunk.min() >= 0 else -1))
        assert zeros[g] == z


def test_custom_f16_roundtrip():
    # crates/aarambh-studio-quant/src/gguf_quant.rs:116-122
    for value in [-12.5, -1.0, 0.0, 0.5, 3.25, 100.0]:
        decoded = orc.f16_to_f32(orc.f32_to_f16(value))
        assert abs(float(decoded) - value) < 0.05
    # exact cases: representable values survive bit-for-bit
    for value in [-12.5, -1.0, 0.0, 0.5, 3.25, 100.0]:
        assert float(orc.f16_to_f32(orc.f32_to_f16(value))) == float(np.float16(value))


def test_custom_f16_rounds_half_up_not_even():
    # gguf_quant.rs:78-82: bit 12 set -> +1, regardless of the bits below.
    tie = np.array([0x3F801000], np.uint32).view(np.float32)[0]   # 1 + 2^-11: exact tie
    assert orc.f32_to_f16(tie) == 0x3C01           # half-up
    assert orc.f32_to_f16_rne(tie) == 0x3C00       # IEEE nearest-even
    assert int(np.float16(tie).view(np.uint16)) == 0x3C00
    # flush below half_exp < -10 to signed zero (gguf_quant.rs:66-68)
    assert orc.f32_to_f16(1e-9) == 0 and orc.f32_to_f16(-1e-9) == 0x8000
    # inf / nan (gguf_quant.rs:58-60)
    assert orc.f32_to_f16(float("inf")) == 0x7C00
    assert orc.f32_to_f16(float("nan")) == 0x7E00


def test_f16_rne_matches_numpy_on_random_bits():
    rng = np.random.default_rng(5)
    vals = rng.standard_normal(4000).astype(np.float32) * np.float32(10.0) ** rng.integers(-8, 5, 4000)
    vals = vals.astype(np.float32)
    with np.errstate(over="ignore"):
        for v in vals:
            assert orc.f32_to_f16_rne(v) == int(np.float16(v).view(np.uint16))


def test_q4_block_ramp_error():
    # crates/aarambh-studio-quant/src/gguf_quant.rs:124-136
    w = (np.arange(256, dtype=np.float32) * np.float32(0.01) - np.float32(1.28)).astype(np.float32)
    enc = orc.quantise_block_q4km(w)
    assert enc.shape == (132,)
    dq = orc.dequantise_block_q4km(enc)
    assert np.abs(w - dq).max() < 0.09


@pytest.mark.parametrize("maker", [sin_vector, sin_vector_rust])
def test_q4_block_codec_equals_tensor_formula_bit_exact(maker):
    # crates/aarambh-studio-quant/src/qat.rs:448-461: two independent statements of the
    # codec inside the reference agree exactly; the oracle must agree with both.
    v = maker()
    via_block = orc.dequantise_block_q4km(orc.quantise_block_q4km(v))
    via_tensor_ops = orc.fake_quant_export_q4km(v)
    assert np.array_equal(via_block.view(np.uint32), via_tensor_ops.view(np.uint32))


@pytest.mark.parametrize("maker", [sin_vector, sin_vector_rust])
def test_q4_padded_tail_bit_exact(maker):
    # crates/aarambh-studio-quant/src/qat.rs:463-476
    v = maker()[:173]
    padded = np.zeros(256, np.float32)
    padded[:173] = v
    expected = orc.dequantise_block_q4km(orc.quantise_block_q4km(padded))[:173]
    actual = orc.fake_quant_export_q4km(v)
    assert np.array_equal(actual.view(np.uint32), expected.view(np.uint32))
    # tensor-level wrappers (crates/aarambh-studio-weights/src/gguf.rs:214-241)
    payload = orc.encode_q4km_tensor(v)
    assert payload.size == 132
    assert np.array_equal(orc.decode_q4km_tensor(payload, (173,)).view(np.uint32),
                          expected.view(np.uint32))


@pytest.mark.parametrize("maker", [sin_vector, sin_vector_rust])
def test_int8_fake_quant_equals_codes_times_scale(maker):
    # crates/aarambh-studio-quant/src/qat.rs:478-495
    v = maker()
    codes, scale = orc.quantise_absmax_i8(v)
    expected = codes.astype(np.float32) * scale
    # fake_quant_symmetric(…, Tensor): round(w / s).clamp(±127) * s   (qat.rs:140-156)
    s = np.float32(np.abs(v).max() / np.float32(127.0))
    w_over_s = (v / s).astype(np.float32)
    rounded = np.sign(w_over_s) * np.floor(np.abs(w_over_s) + np.float32(0.5))
    fake = (np.clip(rounded, -127, 127).astype(np.float32) * s).astype(np.float32)
    assert scale == s
    assert np.array_equal(fake.view(np.uint32), expected.view(np.uint32))
    assert np.array_equal(orc.dequantise_i8(codes, scale).view(np.uint32), expected.view(np.uint32))
    # per-row variant reduces to the per-tensor one for a single row
    rc, rs = orc.quantise_absmax_i8_rows(v.reshape(1, -1))
    assert rs[0] == scale and np.array_equal(rc.ravel(), codes)


def test_int8_degenerate_and_saturation():
    # crates/aarambh-studio-quant/src/absmax.rs:10-17
    codes, scale = orc.quantise_absmax_i8(np.zeros(7, np.float32))
    assert scale == 1.0 and not codes.any()
    codes, scale = orc.quantise_absmax_i8(np.array([1e-8, -1e-8], np.float32))
    assert scale == 1.0
    # round half away from zero (f32::round), not half-to-even
    v = np.array([127.0, 0.5, 1.5, 2.5, -0.5, -2.5], np.float32)
    codes, scale = orc.quantise_absmax_i8(v)
    assert scale == 1.0
    assert codes.tolist() == [127, 1, 2, 3, -1, -3]
    codes, _ = orc.quantise_absmax_i8(np.array([np.nan, 1.0], np.float32))
    assert codes[0] == 0


def test_q4_tensor_shape_and_payload_length():
    # crates/aarambh-studio-weights/src/gguf.rs:324-338
    vals = (np.arange(300, dtype=np.float32) * np.float32(0.01) - np.float32(1.5)).reshape(20, 15)
    payload = orc.encode_q4km_tensor(vals)
    assert payload.size == math.ceil(300 / 256) * 132
    out = orc.decode_q4km_tensor(payload, (20, 15))
    assert out.shape == (20, 15) and np.isfinite(out).all()


def test_encode_f16_pair():
    # crates/aarambh-studio-weights/src/gguf.rs:316-322
    assert abs(float(orc.f16_to_f32(orc.f32_to_f16(0.125))) - 0.125) < 1e-3
    assert abs(float(orc.f16_to_f32(orc.f32_to_f16(-2.5))) + 2.5) < 1e-3


def test_quantised_kv_cache_grows():
    # crates/aarambh-studio-quant/src/kv_quant.rs:81-91
    cache = orc.QuantisedKvCache(1)
    k1 = np.full((1, 1, 1, 4), 0.1, np.float32)
    v1 = np.full((1, 1, 1, 4), 0.2, np.float32)
    cache.append_and_get(0, k1, v1)
    assert cache.seq_len(0) == 1
    k_full, _ = cache.append_and_get(0, k1, v1)
    assert cache.seq_len(0) == 2 and k_full.shape == (1, 2, 1, 4)


def _dense_attention(q, k, v, scale, mask=None):
    # attention_forward_candle, crates/aarambh-studio-kernel/src/dispatch.rs:269-283
    s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) * scale
    if mask is not None:
        s = s + mask
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    return np.einsum("bhqk,bhkd->bhqd", p, v.astype(np.float64))


def test_attention_matches_dense_reference_without_mask():
    # crates/aarambh-studio-kernel/tests/kernel_tests.rs:91-120
    q = patterned_values(2 * 3 * 5 * 16, 0.015).reshape(2, 3, 5, 16)
    k = patterned_values(2 * 3 * 7 * 16, 0.012).reshape(2, 3, 7, 16)
    v = patterned_values(2 * 3 * 7 * 16, 0.01).reshape(2, 3, 7, 16)
    scale = 1.0 / math.sqrt(16.0)
    expected = _dense_attention(q, k, v, scale)
    actual = orc.attention(q, k, v, scale)
    sequential = orc.attention(q, k, v, scale, parallel=False)
    assert np.abs(actual - expected).max() < 1e-4
    assert np.abs(actual - sequential).max() < 1e-6


def test_attention_matches_dense_reference_with_broadcast_mask():
    # crates/aarambh-studio-kernel/tests/kernel_tests.rs:122-161
    qs, kvs = 5, 7
    q = patterned_values(2 * 3 * qs * 16, 0.017).reshape(2, 3, qs, 16)
    k = patterned_values(2 * 3 * kvs * 16, 0.011).reshape(2, 3, kvs, 16)
    v = patterned_values(2 * 3 * kvs * 16, 0.013).reshape(2, 3, kvs, 16)
    mask = np.array([[0.0 if kv <= qi + 2 else -1.0e9 for kv in range(kvs)] for qi in range(qs)],
                    np.float32).reshape(1, 1, qs, kvs)
    scale = 1.0 / math.sqrt(16.0)
    expected = _dense_attention(q, k, v, scale, mask)
    actual = orc.attention(q, k, v, scale, mask=mask)
    assert np.abs(actual - expected).max() < 1e-4


def test_causal_cut_matches_causal_mask():
    # causal_mask rule, crates/aarambh-studio-kernel/src/dispatch.rs:296-316, against the
    # in-loop skip of crates/aarambh-studio-kernel/src/cpu/parallel_attn.rs:205-209
    qs, kvs = 3, 7
    q = patterned_values(1 * 2 * qs * 8, 0.05).reshape(1, 2, qs, 8)
    k = patterned_values(1 * 2 * kvs * 8, 0.04).reshape(1, 2, kvs, 8)
    v = patterned_values(1 * 2 * kvs * 8, 0.03).reshape(1, 2, kvs, 8)
    shift = kvs - qs
    mask = np.array([[0.0 if kv <= shift + qi else -np.inf for kv in range(kvs)]
                     for qi in range(qs)], np.float32).reshape(1, 1, qs, kvs)
    a = orc.attention(q, k, v, 0.35, causal=True)
    b = orc.attention(q, k, v, 0.35, mask=mask)
    assert np.array_equal(a, b)
    assert np.abs(a - _dense_attention(q, k, v, 0.35, mask)).max() < 1e-5


def test_decode_gqa_equals_repeat_heads_path():
    # crates/aarambh-studio-nn/src/attention.rs:265-283,415-428
    rng = np.random.default_rng(0)
    b, h, kvh, hd, cap = 2, 6, 2, 8, 9
    lens = np.array([5, 9], np.int32)
    q = rng.standard_normal((b, h, hd)).astype(np.float32)
    kc = rng.standard_normal((b, cap, kvh, hd)).astype(np.float32)
    vc = rng.standard_normal((b, cap, kvh, hd)).astype(np.float32)
    out = orc.attention_decode_gqa(q, kc, vc, lens, 0.3)
    for bi in range(b):
        L = lens[bi]
        kr = np.repeat(kc[bi:bi + 1, :L], h // kvh, axis=2).transpose(0, 2, 1, 3)
        vr = np.repeat(vc[bi:bi + 1, :L], h // kvh, axis=2).transpose(0, 2, 1, 3)
        ref = orc.attention(q[bi:bi + 1, :, None, :], kr, vr, 0.3, causal=True)
        assert np.array_equal(out[bi], ref[0, :, 0, :])


def test_rms_norm_tail_lanes():
    # crates/aarambh-studio-kernel/tests/kernel_tests.rs:46-66
    x = patterned_values(4 * 7 * 65, 0.02).reshape(4, 7, 65)
    w = (np.float32(0.75) + np.arange(65, dtype=np.float32) * np.float32(0.001)).astype(np.float32)
    x64 = x.astype(np.float64)
    expected = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-5) * w
    for simd in (True, False):
        actual = orc.rms_norm(x, w, 1e-5, simd_order=simd)
        assert actual.shape == x.shape
        assert np.abs(actual - expected).max() < 1e-4


def test_kv_cache_truncate_and_regrow():
    # crates/aarambh-studio-nn/src/kvcache.rs:380-420
    def vals(v):
        return np.array(v, np.float32).reshape(1, len(v), 1, 1)
    for cap in (None, 4):
        cache = orc.KVCache(cap)
        cache.update(vals([1.0, 2.0]), vals([3.0, 4.0]))
        cache.truncate(1)
        keys, _ = cache.update(vals([9.0]), vals([8.0]))
        assert cache.seq_len() == 2
        assert keys.ravel().tolist() == [1.0, 9.0]
    with pytest.raises(ValueError):
        orc.KVCache(4).truncate(1)
    c = orc.KVCache(2)
    c.update(vals([1.0, 2.0]), vals([1.0, 2.0]))
    with pytest.raises(ValueError):
        c.update(vals([3.0]), vals([3.0]))


def test_rope_preserves_norm():
    # crates/aarambh-studio-nn/src/rope.rs:144-172
    rng = np.random.default_rng(1)
    x = rng.standard_normal((1, 4, 8, 64)).astype(np.float32)
    cos, sin = orc.rope_tables(16, 64)
    out = orc.rope_apply(x, cos, sin, 3)
    n0 = np.sqrt((x.astype(np.float64) ** 2).sum(-1))
    n1 = np.sqrt((out.astype(np.float64) ** 2).sum(-1))
    assert np.abs(n0 - n1).max() < 1e-4
    assert np.allclose(orc.rope_apply(x, cos, sin, 0)[:, 0], x[:, 0])  # position 0 = identity


def test_argmax_takes_last_maximum():
    # crates/aarambh-studio-inference/src/sampler.rs:217-224
    assert orc.argmax([1.0, 3.0, 3.0, 2.0]) == 2
    assert orc.argmax([0.0, -0.0]) == 0          # total_cmp: -0 < +0
    assert orc.argmax([-0.0, 0.0]) == 1
    assert orc.argmax([1.0, np.nan, np.inf]) == 1  # +NaN sorts above +inf
    assert orc.argmax([5.0]) == 0


def test_w4a16_dequant_orders():
    rng = np.random.default_rng(2)
    N, K, g = 4, 2048, 128
    codes = rng.integers(0, 16, (N, K), dtype=np.uint32)
    zeros = rng.integers(0, 16, (N, K // g), dtype=np.uint32)
    scales = orc.bf16_bits(rng.uniform(0.005, 0.02, (N, K // g)).astype(np.float32))
    expect = (codes.astype(np.float32) - np.repeat(zeros, g, 1).astype(np.float32)) \
        * np.repeat(orc.bf16_to_f32(scales), g, 1)
    for awq in (False, True):
        order = [0, 2, 4, 6, 1, 3, 5, 7] if awq else list(range(8))
        qw = np.zeros((N, K // 8), np.uint32)
        qz = np.zeros((N, K // g // 8), np.uint32)
        for slot, elem in enumerate(order):
            qw |= codes[:, elem::8] << np.uint32(4 * slot)
            qz |= zeros[:, elem::8] << np.uint32(4 * slot)
        out = orc.dequant_w4a16(qw, scales, qz, N, K, g, awq_order=awq)
        assert np.array_equal(out.view(np.uint32), expect.astype(np.float32).view(np.uint32))
