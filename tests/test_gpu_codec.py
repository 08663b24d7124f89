"""Codec parity on the GPU: packed weights built from the reference layouts
dequantise bit-exactly to the oracle's values, and the device-side quantisers
reproduce the oracle's codes and parameters bit-for-bit."""
import numpy as np
import pytest
import torch

from helpers import AWQ_ORDER, bits, make_w4a16, pack_w4, pkg
from oracle import oracle as orc
from test_oracle_golden import sin_vector_rust

pytestmark = pytest.mark.gpu


def weights(rng, N, K, std=0.02):
    return (rng.standard_normal((N, K)) * std).astype(np.float32)


@pytest.mark.parametrize("shape", [(16, 16), (48, 384), (33, 200)])
def test_i8_tensor_dequant_bit_exact(shape):
    rng = np.random.default_rng(10)
    w = weights(rng, *shape)
    codes, scale = orc.quantise_absmax_i8(w)
    lin = pkg().QuantLinear.from_i8_tensor(codes, scale, *shape)
    got = lin.dequantise().cpu().numpy()
    assert np.array_equal(bits(got), bits(orc.dequantise_i8(codes, scale)))


def test_i8_golden_vector_on_gpu():
    # crates/aarambh-studio-quant/src/qat.rs:478-495 through the GPU codec
    v = sin_vector_rust().reshape(16, 16)
    codes, scale = orc.quantise_absmax_i8(v)
    lin = pkg().QuantLinear.quantise(torch.from_numpy(v).cuda(), "int8")
    gc, gs, _ = lin.export()
    assert np.array_equal(gc, codes) and gs[0] == scale
    assert np.array_equal(bits(lin.dequantise().cpu().numpy()), bits(codes.astype(np.float32) * scale))


def test_i8_channel_quantiser_and_dequant():
    rng = np.random.default_rng(11)
    w = weights(rng, 40, 384)
    w[3] = 0.0  # degenerate row -> scale 1.0 (qat.rs:165-169)
    codes, scales = orc.quantise_absmax_i8_rows(w)
    lin = pkg().QuantLinear.quantise(torch.from_numpy(w).cuda(), "int8_channel")
    gc, gs, _ = lin.export()
    assert np.array_equal(gc, codes)
    assert np.array_equal(bits(gs), bits(scales))
    assert np.array_equal(bits(lin.dequantise().cpu().numpy()), bits(orc.dequantise_i8_rows(codes, scales)))
    lin2 = pkg().QuantLinear.from_i8_channel(codes, scales, 40, 384)
    assert np.array_equal(bits(lin2.dequantise().cpu().numpy()), bits(orc.dequantise_i8_rows(codes, scales)))


@pytest.mark.parametrize("shape,group", [((1, 31), 8), ((8, 384), 128), ((20, 15), 8), ((6, 1024), 128),
                                         ((5, 100), 32)])
def test_i4_affine_dequant_bit_exact(shape, group):
    rng = np.random.default_rng(12)
    w = weights(rng, *shape, std=0.3)
    if shape == (1, 31):  # the reference's ramp (int4.rs:105-121)
        w = (np.arange(31, dtype=np.float32) * np.float32(0.03) - np.float32(0.5)).reshape(1, 31)
    packed, scales, zeros = orc.quantise_affine_i4(w, group)
    lin = pkg().QuantLinear.from_i4_affine(packed, scales, zeros, *shape, group)
    got = lin.dequantise().cpu().numpy().ravel()
    assert np.array_equal(bits(got), bits(orc.dequantise_i4(packed, w.size, group, scales, zeros)))


@pytest.mark.parametrize("shape,group", [((8, 384), 128), ((20, 15), 8), ((7, 96), 64), ((3, 50), 20)])
def test_i4_affine_device_quantiser_bit_exact(shape, group):
    rng = np.random.default_rng(13)
    w = weights(rng, *shape, std=0.5)
    w.ravel()[: group] = 0.25  # degenerate group -> scale 1.0 (int4.rs:20-24)
    packed, scales, zeros = orc.quantise_affine_i4(w, group)
    lin = pkg().QuantLinear.quantise(torch.from_numpy(w).cuda(), "int4", group)
    gc, gs, gz = lin.export()
    assert np.array_equal(gc, packed)
    assert np.array_equal(bits(gs), bits(scales)) and np.array_equal(bits(gz), bits(zeros))


@pytest.mark.parametrize("shape", [(16, 16), (1, 173), (20, 15), (12, 384), (4, 1024)])
def test_q4km_blocks_bit_exact(shape):
    rng = np.random.default_rng(14)
    w = weights(rng, *shape, std=0.4)
    if shape == (16, 16):  # crates/aarambh-studio-quant/src/qat.rs:448-461
        w = sin_vector_rust().reshape(16, 16)
    if shape == (1, 173):  # qat.rs:463-476 (zero-padded tail)
        w = sin_vector_rust()[:173].reshape(1, 173)
    payload = orc.encode_q4km_tensor(w)
    expect = orc.decode_q4km_tensor(payload, shape)
    lin = pkg().QuantLinear.from_q4km_blocks(payload, *shape)
    assert np.array_equal(bits(lin.dequantise().cpu().numpy()), bits(expect))
    assert np.array_equal(lin.export()[0], payload)
    lin2 = pkg().QuantLinear.quantise(torch.from_numpy(w).cuda(), "q4_k_m")
    assert np.array_equal(lin2.export()[0], payload)
    assert np.array_equal(bits(lin2.dequantise().cpu().numpy()), bits(orc.fake_quant_export_q4km(w)))


@pytest.mark.parametrize("awq", [False, True])
def test_w4a16_dequant_bit_exact(awq):
    rng = np.random.default_rng(2)
    N, K, g = 64, 2048, 128
    qw, scales, qz = make_w4a16(rng, N, K, g, awq=awq)
    ctor = pkg().QuantLinear.from_w4a16_awq if awq else pkg().QuantLinear.from_w4a16_gptq
    lin = ctor(qw, scales, qz, N, K, g)
    expect = orc.dequant_w4a16(qw, scales, qz, N, K, g, awq_order=awq)
    assert np.array_equal(bits(lin.dequantise().cpu().numpy()), bits(expect))
    # bf16 output is the f32 value rounded to nearest even
    got16 = lin.dequantise(torch.bfloat16).float().cpu().numpy()
    assert np.array_equal(bits(got16), bits(orc.round_bf16(expect)))


def test_w4a16_device_quantiser_roundtrip():
    rng = np.random.default_rng(15)
    N, K, g = 32, 1024, 128
    w = weights(rng, N, K)
    lin = pkg().QuantLinear.quantise(torch.from_numpy(w).cuda(), "w4a16", g)
    codes, scales, qz = lin.export()
    dense = orc.dequant_w4a16(codes, scales, qz, N, K, g)
    assert np.array_equal(bits(lin.dequantise().cpu().numpy()), bits(dense))
    s = np.repeat(orc.bf16_to_f32(scales), g, axis=1)
    assert np.abs(dense - w).max() <= 0.51 * s.max() + 1e-7


def test_constructor_errors():
    p = pkg()
    with pytest.raises(p.Ab2Error) as e:
        p.QuantLinear.from_w4a16_gptq(np.zeros((4, 12), np.uint32), np.zeros((4, 1), np.uint16),
                                      np.zeros((4, 1), np.uint32), 4, 96, 128)
    assert e.value.status == -1
    with pytest.raises(p.Ab2Error):
        p.QuantLinear.from_i4_affine(np.zeros(8, np.uint8), np.zeros(1, np.float32),
                                     np.zeros(1, np.float32), 4, 4, 0)
