"""Element-wise operators against the oracle (RMSNorm, RoPE, SwiGLU, argmax,
embedding).  f32 tolerances: RoPE bit-exact (same operations, no fused
multiply-add); RMSNorm / SwiGLU 1e-6 relative (summation order, expf)."""
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


def test_rms_norm_reference_vector():
    # crates/aarambh-studio-kernel/tests/kernel_tests.rs:46-66 (tail lanes: 65 columns)
    x = patterned_values(4 * 7 * 65, 0.02).reshape(4, 7, 65)
    w = (np.float32(0.75) + np.arange(65, dtype=np.float32) * np.float32(0.001)).astype(np.float32)
    got = pkg().dispatch.rms_norm(cuda(x), cuda(w), 1e-5).cpu().numpy()
    assert got.shape == x.shape
    assert np.abs(got - orc.rms_norm(x, w, 1e-5, simd_order=True)).max() < 1e-4
    assert rel_err(got, orc.rms_norm(x, w, 1e-5, simd_order=False)) < 1e-6


@pytest.mark.parametrize("d", [384, 4096])
def test_rms_norm_rows(d):
    rng = np.random.default_rng(20)
    x = rng.standard_normal((5, d)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, d).astype(np.float32)
    got = pkg().dispatch.rms_norm(cuda(x), cuda(w), 1e-5).cpu().numpy()
    assert rel_err(got, orc.rms_norm(x, w, 1e-5)) < 1e-6
    xb = orc.round_bf16(x)
    gb = pkg().dispatch.rms_norm(cuda(xb, torch.bfloat16), cuda(w), 1e-5).float().cpu().numpy()
    assert rel_err(gb, orc.rms_norm(xb, w, 1e-5)) < 1e-2


def test_rms_norm_errors():
    p = pkg()
    with pytest.raises(p.Ab2Error):
        p.dispatch.rms_norm(torch.zeros(2, 8, device="cuda"), torch.zeros(7, device="cuda"), 1e-5)
    with pytest.raises(p.Ab2Error):
        p.dispatch.rms_norm(torch.zeros(2, 8), torch.zeros(8), 1e-5)  # CPU tensors: no fallback


@pytest.mark.parametrize("hd,offset", [(64, 0), (64, 3), (128, 17)])
def test_rope_bit_exact_and_norm_preserving(hd, offset):
    # crates/aarambh-studio-nn/src/rope.rs:144-172
    rng = np.random.default_rng(21)
    x = rng.standard_normal((1, 4, 8, hd)).astype(np.float32)
    cos, sin = orc.rope_tables(32, hd)
    got = pkg().dispatch.fused_rope_apply(cuda(x), cuda(cos), cuda(sin), offset).cpu().numpy()
    ref = orc.rope_apply(x, cos, sin, offset)
    assert np.array_equal(bits(got), bits(ref))
    assert np.abs(np.linalg.norm(got, axis=-1) - np.linalg.norm(x, axis=-1)).max() < 1e-4


def test_rope_table_overflow_is_an_error():
    p = pkg()
    cos, sin = orc.rope_tables(8, 64)
    with pytest.raises(p.Ab2Error):
        p.dispatch.fused_rope_apply(torch.zeros(1, 4, 2, 64, device="cuda"), cuda(cos), cuda(sin), 6)


def test_swiglu():
    rng = np.random.default_rng(22)
    g = (rng.standard_normal(4099) * 3).astype(np.float32)
    u = rng.standard_normal(4099).astype(np.float32)
    got = pkg().dispatch.fused_swiglu(cuda(g), cuda(u)).cpu().numpy()
    assert rel_err(got, orc.swiglu(g, u)) < 1e-6


def test_argmax_last_maximum_and_total_order():
    # crates/aarambh-studio-inference/src/sampler.rs:217-224
    p = pkg()
    cases = [[1.0, 3.0, 3.0, 2.0], [0.0, -0.0], [-0.0, 0.0], [1.0, float("nan"), float("inf")], [5.0],
             [-1.0, -1.0, -2.0]]
    for c in cases:
        got = int(p.dispatch.argmax(cuda(np.array([c], np.float32)))[0])
        assert got == orc.argmax(c), c
    rng = np.random.default_rng(23)
    logits = rng.standard_normal((3, 8192)).astype(np.float32)
    logits[1, 100] = logits[1, 7000] = 9.0
    got = p.dispatch.argmax(cuda(logits)).cpu().tolist()
    assert got == [orc.argmax(r) for r in logits] and got[1] == 7000


@pytest.mark.parametrize("method", ["int8", "int8_channel", "int4", "q4_k_m", "w4a16"])
def test_embedding_gathers_dequantised_rows(method):
    rng = np.random.default_rng(24)
    table = (rng.standard_normal((512, 384)) * 0.02).astype(np.float32)
    lin = pkg().QuantLinear.quantise(cuda(table), method, 128)
    dense = lin.dequantise().cpu().numpy()
    ids = np.array([[0, 511, 17], [3, 3, 200]])
    got = pkg().dispatch.embedding_forward(lin, torch.from_numpy(ids).cuda(), torch.float32).cpu().numpy()
    assert np.array_equal(bits(got), bits(dense[ids]))
