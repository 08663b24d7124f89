"""Shared helpers for the test-suite."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from __graft_entry__ import import_package  # noqa: E402


def pkg():
    return import_package()


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({4: np.uint32, 2: np.uint16, 1: np.uint8}[a.dtype.itemsize])


def rel_err(got, ref):
    """max |got - ref| / max |ref| — the relative error the parity bar is stated in."""
    got = np.asarray(got, np.float64); ref = np.asarray(ref, np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def pack_w4(codes, order=None):
    """[N, K] nibble values -> [N, K/8] u32 words; slot i holds element order[i]."""
    order = list(range(8)) if order is None else order
    codes = np.ascontiguousarray(codes, np.uint32)
    if codes.shape[1] % 8:
        codes = np.pad(codes, ((0, 0), (0, 8 - codes.shape[1] % 8)))
    out = np.zeros((codes.shape[0], codes.shape[1] // 8), np.uint32)
    for slot, elem in enumerate(order):
        out |= codes[:, elem::8] << np.uint32(4 * slot)
    return out


AWQ_ORDER = [0, 2, 4, 6, 1, 3, 5, 7]


def make_w4a16(rng, N, K, g=128, awq=False):
    """Random W4A16 weight per the microbenchmark spec: uniform packed ints,
    bf16 scales in [0.005, 0.02], zero points 0..15."""
    from oracle import oracle as orc
    codes = rng.integers(0, 16, (N, K), dtype=np.uint32)
    zeros = rng.integers(0, 16, (N, K // g), dtype=np.uint32)
    scales = orc.bf16_bits(rng.uniform(0.005, 0.02, (N, K // g)).astype(np.float32))
    order = AWQ_ORDER if awq else None
    return pack_w4(codes, order), scales, pack_w4(zeros, order)
