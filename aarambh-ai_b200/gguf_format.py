"""Parser of the reference's v1 "GGUF-compatible" checkpoint container (no GPU, no
dependency on the rest of the package).  The loader built on it keeps the
quantised payloads packed: Q8_0 and Q4_K_M tensors go to the GPU as codes and
are consumed by the fused dequant kernels, instead of being dequantised to dense
f32 on the host as ``load_gguf_tensors`` does
(crates/aarambh-studio-weights/src/gguf.rs:91-131,152-241).

Layout (gguf.rs:46-72), little endian: ``b"GGUF"``, u32 version (1), u64 length +
JSON ``{"config": ModelConfig, "format": "q4_k_m" | "q5_k_m" | "q80"}``, u64
tensor count, then per tensor (sorted by name): u64 length + UTF-8 name, u64 rank
+ u64 dims, u8 encoding (0 = f32, 1 = Q8_0: f32 scale + i8 codes, 2 = Q4_K_M:
132-byte blocks of 256 values over the flattened tensor), u64 payload length,
payload.  Tensor names are those of ``AarambhModel::named_tensors``
(crates/aarambh-studio-model/src/model.rs:665-698).
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass

import numpy as np

MAGIC = b"GGUF"
VERSION = 1
ENC_F32, ENC_Q8_0, ENC_Q4KM = 0, 1, 2
Q4KM_BLOCK, Q4KM_BYTES = 256, 132


class GgufError(RuntimeError):
    """A malformed or unsupported checkpoint (AarambhError::Checkpoint in the reference)."""


@dataclass
class GgufTensor:
    name: str
    shape: tuple
    encoding: int
    payload: memoryview   # view into the mapped file


def read_gguf(path: str):
    """Parses the container.  Returns (config dict, format string, {name: GgufTensor}, the mapping to keep alive)."""
    f = open(path, "rb")
    mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    view = memoryview(mm)
    pos = 0

    def take(n):
        nonlocal pos
        if pos + n > len(view):
            raise GgufError(f"{path}: truncated checkpoint (wanted {n} bytes at offset {pos})")
        out = view[pos:pos + n]
        pos += n
        return out

    def u64():
        return struct.unpack("<Q", take(8))[0]

    if bytes(take(4)) != MAGIC:
        raise GgufError(f"{path} is not an Aarambh GGUF file")
    version = struct.unpack("<I", take(4))[0]
    if version != VERSION:
        raise GgufError(f"unsupported GGUF version {version}, expected {VERSION}")
    meta = json.loads(bytes(take(u64())))
    tensors = {}
    for _ in range(u64()):
        name = bytes(take(u64())).decode("utf-8")
        shape = tuple(u64() for _ in range(u64()))
        enc = take(1)[0]
        if enc not in (ENC_F32, ENC_Q8_0, ENC_Q4KM):
            raise GgufError(f"unknown GGUF tensor encoding {enc}")
        payload = take(u64())
        n = int(np.prod(shape)) if shape else 1
        if enc == ENC_F32 and len(payload) != 4 * n:
            raise GgufError("invalid F32 GGUF payload length")
        if enc == ENC_Q8_0 and len(payload) != 4 + n:
            raise GgufError("invalid Q8_0 payload")
        if enc == ENC_Q4KM and len(payload) != (n + Q4KM_BLOCK - 1) // Q4KM_BLOCK * Q4KM_BYTES:
            raise GgufError("invalid Q4_K_M GGUF payload length")
        tensors[name] = GgufTensor(name, shape, enc, payload)
    return meta["config"], meta["format"], tensors, (f, mm)


