"""Test infrastructure: writes a checkpoint in the reference's v1 GGUF-compatible
container exactly as ``save_gguf`` does (crates/aarambh-studio-weights/src/gguf.rs:
46-72), with the tensor encodings of ``encode_tensor`` (gguf.rs:133-150): rank != 2
-> f32; otherwise Q8_0 (f32 absmax scale + i8 codes, gguf.rs:187-193) for format
"q80", Q4_K_M-style 132-byte blocks over the flattened, zero-padded tensor
(gguf.rs:214-224) for "q4_k_m" / "q5_k_m".  The codecs are the oracle's
restatements of absmax.rs and gguf_quant.rs.  Only tests use this module.
"""
import json
import struct

import numpy as np

from . import oracle as orc

ENC_F32, ENC_Q8_0, ENC_Q4KM = 0, 1, 2


def encode_tensor(name, value, fmt):
    """(encoding byte, payload bytes) of one tensor (gguf.rs:133-150)."""
    v = np.ascontiguousarray(value, np.float32)
    if v.ndim != 2 or "_conv." in name:
        return ENC_F32, v.astype("<f4").tobytes()
    if ".dsa.index_" in name or fmt == "q80":
        codes, scale = orc.quantise_absmax_i8(v)
        return ENC_Q8_0, struct.pack("<f", float(scale)) + codes.astype(np.int8).tobytes()
    if fmt in ("q4_k_m", "q5_k_m"):
        return ENC_Q4KM, orc.encode_q4km_tensor(v).tobytes()
    raise ValueError(f"unknown GGUF format {fmt}")


def decode_tensor(enc, shape, payload):
    """Dense f32 values as ``decode_tensor`` returns them (gguf.rs:152-241)."""
    if enc == ENC_F32:
        return np.frombuffer(payload, "<f4").reshape(shape).copy()
    if enc == ENC_Q8_0:
        scale = struct.unpack("<f", payload[:4])[0]
        return orc.dequantise_i8(np.frombuffer(payload, np.int8, offset=4).reshape(shape), scale)
    return orc.decode_q4km_tensor(np.frombuffer(payload, np.uint8), shape)


def save_gguf(path, config, tensors, fmt):
    """config: the ModelConfig JSON object; tensors: name -> f32 array (reference tensor names)."""
    with open(path, "wb") as f:
        f.write(b"GGUF")
        f.write(struct.pack("<I", 1))
        meta = json.dumps({"config": config, "format": fmt}).encode()
        f.write(struct.pack("<Q", len(meta)))
        f.write(meta)
        f.write(struct.pack("<Q", len(tensors)))
        for name in sorted(tensors):
            value = np.asarray(tensors[name], np.float32)
            nb = name.encode()
            f.write(struct.pack("<Q", len(nb)))
            f.write(nb)
            f.write(struct.pack("<Q", value.ndim))
            for dim in value.shape:
                f.write(struct.pack("<Q", dim))
            enc, payload = encode_tensor(name, value, fmt)
            f.write(bytes([enc]))
            f.write(struct.pack("<Q", len(payload)))
            f.write(payload)
