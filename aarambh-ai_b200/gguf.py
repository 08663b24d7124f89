"""Loader of the reference's v1 "GGUF-compatible" checkpoints that keeps the
quantised payloads packed: Q8_0 and Q4_K_M tensors go to the GPU as codes and are
consumed by the fused dequant kernels, instead of being dequantised to dense f32
on the host as ``load_gguf_tensors`` does
(crates/aarambh-studio-weights/src/gguf.rs:79-131,152-241).  The container
itself is parsed by ``gguf_format``.
"""
from __future__ import annotations

import struct

import numpy as np
import torch

from .gguf_format import ENC_F32, ENC_Q8_0, GgufError, GgufTensor, read_gguf  # noqa: F401
from .model import AarambhModel, ModelConfig
from .qlinear import QuantLinear


def _config(c: dict) -> ModelConfig:
    """ModelConfig JSON (crates/aarambh-studio-core/src/config.rs:734-773) -> the fields this path uses."""
    for unsupported in ("moe", "attention_schedule", "dsa_config", "mtp", "rope_scaling"):
        if c.get(unsupported) is not None:
            raise GgufError(f"checkpoint uses '{unsupported}', which this decoder does not serve")
    d, h = c["hidden_dim"], c["n_heads"]
    return ModelConfig(c["n_layers"], d, h, c["n_kv_heads"], d // h, c["ffn_dim"], c["vocab_size"], c["max_seq_len"],
                       float(c.get("norm_eps", 1e-5)), float(c.get("rope_theta", 10000.0)),
                       bool(c.get("tie_embeddings", True)))


def _packed(t: GgufTensor):
    """A rank-2 tensor as packed device weights (no host dequantisation); 1-D f32 as a device tensor."""
    if t.encoding == ENC_F32:
        return torch.from_numpy(np.frombuffer(t.payload, dtype="<f4").reshape(t.shape).copy()).cuda()
    if len(t.shape) != 2:
        raise GgufError(f"{t.name}: quantised tensors must have rank 2, got shape {t.shape}")
    N, K = t.shape
    if t.encoding == ENC_Q8_0:
        scale = struct.unpack("<f", t.payload[:4])[0]
        codes = np.frombuffer(t.payload, dtype=np.int8, offset=4).reshape(N, K)
        return QuantLinear.from_i8_tensor(codes, scale, N, K)
    return QuantLinear.from_q4km_blocks(np.frombuffer(t.payload, dtype=np.uint8), N, K)


def load_gguf_model(path: str, dtype: torch.dtype = torch.float32, max_tokens: int = 512) -> AarambhModel:
    """``load_gguf_with_dtype`` (gguf.rs:79-88) with the weights left packed on the GPU."""
    cfg_json, _fmt, tensors, keep = read_gguf(path)
    cfg = _config(cfg_json)
    names = {"embedding.weight": "embedding", "final_norm.weight": "final_norm", "lm_head.weight": "lm_head"}
    for i in range(cfg.n_layers):
        names[f"blocks.{i}.norm1.weight"] = f"layers.{i}.norm1"
        names[f"blocks.{i}.norm2.weight"] = f"layers.{i}.norm2"
        for w in ("wq", "wk", "wv", "wo"):
            names[f"blocks.{i}.attn.{w}.weight"] = f"layers.{i}.{w}"
        for w in ("w_gate", "w_up", "w_down"):
            names[f"blocks.{i}.ffn.{w}.weight"] = f"layers.{i}.{w}"
    weights = {}
    for name, t in tensors.items():
        if name not in names:
            raise GgufError(f"checkpoint tensor '{name}' has no place in the dense decoder")
        weights[names[name]] = _packed(t)
    missing = [n for n in names.values() if n not in weights and not (n == "lm_head" and cfg.tie_embeddings)]
    if missing:
        raise GgufError(f"checkpoint lacks {missing[:3]}{'...' if len(missing) > 3 else ''}")
    model = AarambhModel(cfg, weights, dtype=dtype, max_tokens=max_tokens)
    del keep
    return model
