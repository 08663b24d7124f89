"""Host-side mirror of the reference's kernel dispatch entry points
(crates/aarambh-studio-kernel/src/dispatch.rs): rms_norm, attention_forward_causal,
plus the fused RoPE / SwiGLU wrappers and the greedy argmax.  Outputs are freshly
allocated, inputs are borrowed, tensors must be CUDA and are made contiguous.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, lib
from .qlinear import dtype_code, stream_ptr


def _cuda(t: torch.Tensor, what: str) -> torch.Tensor:
    if not t.is_cuda:
        raise _lib.Ab2Error(-7, f"{what} must be a CUDA tensor (this library has no CPU path)")
    return t.contiguous()


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x = _cuda(x, "x")
    d = x.shape[-1] if x.dim() else 0
    if x.dim() < 1 or d == 0:
        raise _lib.Ab2Error(-1, "rms_norm hidden dimension must be non-zero")
    if tuple(weight.shape) != (d,):
        raise _lib.Ab2Error(-1, f"rms_norm weight must have shape [{d}], got {list(weight.shape)}")
    w = _cuda(weight, "weight").float()
    out = torch.empty_like(x)
    check(lib.ab2_rms_norm(x.data_ptr(), w.data_ptr(), out.data_ptr(), x.numel() // d, d, float(eps),
                           dtype_code(x.dtype), stream_ptr()))
    return out


def fused_rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seqlen_offset: int) -> torch.Tensor:
    """x [batch, seq, heads, head_dim]; cos, sin [max_seq, head_dim/2] (f32)."""
    x = _cuda(x, "x")
    if x.dim() != 4:
        raise _lib.Ab2Error(-1, f"RoPE input must be [batch, seq, heads, head_dim], got {list(x.shape)}")
    b, s, h, hd = x.shape
    cos = _cuda(cos, "cos").float(); sin = _cuda(sin, "sin").float()
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] * 2 != hd:
        raise _lib.Ab2Error(-1, "RoPE tables must be [max_seq, head_dim/2]")
    out = torch.empty_like(x)
    check(lib.ab2_rope_apply(x.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), b, s, h, hd,
                             seqlen_offset, cos.shape[0], dtype_code(x.dtype), stream_ptr()))
    return out


def fused_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise _lib.Ab2Error(-1, "SwiGLU gate and up must have the same shape and dtype")
    gate = _cuda(gate, "gate"); up = _cuda(up, "up")
    out = torch.empty_like(gate)
    check(lib.ab2_swiglu(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), dtype_code(gate.dtype),
                         stream_ptr()))
    return out


def attention_forward_causal(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q [b, h, q_len, hd]; k, v [b, kv_heads, kv_len, hd] (kv heads not repeated)."""
    q = _cuda(q, "q"); k = _cuda(k, "k"); v = _cuda(v, "v")
    if q.dim() != 4 or k.dim() != 4 or v.shape != k.shape:
        raise _lib.Ab2Error(-1, "attention expects rank-4 q and matching rank-4 k, v")
    if q.shape[0] != k.shape[0]:
        raise _lib.Ab2Error(-1, "attention batch dimensions must match")
    if q.shape[3] != k.shape[3]:
        raise _lib.Ab2Error(-1, "attention head dimensions must match")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise _lib.Ab2Error(-3, "attention tensors must share one dtype")
    b, h, ql, hd = q.shape
    out = torch.empty_like(q)
    check(lib.ab2_attention_causal(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), b, h, k.shape[1],
                                   ql, k.shape[2], hd, float(scale), dtype_code(q.dtype), stream_ptr()))
    return out


def attention_decode(cache, q: torch.Tensor, scale: float, layer: int = 0, row0: int = 0) -> torch.Tensor:
    """q [rows, n_heads, head_dim]: one query per sequence over its cache."""
    q = _cuda(q, "q")
    out = torch.empty_like(q)
    check(lib.ab2_attention_decode(cache._h, layer, q.data_ptr(), out.data_ptr(), row0, q.shape[0],
                                   float(scale), dtype_code(q.dtype), stream_ptr()))
    return out


def attention_decode_static(cache, q: torch.Tensor, scale: float, out: torch.Tensor, layer: int = 0,
                            row0: int = 0) -> torch.Tensor:
    """``attention_decode`` for hosts that must not allocate on the device: the
    caller supplies ``out`` and the split scratch is a fixed array inside the
    library (8 MiB; larger problems are rejected).  Calls on different streams
    must not overlap."""
    if not q.is_contiguous() or not out.is_contiguous() or out.shape != q.shape or out.dtype != q.dtype:
        raise _lib.Ab2Error(-1, "q and out must be contiguous tensors of the same shape and dtype")
    check(lib.ab2_attention_decode_static(cache._h, layer, q.data_ptr(), out.data_ptr(), row0, q.shape[0],
                                          float(scale), dtype_code(q.dtype), stream_ptr()))
    return out


def attention_cached(cache, q: torch.Tensor, scale: float, layer: int = 0, row0: int = 0) -> torch.Tensor:
    """q [rows, S, n_heads, head_dim]: S new queries per sequence, causal."""
    q = _cuda(q, "q")
    out = torch.empty_like(q)
    check(lib.ab2_attention_cached(cache._h, layer, q.data_ptr(), out.data_ptr(), q.shape[1], row0, q.shape[0],
                                   float(scale), dtype_code(q.dtype), stream_ptr()))
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Greedy token per row: the last index among equal maxima."""
    logits = _cuda(logits, "logits")
    rows = logits.numel() // logits.shape[-1]
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    check(lib.ab2_argmax(logits.data_ptr(), rows, logits.shape[-1], dtype_code(logits.dtype), out.data_ptr(),
                         stream_ptr()))
    return out


def embedding_forward(table, ids: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    ids = _cuda(ids, "ids").to(torch.int32)
    out = torch.empty((*ids.shape, table.in_features), dtype=dtype, device=ids.device)
    check(lib.ab2_embedding_forward(table._h, ids.data_ptr(), ids.numel(), out.data_ptr(), dtype_code(dtype),
                                    stream_ptr()))
    return out
