"""Host-side mirror of the reference's model and engine entry points for the
dense grouped-query decoder: ``AarambhModel.forward_with_cache`` /
``forward_decode_batch`` / ``empty_kv_cache_with_capacity``
(crates/aarambh-studio-model/src/model.rs:508-662) and the greedy loop of
``InferenceEngine.generate_from_token_ids`` (crates/aarambh-studio-inference/src/
engine.rs:423-467) with ``Sampler`` argmax (sampler.rs:217-224).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import ModelConfig as _CConfig, check, lib
from .kvcache import KVCache
from .qlinear import QuantLinear, dtype_code, stream_ptr

LAYER_LINEARS = ["wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down"]


@dataclass
class ModelConfig:
    """The ModelConfig fields this path uses (crates/aarambh-studio-core/src/config.rs:734-868)."""
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn_hidden: int
    vocab_size: int
    max_seq_len: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_embeddings: bool = True

    @classmethod
    def tiny_class(cls):
        return cls(6, 384, 6, 2, 64, 1024, 8192, 512)

    @classmethod
    def large_class(cls):
        return cls(32, 4096, 32, 8, 128, 14336, 32000, 1024, tie_embeddings=False)


class AarambhModel:
    """weights: name -> QuantLinear for ``embedding``, optional ``lm_head`` and
    ``layers.{i}.{wq,wk,wv,wo,w_gate,w_up,w_down}``; name -> f32 tensor for
    ``final_norm`` and ``layers.{i}.{norm1,norm2}``."""

    def __init__(self, cfg: ModelConfig, weights: dict, dtype: torch.dtype = torch.float32,
                 max_tokens: int = 512, tp=None):
        """With ``tp`` (a ``parallel.TensorParallel``), ``cfg`` and ``weights`` are
        this rank's shard (``parallel.shard_config`` / ``shard_weight``)."""
        self.cfg, self.dtype, self.weights, self.tp = cfg, dtype, weights, tp
        c = _CConfig(cfg.n_layers, cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn_hidden,
                     cfg.vocab_size, cfg.max_seq_len, cfg.rms_norm_eps, cfg.rope_theta,
                     1 if cfg.tie_embeddings else 0)
        h = C.c_void_p()
        check(lib.ab2_model_create(C.byref(h), C.byref(c), dtype_code(dtype), max_tokens))
        self._h = h
        if tp is not None:
            check(lib.ab2_model_set_tp(self._h, tp._h))
        check(lib.ab2_model_set_linear(self._h, -1, 0, weights["embedding"]._h))
        if "lm_head" in weights:
            check(lib.ab2_model_set_linear(self._h, -1, 1, weights["lm_head"]._h))
        self._norm(-1, 0, weights["final_norm"])
        for l in range(cfg.n_layers):
            for which, name in enumerate(LAYER_LINEARS):
                check(lib.ab2_model_set_linear(self._h, l, which, weights[f"layers.{l}.{name}"]._h))
            self._norm(l, 0, weights[f"layers.{l}.norm1"])
            self._norm(l, 1, weights[f"layers.{l}.norm2"])
        check(lib.ab2_model_finalize(self._h))

    def _norm(self, layer, which, w):
        w = w.detach().to(torch.float32).contiguous()
        check(lib.ab2_model_set_norm(self._h, layer, which, w.data_ptr()))

    def empty_kv_cache_with_capacity(self, capacity: int, batch: int = 1, dtype: str = "f32") -> KVCache:
        c = self.cfg
        return KVCache(capacity, c.n_kv_heads, c.head_dim, c.n_heads, batch, c.n_layers, dtype)

    def _ids(self, token_ids):
        ids = token_ids if isinstance(token_ids, torch.Tensor) else torch.tensor(token_ids)
        if ids.dim() != 2:
            raise _lib.Ab2Error(-1, f"token ids must have shape [batch, seq], got {list(ids.shape)}")
        if int(ids.max()) >= self.cfg.vocab_size or int(ids.min()) < 0:
            raise _lib.Ab2Error(-1, "token id outside the vocabulary")
        return ids.to(device="cuda", dtype=torch.int32).contiguous()

    def forward_with_cache(self, token_ids, seqlen_offset: int, cache: KVCache, row: int = 0,
                           last_only: bool = False) -> torch.Tensor:
        """ids [1, S] -> logits [1, S, vocab] (or [1, 1, vocab] with last_only)."""
        ids = self._ids(token_ids)
        if ids.shape[0] != 1:
            raise _lib.Ab2Error(-1, "forward_with_cache takes one sequence")
        S = ids.shape[1]
        out = torch.empty((1, 1 if last_only else S, self.cfg.vocab_size), dtype=self.dtype, device="cuda")
        offs = (C.c_int * 1)(seqlen_offset)
        check(lib.ab2_model_forward(self._h, cache._h, ids.data_ptr(), S, row, 1, offs, 1 if last_only else 2,
                                    out.data_ptr(), None, stream_ptr()))
        return out

    def forward_decode_batch(self, token_ids, seqlen_offsets, cache: KVCache, row0: int = 0) -> torch.Tensor:
        """ids [B, 1], offsets [B] -> logits [B, 1, vocab]."""
        ids = self._ids(token_ids)
        if ids.shape[1] != 1:
            raise _lib.Ab2Error(-1, f"batched decode token ids must have shape [batch, 1], got {list(ids.shape)}")
        B = ids.shape[0]
        if len(seqlen_offsets) != B:
            raise _lib.Ab2Error(-1, f"batched decode received batch {B} and {len(seqlen_offsets)} offsets")
        out = torch.empty((B, 1, self.cfg.vocab_size), dtype=self.dtype, device="cuda")
        offs = (C.c_int * B)(*[int(o) for o in seqlen_offsets])
        check(lib.ab2_model_forward(self._h, cache._h, ids.data_ptr(), 1, row0, B, offs, 1, out.data_ptr(), None,
                                    stream_ptr()))
        return out

    def forward_decode_rows(self, token_ids, rows, cache: KVCache) -> torch.Tensor:
        """One token for each of an arbitrary set of cache rows in ONE forward: ids [n, 1],
        rows [n] distinct cache rows; positions are the rows' cache lengths -> logits [n, 1, vocab]."""
        ids = self._ids(token_ids)
        rows = [int(r) for r in rows]
        if ids.shape[1] != 1 or ids.shape[0] != len(rows):
            raise _lib.Ab2Error(-1, f"expected ids [{len(rows)}, 1], got {list(ids.shape)}")
        n = len(rows)
        out = torch.empty((n, 1, self.cfg.vocab_size), dtype=self.dtype, device="cuda")
        check(lib.ab2_model_forward_rows(self._h, cache._h, ids.data_ptr(), 1, (C.c_int * n)(*rows), n, 1,
                                         out.data_ptr(), None, stream_ptr()))
        return out

    def decode_step_rows(self, ids_dev: torch.Tensor, rows, cache: KVCache, logits: torch.Tensor | None,
                         argmax_dev: torch.Tensor | None):
        """Graph-replayed one-token step over an arbitrary set of cache rows (ids_dev [n] int32)."""
        rows = [int(r) for r in rows]
        n = len(rows)
        check(lib.ab2_model_decode_step_rows(self._h, cache._h, ids_dev.data_ptr(), (C.c_int * n)(*rows), n,
                                             logits.data_ptr() if logits is not None else None,
                                             argmax_dev.data_ptr() if argmax_dev is not None else None, stream_ptr()))

    def decode_step(self, ids_dev: torch.Tensor, cache: KVCache, logits: torch.Tensor | None,
                    argmax_dev: torch.Tensor | None, row0: int = 0):
        """Graph-replayed one-token step; ids_dev [B] int32 is read on the device."""
        check(lib.ab2_model_decode_step(self._h, cache._h, ids_dev.data_ptr(), row0, ids_dev.numel(),
                                        logits.data_ptr() if logits is not None else None,
                                        argmax_dev.data_ptr() if argmax_dev is not None else None, stream_ptr()))

    def decode_step_host(self, ids_host: torch.Tensor, cache: KVCache, out_host: torch.Tensor, row0: int = 0):
        """One greedy step with the tokens in host memory: ids_host [B] int32 in, out_host [B] int32
        out (pinned tensors make both copies asynchronous); returns when out_host is filled."""
        if ids_host.is_cuda or out_host.is_cuda or ids_host.dtype != torch.int32 or out_host.dtype != torch.int32:
            raise _lib.Ab2Error(-1, "decode_step_host takes int32 host tensors")
        if out_host.numel() < ids_host.numel() or not ids_host.is_contiguous() or not out_host.is_contiguous():
            raise _lib.Ab2Error(-1, "out_host must be contiguous and hold one token per row")
        check(lib.ab2_model_decode_step_host(self._h, cache._h, ids_host.data_ptr(), row0, ids_host.numel(),
                                             out_host.data_ptr(), stream_ptr()))

    def step_trace(self):
        """Phase timestamps (ns) of the last persistent one-row decode step as an int64
        array [3 CTAs, phases, 10]: phase start, prologue done, CTA done, barrier passed, then
        up to six points inside the phase (0 where unused)."""
        import numpy as np
        n = C.c_int(0)
        buf = np.zeros(3 * 4096 * 10, np.uint64)
        check(lib.ab2_model_step_trace(self._h, buf.ctypes.data, buf.size, C.byref(n)))
        return buf[:3 * n.value * 10].astype(np.int64).reshape(3, n.value, 10)

    def __del__(self):
        try:
            if self._h:
                lib.ab2_model_destroy(self._h)
                self._h = None
        except Exception:
            pass


class InferenceEngine:
    """Greedy generation from raw token ids, at model level: exactly
    ``max_new_tokens`` steps, no end-of-text stop (the reference engine stops on
    token 0, crates/aarambh-studio-inference/src/engine.rs:898-911; ``eos_step``
    reports where it would have)."""

    def __init__(self, model: AarambhModel, kv_dtype: str = "f32"):
        self.model, self.kv_dtype = model, kv_dtype

    def generate_from_token_ids(self, prompt_ids, max_new_tokens: int, eos_token_id: int = 0,
                                on_device_sampling: bool = True):
        m = self.model
        prompt = torch.as_tensor(prompt_ids, dtype=torch.int64).view(1, -1)
        P = prompt.shape[1]
        if P + max_new_tokens > m.cfg.max_seq_len:
            raise _lib.Ab2Error(-1, "prompt plus new tokens exceed max_seq_len")
        cache = m.empty_kv_cache_with_capacity(P + max_new_tokens, 1, self.kv_dtype)
        from .dispatch import argmax
        stream = torch.cuda.Stream()   # a capturable (non-default) stream for the graph-replayed steps
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            logits = m.forward_with_cache(prompt, 0, cache, last_only=True)
            tokens = torch.empty(max_new_tokens, dtype=torch.int32, device="cuda")
            tokens[0:1] = argmax(logits.view(1, -1))
            if on_device_sampling:
                # two token buffers alternate as input and output, so two graphs
                # serve every step and no token visits the host
                bufs = [tokens[0:1].clone(), torch.empty(1, dtype=torch.int32, device="cuda")]
                for i in range(1, max_new_tokens):
                    m.decode_step(bufs[(i - 1) % 2], cache, None, bufs[i % 2])
                    tokens[i:i + 1].copy_(bufs[i % 2])
            else:
                for i in range(1, max_new_tokens):
                    lg = m.forward_decode_batch(tokens[i - 1:i].view(1, 1), [P + i - 1], cache)
                    tokens[i:i + 1] = argmax(lg.view(1, -1))
        torch.cuda.current_stream().wait_stream(stream)
        stream.synchronize()
        out = tokens.cpu().tolist()
        eos_step = next((i for i, t in enumerate(out) if t == eos_token_id), None)
        return {"token_ids": out, "eos_step": eos_step, "cache": cache}
