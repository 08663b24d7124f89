"""Host-side mirror of the reference's KV caches.

``KVCache`` follows ``KVCache`` of crates/aarambh-studio-nn/src/kvcache.rs:236-369
(update / truncate / clear / seq_len / capacity) for ``batch`` independent
sequences, and with ``n_layers > 1`` the engine-level ``KvCache`` of
crates/aarambh-studio-inference/src/kvcache.rs:7-80 (one length shared by all
layers, snapshot / restore).  Storage is f32, bf16 or per-token-per-head INT8.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import check, lib
from .qlinear import dtype_code, stream_ptr

_KV_DTYPES = {"f32": _lib.KV_F32, "bf16": _lib.KV_BF16, "int8": _lib.KV_INT8}


class KVCache:
    def __init__(self, capacity: int, kv_heads: int, head_dim: int, n_heads: int, batch: int = 1,
                 n_layers: int = 1, dtype: str = "f32", _handle=None):
        self.cap, self.kv_heads, self.head_dim, self.n_heads = capacity, kv_heads, head_dim, n_heads
        self.batch, self.n_layers, self.dtype = batch, n_layers, dtype
        if _handle is None:
            h = C.c_void_p()
            check(lib.ab2_kv_create(C.byref(h), n_layers, batch, capacity, kv_heads, head_dim, n_heads,
                                    _KV_DTYPES[dtype]))
            _handle = h.value
        self._h = C.c_void_p(_handle)

    @classmethod
    def with_capacity(cls, capacity, kv_heads, head_dim, n_heads, **kw):
        return cls(capacity, kv_heads, head_dim, n_heads, **kw)

    def update(self, k: torch.Tensor, v: torch.Tensor, row0: int = 0):
        """Appends k, v [rows, S, kv_heads, head_dim] and returns the cached tensors
        of the first row touched, dequantised ([len, kv_heads, head_dim])."""
        if k.dim() != 4 or v.shape != k.shape:
            raise _lib.Ab2Error(-1, f"KV cache expects matching rank-4 tensors, got {tuple(k.shape)} and {tuple(v.shape)}")
        k = k.contiguous(); v = v.contiguous()
        check(lib.ab2_kv_update(self._h, k.data_ptr(), v.data_ptr(), k.shape[1], row0, k.shape[0],
                                dtype_code(k.dtype), stream_ptr()))
        return self.read(row0)

    def append(self, layer, k, v, row0=0, cos=None, sin=None, positions=None, max_seq=0):
        k = k.contiguous(); v = v.contiguous()
        check(lib.ab2_kv_append(self._h, layer, k.data_ptr(), v.data_ptr(), k.shape[1], row0, k.shape[0],
                                dtype_code(k.dtype), cos.data_ptr() if cos is not None else None,
                                sin.data_ptr() if sin is not None else None,
                                positions.data_ptr() if positions is not None else None, max_seq,
                                stream_ptr()))

    def commit(self, S, row0=0, nrows=None):
        check(lib.ab2_kv_commit(self._h, S, row0, self.batch - row0 if nrows is None else nrows, stream_ptr()))

    def read(self, row: int = 0, layer: int = 0):
        n = self.seq_len(row)
        k = torch.empty((n, self.kv_heads, self.head_dim), dtype=torch.float32, device="cuda")
        v = torch.empty_like(k)
        check(lib.ab2_kv_read(self._h, layer, row, k.data_ptr(), v.data_ptr(), stream_ptr()))
        return k, v

    def truncate(self, new_len: int, row: int = 0):
        check(lib.ab2_kv_truncate(self._h, row, new_len, stream_ptr()))

    def clear(self):
        check(lib.ab2_kv_clear(self._h, stream_ptr()))

    def seq_len(self, row: int = 0) -> int:
        n = C.c_int()
        check(lib.ab2_kv_seq_len(self._h, row, C.byref(n)))
        return n.value

    def capacity(self) -> int:
        n = C.c_int()
        check(lib.ab2_kv_capacity(self._h, C.byref(n)))
        return n.value

    def snapshot(self) -> "KVCache":
        h = C.c_void_p()
        check(lib.ab2_kv_clone(C.byref(h), self._h, stream_ptr()))
        return KVCache(self.cap, self.kv_heads, self.head_dim, self.n_heads, self.batch, self.n_layers,
                       self.dtype, _handle=h.value)

    def restore(self, snapshot: "KVCache"):
        """Takes over the snapshot's storage (KvCache::restore)."""
        old = self._h
        self._h, snapshot._h = snapshot._h, None
        lib.ab2_kv_destroy(old)

    def __del__(self):
        try:
            if self._h:
                lib.ab2_kv_destroy(self._h)
                self._h = None
        except Exception:
            pass
