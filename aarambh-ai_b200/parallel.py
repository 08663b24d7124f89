"""Tensor-parallel sharding of the decoder over the GPUs of one box.

One process per GPU.  ``TensorParallel`` wraps the library's NCCL communicator
(``ab2_tp_*``); the 128-byte unique id travels through ``torch.distributed``
(plumbing only).  The ``shard_*`` helpers are pure tensor slicing and define
which part of every weight a rank owns:

* column parallel (wq, wk, wv, w_gate, w_up, lm_head): a contiguous block of
  output rows of the ``[out, in]`` weight — whole heads for the attention
  projections, so the KV cache and the attention of a rank are local;
* row parallel (wo, w_down): a contiguous block of input columns, a multiple
  of the quantisation group so no group straddles two ranks; the partial
  outputs are summed by an all-reduce.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import replace

import torch

from . import _lib
from ._lib import check, lib

COLUMN_PARALLEL = ("wq", "wk", "wv", "w_gate", "w_up", "lm_head")
ROW_PARALLEL = ("wo", "w_down")


def shard_config(cfg, world: int):
    """The ModelConfig a rank builds its model with (local heads and FFN width)."""
    if cfg.n_heads % world or cfg.n_kv_heads % world or cfg.ffn_hidden % world or cfg.vocab_size % world:
        raise _lib.Ab2Error(-1, f"heads {cfg.n_heads}/{cfg.n_kv_heads}, ffn {cfg.ffn_hidden} and vocab "
                                f"{cfg.vocab_size} must be divisible by the world size {world}")
    return replace(cfg, n_heads=cfg.n_heads // world, n_kv_heads=cfg.n_kv_heads // world,
                   ffn_hidden=cfg.ffn_hidden // world)


def shard_rows(weight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Column-parallel shard: rows [rank * N/world, (rank + 1) * N/world) of [N, K]."""
    n = weight.shape[0]
    if n % world:
        raise _lib.Ab2Error(-1, f"{n} output rows are not divisible by {world}")
    step = n // world
    return weight[rank * step:(rank + 1) * step].contiguous()


def shard_cols(weight: torch.Tensor, rank: int, world: int, group: int = 128) -> torch.Tensor:
    """Row-parallel shard: input columns [rank * K/world, (rank + 1) * K/world) of [N, K]."""
    k = weight.shape[1]
    if k % world or (k // world) % group:
        raise _lib.Ab2Error(-1, f"{k} input columns do not split into {world} multiples of the group size {group}")
    step = k // world
    return weight[:, rank * step:(rank + 1) * step].contiguous()


def shard_weight(name: str, weight: torch.Tensor, rank: int, world: int, group: int = 128) -> torch.Tensor:
    """The part of tensor ``name`` (e.g. ``layers.3.wo``) that ``rank`` owns."""
    leaf = name.split(".")[-1]
    if world == 1 or weight.dim() != 2:
        return weight
    if leaf in COLUMN_PARALLEL:
        return shard_rows(weight, rank, world)
    if leaf in ROW_PARALLEL:
        return shard_cols(weight, rank, world, group)
    return weight  # embedding and norms are replicated


class TensorParallel:
    """The NCCL communicator of this process inside the library."""

    def __init__(self, rank: int, world: int, unique_id: bytes | None):
        self.rank, self.world = rank, world
        h = C.c_void_p()
        buf = C.create_string_buffer(unique_id, 128) if unique_id is not None else None
        check(lib.ab2_tp_create(C.byref(h), rank, world, buf))
        self._h = h

    @staticmethod
    def new_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(lib.ab2_tp_unique_id(buf))
        return buf.raw

    @classmethod
    def from_torch_distributed(cls, peer_exchange: bool = True, max_elems: int = 16 * 8192):
        """Rank 0 makes the id; it is broadcast over the default process group.  With
        `peer_exchange` the ranks also swap CUDA IPC handles so that the decoder's
        partial sums travel over NVLink peer memory instead of NCCL (up to
        `max_elems` sums per exchange: 16 tokens of d_model 8192 by default)."""
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        if world == 1:
            return cls(0, 1, None)
        ids = [cls.new_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        tp = cls(rank, world, ids[0])
        if peer_exchange and world <= 8 and os.environ.get("AB2_TP_NCCL_ONLY") is None:
            tp.attach_peers(max_elems)
        return tp

    def attach_peers(self, max_elems: int) -> None:
        """Exports this rank's inbox, gathers every rank's handle, attaches."""
        import torch.distributed as dist
        buf = C.create_string_buffer(64)
        check(lib.ab2_tp_peer_export(self._h, max_elems, buf))
        handles = [None] * self.world
        dist.all_gather_object(handles, buf.raw)
        check(lib.ab2_tp_peer_attach(self._h, C.create_string_buffer(b"".join(handles), 64 * self.world)))
        dist.barrier()

    # -- the peer exchange as a stand-alone one-shot all-reduce --------------------
    def export_block(self, max_elems: int):
        """Allocates this rank's inbox without an IPC handle and returns (device pointer, bytes)."""
        check(lib.ab2_tp_peer_export(self._h, max_elems, None))
        ptr, n = C.c_void_p(), C.c_size_t()
        check(lib.ab2_tp_peer_block(self._h, C.byref(ptr), C.byref(n)))
        return ptr.value, n.value

    def attach_blocks(self, block_ptrs) -> None:
        """Attaches by device pointers of every rank's block as this process sees them."""
        arr = (C.c_void_p * self.world)(*[int(b) if b else None for b in block_ptrs])
        check(lib.ab2_tp_peer_attach_ptrs(self._h, arr))

    def set_wait_limit_ns(self, ns: int) -> None:
        check(lib.ab2_tp_set_wait_limit_ns(self._h, int(ns)))

    def peer_reset(self) -> None:
        check(lib.ab2_tp_peer_reset(self._h))

    def peer_deposit(self, partial: torch.Tensor) -> None:
        from .qlinear import stream_ptr
        if partial.dtype != torch.float32 or not partial.is_contiguous():
            raise ValueError("partial sums must be a contiguous float32 tensor")
        check(lib.ab2_tp_peer_deposit(self._h, partial.data_ptr(), partial.numel(), stream_ptr()))

    def peer_reduce_add(self, x: torch.Tensor) -> torch.Tensor:
        from .qlinear import stream_ptr
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("the residual stream must be a contiguous bfloat16 tensor")
        check(lib.ab2_tp_peer_reduce_add(self._h, x.data_ptr(), x.numel(), stream_ptr()))
        return x

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        from .qlinear import dtype_code, stream_ptr
        check(lib.ab2_tp_all_reduce(self._h, t.data_ptr(), t.numel(), dtype_code(t.dtype), stream_ptr()))
        return t

    def __del__(self):
        try:
            if self._h:
                lib.ab2_tp_destroy(self._h)
                self._h = None
        except Exception:
            pass
