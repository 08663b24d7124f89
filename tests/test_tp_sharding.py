"""Tensor-parallel sharding rules on CPU ranks (gloo, world size 2): the shards
the helpers hand out reassemble the unsharded block exactly as the decoder
uses them — column-parallel outputs concatenate, row-parallel partial sums
all-reduce to the full projection, heads stay whole."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import pkg


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        par = pkg().parallel
        cfg = pkg().ModelConfig(2, 256, 4, 2, 64, 512, 1024, 64)
        local = par.shard_config(cfg, world)
        assert (local.n_heads, local.n_kv_heads, local.ffn_hidden, local.d_model) == (2, 1, 256, 256)
        gen = torch.Generator().manual_seed(7)       # same full weights on every rank
        full = {n: torch.randn(s, generator=gen) for n, s in {
            "layers.0.wq": (256, 256), "layers.0.wk": (128, 256), "layers.0.wo": (256, 256),
            "layers.0.w_gate": (512, 256), "layers.0.w_up": (512, 256), "layers.0.w_down": (256, 512),
            "lm_head": (1024, 256), "embedding": (1024, 256), "layers.0.norm1": (256,)}.items()}
        mine = {n: par.shard_weight(n, w, rank, world) for n, w in full.items()}
        assert mine["embedding"].shape == (1024, 256) and mine["layers.0.norm1"].shape == (256,)
        assert mine["layers.0.wk"].shape == (64, 256)          # one whole kv head per rank
        x = torch.randn(3, 256, generator=gen)
        # column parallel: gather of the shards' outputs == full projection
        q_local = x @ mine["layers.0.wq"].T
        gathered = [torch.empty_like(q_local) for _ in range(world)]
        dist.all_gather(gathered, q_local)
        assert torch.allclose(torch.cat(gathered, 1), x @ full["layers.0.wq"].T, atol=1e-5)
        # gate/up (column) feeding down (row): SwiGLU is element-wise, so it stays local,
        # and the row-parallel partial sums all-reduce to the full FFN output
        h_local = torch.nn.functional.silu(x @ mine["layers.0.w_gate"].T) * (x @ mine["layers.0.w_up"].T)
        y = h_local @ mine["layers.0.w_down"].T
        dist.all_reduce(y)
        h_full = torch.nn.functional.silu(x @ full["layers.0.w_gate"].T) * (x @ full["layers.0.w_up"].T)
        assert torch.allclose(y, h_full @ full["layers.0.w_down"].T, atol=1e-3)
        # attention output (heads local) into the row-parallel O projection
        a_full = torch.randn(3, 256, generator=gen)
        a_local = a_full[:, rank * 128:(rank + 1) * 128]
        o = a_local @ mine["layers.0.wo"].T
        dist.all_reduce(o)
        assert torch.allclose(o, a_full @ full["layers.0.wo"].T, atol=1e-3)
        # a split that would cut a quantisation group is refused
        with pytest.raises(pkg().Ab2Error):
            par.shard_cols(torch.zeros(8, 192), rank, world, group=128)
        out.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_shards_reassemble_under_gloo_world_2():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results
