"""Tensor-parallel decoder against the single-GPU decoder (needs 2 GPUs; skipped
otherwise): same seeded weights, sharded over 2 ranks, logits within 1e-2
relative and the same greedy tokens - once with the partial sums exchanged over
NVLink peer memory, once through NCCL; plain launches, graph-replayed steps,
three rows decoded together and a 20-token prompt."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

CFG = dict(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn_hidden=1024, vocab=2048, max_seq=64)
SHAPES = {"wq": (512, 512), "wk": (256, 512), "wv": (256, 512), "wo": (512, 512), "w_gate": (1024, 512),
          "w_up": (1024, 512), "w_down": (512, 1024)}


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _build(pkg, rank, world, tp):
    gen = torch.Generator(device="cuda").manual_seed(11)

    def dense(shape):
        return torch.randn(shape, generator=gen, device="cuda") * 0.05

    def pack(name, w):
        return pkg.QuantLinear.quantise(pkg.parallel.shard_weight(name, w, rank, world), "w4a16", 128)

    weights = {"embedding": pack("embedding", dense((CFG["vocab"], CFG["d_model"]))),
               "lm_head": pack("lm_head", dense((CFG["vocab"], CFG["d_model"]))),
               "final_norm": torch.ones(CFG["d_model"], device="cuda")}
    for l in range(CFG["n_layers"]):
        for n, s in SHAPES.items():
            weights[f"layers.{l}.{n}"] = pack(f"layers.{l}.{n}", dense(s))
        weights[f"layers.{l}.norm1"] = torch.ones(CFG["d_model"], device="cuda")
        weights[f"layers.{l}.norm2"] = torch.ones(CFG["d_model"], device="cuda")
    cfg = pkg.ModelConfig(CFG["n_layers"], CFG["d_model"], CFG["n_heads"], CFG["n_kv_heads"], CFG["head_dim"],
                          CFG["ffn_hidden"], CFG["vocab"], CFG["max_seq"], 1e-5, 10000.0, False)
    if world > 1:
        cfg = pkg.parallel.shard_config(cfg, world)
    return pkg.AarambhModel(cfg, weights, dtype=torch.bfloat16, max_tokens=32, tp=tp)


def _run(model, steps=6):
    ids = torch.tensor([[3, 99, 1500, 7, 42]])
    cache = model.empty_kv_cache_with_capacity(32, dtype="int8")
    logits = [model.forward_with_cache(ids, 0, cache, last_only=True).float().cpu().numpy().ravel()]
    toks = [int(np.argmax(logits[0]))]
    for i in range(steps):
        lg = model.forward_decode_batch(torch.tensor([[toks[-1]]]), [5 + i], cache).float().cpu().numpy().ravel()
        logits.append(lg)
        toks.append(int(np.argmax(lg)))
    # the graph-replayed step on a side stream
    side = torch.cuda.Stream()
    out = torch.empty((1, CFG["vocab"]), dtype=torch.bfloat16, device="cuda")
    tok = torch.empty(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    for i in range(steps):
        with torch.cuda.stream(side):
            tok.fill_(toks[-1])
            model.decode_step(tok, cache, out, None)
            side.synchronize()
        lg = out.float().cpu().numpy().ravel()
        logits.append(lg)
        toks.append(int(np.argmax(lg)))
    # three rows decoded together (2..16 tokens per step: the stand-alone reduce over the inboxes)
    rows = 3
    bcache = model.empty_kv_cache_with_capacity(32, batch=rows, dtype="int8")
    for b in range(rows):
        model.forward_with_cache(ids[:, :3 + b], 0, bcache, row=b, last_only=True)
    bout = torch.empty((rows, CFG["vocab"]), dtype=torch.bfloat16, device="cuda")
    btok = torch.tensor([11, 600, 1999], dtype=torch.int32, device="cuda")
    for i in range(3):
        with torch.cuda.stream(side):
            model.decode_step(btok, bcache, bout, None)
            side.synchronize()
        logits.extend(bout.float().cpu().numpy())
    # a 20-token prompt (more than 16 tokens: partial sums through the collective library, the
    # SwiGLU and f32 epilogues of the 9..32-token GEMM)
    long_ids = torch.randint(0, CFG["vocab"], (1, 20), generator=torch.Generator().manual_seed(5))
    lcache = model.empty_kv_cache_with_capacity(32, dtype="int8")
    logits.append(model.forward_with_cache(long_ids, 0, lcache, last_only=True).float().cpu().numpy().ravel())
    return np.stack(logits), toks


def _worker(rank, world, port, out, peer):
    import torch.distributed as dist
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from __graft_entry__ import import_package
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        pkg = import_package()
        tp = pkg.TensorParallel.from_torch_distributed(peer_exchange=peer)
        logits, toks = _run(_build(pkg, rank, world, tp))
        if rank == 0:
            ref_logits, ref_toks = _run(_build(pkg, 0, 1, None))
            err = float(np.abs(logits - ref_logits).max() / np.abs(ref_logits).max())
            out.put(("result", err, toks, ref_toks, pkg.device_status()))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        out.put(("error", rank, repr(e)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("peer", [True, False])
def test_tp2_matches_single_gpu(peer):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out, peer)) for r in range(2)]
    for p in procs:
        p.start()
    msg = out.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
    assert msg[0] == "result", msg
    _, err, toks, ref_toks, status = msg
    assert status == 0
    assert err < 1e-2, err
    assert toks == ref_toks
