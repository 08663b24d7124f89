"""Callers above the decoder: ragged batched decode of sessions that join and
leave (every live session in ONE forward, whatever rows they occupy), chunked
prefill, and the verification forward of speculative decoding - each against
the oracle's dense f32 model running the same sequence alone: greedy tokens
identical, logits within 1e-4 (f32 path) or 2e-2 (bf16 / INT8-KV path)."""
import numpy as np
import pytest
import torch

from helpers import pkg, rel_err
from model_fixtures import SMALL, build_pair
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _alone(cpu, ids, new_tokens):
    """Greedy tokens and per-step logits of one sequence on the oracle (one prefill, one-token steps)."""
    cpu.reset()
    lg = cpu.forward(np.array([ids]), [0])[0, -1]
    toks, logits = [], []
    for i in range(new_tokens):
        logits.append(lg.copy())
        toks.append(orc.argmax(lg))
        if i + 1 < new_tokens:
            lg = cpu.forward(np.array([[toks[-1]]]), [len(ids) + i])[0, 0]
    return toks, logits


def test_sessions_join_leave_and_decode_together():
    p = pkg()
    gpu, cpu, _ = build_pair(SMALL, "int8_channel", capacity=64)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, SMALL["vocab"], n).tolist() for n in (3, 17, 9, 6)]
    new = [10, 6, 12, 5]
    want = [_alone(cpu, ids, n) for ids, n in zip(prompts, new)]

    eng = p.sessions.SessionEngine(gpu, max_batch=3, capacity=SMALL["max_seq"])
    got = {i: ([], []) for i in range(4)}
    live = {}
    waiting = [0, 1, 2, 3]
    passes_with_a_gap = 0
    while waiting or live:
        while waiting and eng.free_rows:          # a fourth session joins when a row frees up
            i = waiting.pop(0)
            live[i] = eng.prepare_session_with_chunk_size(prompts[i], new[i], chunk_size=4)
        for i, s in list(live.items()):
            got[i][1].append(s.next_logits.float().cpu().numpy())
            got[i][0].append(eng.advance(s))
            if s.is_finished():
                eng.release(s)
                del live[i]
        rows = sorted(s.row for s in live.values())
        if len(rows) > 1 and rows[-1] - rows[0] + 1 > len(rows):
            passes_with_a_gap += 1                # e.g. rows {0, 2}: still one forward
        eng.decode_sessions(list(live.values()))
    assert passes_with_a_gap > 0
    for i in range(4):
        assert got[i][0] == want[i][0], i
        for a, b in zip(got[i][1], want[i][1]):
            assert rel_err(a, b) < 1e-4
    with pytest.raises(p.Ab2Error, match="chunk size must be greater than zero"):
        eng.prepare_session_with_chunk_size([1, 2], 4, chunk_size=0)
    with pytest.raises(p.Ab2Error, match="max_seq_len"):
        eng.prepare_session_with_chunk_size(list(range(SMALL["max_seq"])), 4)
    s = eng.prepare_session_with_chunk_size([1, 2, 3], 2)
    with pytest.raises(p.Ab2Error, match="no pending token"):
        eng.decode_sessions([s])


def test_speculative_verification_accepts_exactly_the_greedy_prefix():
    p = pkg()
    gpu, cpu, _ = build_pair(SMALL, "int8_channel", capacity=64)
    prompt = np.random.default_rng(9).integers(0, SMALL["vocab"], 8).tolist()
    toks, logits = _alone(cpu, prompt, 9)          # toks[0] follows the prompt, toks[i+1] follows toks[i]
    cache = gpu.empty_kv_cache_with_capacity(SMALL["max_seq"])
    gpu.forward_with_cache(torch.tensor([prompt]), 0, cache, last_only=True)
    base = len(prompt)
    # a draft that is right for 3 tokens and then wrong
    draft = toks[1:4] + [(toks[4] + 1) % SMALL["vocab"], 7]
    accepted, nxt, lg = p.sessions.verify_draft(gpu, cache, 0, base, toks[0], draft)
    assert accepted == 3 and nxt == toks[4]
    assert cache.seq_len(0) == base + 1 + 3
    for i in range(4):   # rows 0..3 of the verification forward are the one-token steps' logits
        assert rel_err(lg[i].float().cpu().numpy(), logits[i + 1]) < 1e-4
    # the row now continues exactly like the sequence decoded alone
    accepted2, nxt2, _ = p.sessions.verify_draft(gpu, cache, 0, base + 4, toks[4], toks[5:8])
    assert accepted2 == 3 and nxt2 == toks[8]
    with pytest.raises(p.Ab2Error, match="expected"):
        p.sessions.verify_draft(gpu, cache, 0, base, toks[0], draft)


@pytest.mark.parametrize("rows,lens", [([0, 2], [40, 7]), ([3, 1, 2], [300, 5, 64]), ([2], [20])])
def test_rows_in_any_order_decode_in_one_pass_on_the_w4a16_path(rows, lens):
    """Non-adjacent cache rows, in any order, through one forward (plain launches) and through
    the graph-replayed step (bf16, W4A16 weights, INT8 KV, head_dim 128: the row list reaches the
    append, the cluster / tensor-core attention and the length commit) against the oracle."""
    cfg = dict(SMALL, d_model=512, ffn_hidden=1024, n_heads=4, n_kv_heads=2, head_dim=128, n_layers=2, max_seq=512)
    gpu, cpu, _ = build_pair(cfg, "w4a16", dtype=torch.bfloat16, max_tokens=320, capacity=320)
    steps = 3
    seqs = [np.random.default_rng(50 + i).integers(0, cfg["vocab"], n + 2 * steps) for i, n in enumerate(lens)]
    refs = []
    for sq in seqs:
        cpu.reset()
        refs.append(cpu.forward(sq[None], [0])[0])
    cache = gpu.empty_kv_cache_with_capacity(320, batch=4, dtype="int8")
    for r, sq, n in zip(rows, seqs, lens):
        gpu.forward_with_cache(sq[None, :n], 0, cache, row=r)
    n_rows = len(rows)
    side = torch.cuda.Stream()
    logits = torch.empty((n_rows, cfg["vocab"]), dtype=torch.bfloat16, device="cuda")
    tok = torch.empty(n_rows, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    for s in range(2 * steps):
        ids = [int(sq[n + s]) for sq, n in zip(seqs, lens)]
        if s < steps:       # plain launches
            got = gpu.forward_decode_rows(torch.tensor(ids).view(-1, 1), rows, cache)[:, 0].float().cpu().numpy()
        else:               # graph-replayed steps
            with torch.cuda.stream(side):
                tok.copy_(torch.tensor(ids, dtype=torch.int32))
                gpu.decode_step_rows(tok, rows, cache, logits, None)
                side.synchronize()
            got = logits.float().cpu().numpy()
        for i, (r, n) in enumerate(zip(rows, lens)):
            assert rel_err(got[i], refs[i][n + s]) < 2e-2, (s, r)
            assert cache.seq_len(r) == n + s + 1
    assert pkg().device_status() == 0
    with pytest.raises(pkg().Ab2Error):
        gpu.forward_decode_rows(torch.tensor([[1], [2]]), [1, 1], cache)     # a row selected twice
