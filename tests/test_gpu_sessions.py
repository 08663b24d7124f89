"""Callers above the decoder: ragged batched decode of sessions that join and
leave, chunked prefill, and the verification forward of speculative decoding -
each against the same sequences run alone, token for token."""
import numpy as np
import pytest
import torch

from helpers import pkg, rel_err
from model_fixtures import SMALL, build_pair

pytestmark = pytest.mark.gpu


def _alone(gpu, ids, new_tokens):
    """Greedy tokens and per-step logits of one sequence on its own cache (one prefill, one-token steps)."""
    p = pkg()
    cache = gpu.empty_kv_cache_with_capacity(SMALL["max_seq"])
    lg = gpu.forward_with_cache(torch.tensor([ids]), 0, cache, last_only=True).view(1, -1)
    toks, logits = [], []
    for i in range(new_tokens):
        logits.append(lg.float().cpu().numpy().ravel())
        toks.append(int(p.dispatch.argmax(lg)[0]))
        if i + 1 < new_tokens:
            lg = gpu.forward_decode_batch(torch.tensor([[toks[-1]]]), [len(ids) + i], cache).view(1, -1)
    return toks, logits


def test_sessions_join_leave_and_decode_together():
    p = pkg()
    gpu, _, _ = build_pair(SMALL, "int8_channel", capacity=64)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, SMALL["vocab"], n).tolist() for n in (3, 17, 9, 6)]
    new = [10, 6, 12, 5]
    want = [_alone(gpu, ids, n) for ids, n in zip(prompts, new)]

    eng = p.sessions.SessionEngine(gpu, max_batch=3, capacity=SMALL["max_seq"])
    got = {i: ([], []) for i in range(4)}
    live = {}
    waiting = [0, 1, 2, 3]
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
        eng.decode_sessions(list(live.values()))
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
    gpu, _, _ = build_pair(SMALL, "int8_channel", capacity=64)
    prompt = np.random.default_rng(9).integers(0, SMALL["vocab"], 8).tolist()
    toks, logits = _alone(gpu, prompt, 9)          # toks[0] follows the prompt, toks[i+1] follows toks[i]
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
