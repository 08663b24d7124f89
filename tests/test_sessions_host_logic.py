"""Host logic of the session callers (aarambh-ai_b200/sessions.py) without a GPU: a scripted
model and cache stand in for the decoder, the greedy pick is torch's last maximum.  What is
checked is the bookkeeping the reference's engine and batcher do around the model
(crates/aarambh-studio-inference/src/engine.rs:271-355, 822-976;
crates/aarambh-studio-inference/src/speculative.rs:304-318, 388-418): prefill in chunks at the
right offsets, one decode pass over the live rows in row order, pending tokens, the finish
conditions, rows given back, the error for every misuse, and the accepted prefix and cache
length after a draft verification."""
import pytest
import torch

from helpers import pkg


class FakeCache:
    def __init__(self, rows):
        self.lens = [0] * rows

    def truncate(self, n, row=0):
        assert n <= self.lens[row] or n == 0
        self.lens[row] = n

    def seq_len(self, row=0):
        return self.lens[row]


class FakeModel:
    """Logits put the maximum at (last token + 1) % vocab; every call is recorded."""

    class Cfg:
        max_seq_len = 64
        vocab_size = 32

    def __init__(self):
        self.cfg = self.Cfg()
        self.calls = []

    def empty_kv_cache_with_capacity(self, capacity, batch=1, dtype="f32"):
        self.cache = FakeCache(batch)
        return self.cache

    def _logits(self, tokens):
        out = torch.zeros(len(tokens), self.cfg.vocab_size)
        for i, t in enumerate(tokens):
            out[i, (int(t) + 1) % self.cfg.vocab_size] = 1.0
        return out

    def forward_with_cache(self, ids, offset, cache, row=0, last_only=False):
        ids = [int(t) for t in ids[0]]
        assert cache.lens[row] == offset, "a chunk starts where the row's cache ends"
        cache.lens[row] += len(ids)
        self.calls.append(("prefill", row, offset, len(ids)))
        lg = self._logits(ids)
        return lg[-1:].view(1, 1, -1) if last_only else lg.view(1, len(ids), -1)

    def forward_decode_rows(self, ids, rows, cache):
        self.calls.append(("decode", list(rows), [int(t) for t in ids[:, 0]]))
        for r in rows:
            cache.lens[r] += 1
        return self._logits([int(t) for t in ids[:, 0]]).view(len(rows), 1, -1)


@pytest.fixture
def sessions(monkeypatch):
    mod = pkg().sessions

    def last_max(logits):
        v = logits.float()
        return (v.shape[-1] - 1 - torch.flip(v, [-1]).argmax(-1)).to(torch.int32)

    monkeypatch.setattr(mod, "argmax", last_max)
    return mod


def test_prefill_runs_in_chunks_at_consecutive_offsets(sessions):
    model = FakeModel()
    eng = sessions.SessionEngine(model, max_batch=2, capacity=48)
    s = eng.prepare_session_with_chunk_size(list(range(1, 12)), max_new_tokens=100, chunk_size=4)
    assert model.calls == [("prefill", 0, 0, 4), ("prefill", 0, 4, 4), ("prefill", 0, 8, 3)]
    assert (s.row, s.prompt_len) == (0, 11)
    assert s.max_new_tokens == 48 - 11, "new tokens are capped by the room left in the sequence"
    assert int(torch.argmax(s.next_logits)) == 12


def test_two_sessions_decode_in_one_pass_in_row_order_until_they_finish(sessions):
    model = FakeModel()
    eng = sessions.SessionEngine(model, max_batch=3, capacity=32)
    a = eng.prepare_session_with_chunk_size([5, 6], max_new_tokens=2)
    b = eng.prepare_session_with_chunk_size([9], max_new_tokens=4, eos_token_id=12)
    assert (a.row, b.row) == (0, 1)
    assert eng.advance(a) == 7 and eng.advance(b) == 10
    assert a.pending_token == 7 and b.pending_token == 10
    model.calls.clear()
    eng.decode_sessions([b, a])                       # any order in, row order through the model
    assert model.calls == [("decode", [0, 1], [7, 10])]
    assert a.pending_token is None and b.pending_token is None
    assert eng.advance(a) == 8 and a.finished, "max_new_tokens reached"
    assert a.pending_token is None and eng.advance(a) is None
    assert eng.advance(b) == 11 and not b.finished
    eng.decode_sessions([b])
    assert eng.advance(b) == 12 and b.finished, "the end-of-sequence token finishes the session"
    assert b.generated_ids == [10, 11, 12]
    eng.release(a)
    c = eng.prepare_session_with_chunk_size([1], max_new_tokens=1)
    assert c.row == 0 and model.cache.seq_len(0) == 1, "a released row is reused from empty"


def test_misuse_is_refused_with_the_engines_errors(sessions):
    err = pkg().Ab2Error
    model = FakeModel()
    eng = sessions.SessionEngine(model, max_batch=1, capacity=16)
    with pytest.raises(err, match="chunk size"):
        eng.prepare_session_with_chunk_size([1], 4, chunk_size=0)
    with pytest.raises(err, match="must not be empty"):
        eng.prepare_session_with_chunk_size([], 4)
    with pytest.raises(err, match="max_seq_len"):
        eng.prepare_session_with_chunk_size(list(range(16)), 4)
    s = eng.prepare_session_with_chunk_size([1, 2, 3], 4)
    with pytest.raises(err, match="every row"):
        eng.prepare_session_with_chunk_size([1], 4)
    with pytest.raises(err, match="no pending token"):
        eng.decode_sessions([s])
    eng.advance(s)
    model.cache.lens[s.row] += 1                      # the cache and the session disagree
    with pytest.raises(err, match="the session expects"):
        eng.decode_sessions([s])
    model.cache.lens[s.row] -= 1
    eng.decode_sessions([s])
    eng.release(s)
    with pytest.raises(err, match="finished session"):
        eng.decode_sessions([s])
    eng.decode_sessions([])                           # nothing to do is not an error


def test_draft_verification_keeps_the_accepted_prefix(sessions):
    model = FakeModel()
    cache = model.empty_kv_cache_with_capacity(32, 1)
    model.forward_with_cache(torch.tensor([[3, 4, 5]]), 0, cache)
    # the target continues t -> t + 1: after pending 6 it wants 7, 8, 9, ...
    accepted, nxt, logits = sessions.verify_draft(model, cache, 0, 3, 6, [7, 8, 20, 21])
    assert (accepted, nxt) == (2, 9), "draft tokens are accepted while they equal the target's greedy choice"
    assert cache.seq_len(0) == 3 + 1 + 2, "pending token + accepted draft tokens stay in the cache"
    assert tuple(logits.shape) == (5, model.cfg.vocab_size)
    accepted, nxt, _ = sessions.verify_draft(model, cache, 0, 6, 9, [10, 11])
    assert (accepted, nxt) == (2, 12) and cache.seq_len(0) == 9
    accepted, nxt, _ = sessions.verify_draft(model, cache, 0, 9, 12, [])
    assert (accepted, nxt) == (0, 13) and cache.seq_len(0) == 10
    with pytest.raises(pkg().Ab2Error, match="expected"):
        sessions.verify_draft(model, cache, 0, 4, 1, [2])
