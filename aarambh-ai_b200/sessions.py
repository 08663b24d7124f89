"""The callers one step above the decoder, at token-id level: chunked prefill
and ragged batched decode of independent generation sessions
(``InferenceEngine::{prepare_session_with_chunk_size, decode_sessions}``,
crates/aarambh-studio-inference/src/engine.rs:271-355, driven by the serving
batcher, crates/aarambh-studio-serve/src/batching.rs:314-461), and the target-side
verification forward of speculative decoding
(crates/aarambh-studio-inference/src/speculative.rs:304-318,388-418).

Sessions live in the rows of ONE batched KV cache; a decode pass over sessions
with different lengths is ONE forward over the list of their rows, whatever rows
they occupy (per-row lengths, one attention launch for all of them), where the
reference loops over rows.  Sampling here is greedy (last maximum, as ``argmax`` in
sampler.rs:217-224); text, tools and stochastic samplers stay with the caller.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import _lib
from .dispatch import argmax
from .model import AarambhModel


@dataclass
class GenerationSession:
    row: int
    prompt_len: int
    max_new_tokens: int
    next_logits: torch.Tensor                 # [vocab], logits of the next position
    generated_ids: list = field(default_factory=list)
    pending_token: int | None = None
    eos_token_id: int | None = None
    finished: bool = False

    def is_finished(self) -> bool:
        return self.finished


class SessionEngine:
    """Up to ``max_batch`` concurrent sessions over one model (the serving
    batcher's default is 8, prefill chunks of 128 tokens; batching.rs:35-52)."""

    def __init__(self, model: AarambhModel, max_batch: int = 8, capacity: int | None = None, kv_dtype: str = "f32"):
        self.model = model
        self.capacity = capacity or model.cfg.max_seq_len
        self.cache = model.empty_kv_cache_with_capacity(self.capacity, max_batch, kv_dtype)
        self.free_rows = list(range(max_batch))

    # -- engine.rs:271-318 ---------------------------------------------------
    def prepare_session_with_chunk_size(self, prompt_ids, max_new_tokens: int, chunk_size: int = 128,
                                        eos_token_id: int | None = None) -> GenerationSession:
        if chunk_size <= 0:
            raise _lib.Ab2Error(-1, "prefill chunk size must be greater than zero")
        ids = [int(t) for t in prompt_ids]
        if not ids:
            raise _lib.Ab2Error(-1, "prompt ids must not be empty")
        max_seq = min(self.model.cfg.max_seq_len, self.capacity)
        if len(ids) >= max_seq:
            raise _lib.Ab2Error(-1, f"prompt has {len(ids)} tokens but model max_seq_len is {max_seq}")
        if not self.free_rows:
            raise _lib.Ab2Error(-1, "every row of the batch holds a session")
        row = self.free_rows.pop(0)
        self.cache.truncate(0, row)
        logits = None
        for off in range(0, len(ids), chunk_size):
            chunk = torch.tensor([ids[off:off + chunk_size]])
            logits = self.model.forward_with_cache(chunk, off, self.cache, row=row, last_only=True)
        return GenerationSession(row, len(ids), min(max_new_tokens, max_seq - len(ids)), logits.view(-1),
                                 eos_token_id=eos_token_id)

    # -- GenerationSession::advance, greedy (engine.rs:822-976) ---------------
    def advance(self, session: GenerationSession) -> int | None:
        """Samples the next token from ``next_logits``; it becomes the pending
        token of the next decode pass.  Returns it, or None once finished."""
        if session.finished:
            return None
        token = int(argmax(session.next_logits.view(1, -1))[0])
        session.generated_ids.append(token)
        if len(session.generated_ids) >= session.max_new_tokens or token == session.eos_token_id:
            session.finished = True
            session.pending_token = None
        else:
            session.pending_token = token
        return token

    # -- engine.rs:323-355 -----------------------------------------------------
    def decode_sessions(self, sessions) -> None:
        """One shared decode pass: every session's pending token goes through the
        model at its own offset; ``next_logits`` of each is replaced."""
        if not sessions:
            return
        for s in sessions:
            if s.finished:
                raise _lib.Ab2Error(-1, "finished session cannot enter a decode batch")
            if s.pending_token is None:
                raise _lib.Ab2Error(-1, "session has no pending token for batched decode")
        ordered = sorted(sessions, key=lambda s: s.row)
        for s in ordered:
            expect = s.prompt_len + len(s.generated_ids) - 1
            if self.cache.seq_len(s.row) != expect:
                raise _lib.Ab2Error(-1, f"cache row {s.row} holds {self.cache.seq_len(s.row)} tokens, the session expects {expect}")
        ids = torch.tensor([[s.pending_token] for s in ordered])
        logits = self.model.forward_decode_rows(ids, [s.row for s in ordered], self.cache)
        for i, s in enumerate(ordered):
            s.next_logits = logits[i, 0]
            s.pending_token = None

    def release(self, session: GenerationSession) -> None:
        """Gives the session's row back (its cached tokens are dropped)."""
        self.cache.truncate(0, session.row)
        self.free_rows.append(session.row)
        self.free_rows.sort()
        session.finished = True


def verify_draft(model: AarambhModel, cache, row: int, base_len: int, pending_token: int, draft_tokens):
    """Target-side round of greedy speculative decoding (speculative.rs:304-318,
    388-418): one forward of ``[pending_token] + draft_tokens`` against the cache
    at ``base_len``; draft token i is accepted while it equals the target's greedy
    choice after the tokens before it.  The cache row is left holding exactly the
    accepted prefix (an O(1) ``truncate`` where the reference restores a snapshot
    and replays the accepted tokens).  Returns (number of accepted draft tokens,
    the target's next token after them, logits [1 + len(draft), vocab])."""
    draft = [int(t) for t in draft_tokens]
    if cache.seq_len(row) != base_len:
        raise _lib.Ab2Error(-1, f"cache row holds {cache.seq_len(row)} tokens, expected {base_len}")
    ids = torch.tensor([[int(pending_token)] + draft])
    logits = model.forward_with_cache(ids, base_len, cache, row=row)[0]
    choice = argmax(logits).cpu().tolist()
    accepted = 0
    while accepted < len(draft) and choice[accepted] == draft[accepted]:
        accepted += 1
    cache.truncate(base_len + 1 + accepted, row)
    return accepted, choice[accepted], logits
