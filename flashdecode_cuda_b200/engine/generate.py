"""The generation loop: batches of unequal prompts, stop tokens, sequences
that end early, batch after batch.

``LlamaEngine.generate`` of davidjoyme/flashdecode-cuda (engine/model.py:315-329)
runs one batch of equal-length prompts for a fixed number of greedy steps.
Here requests wait in a queue; a batch is as many of them, in order, as the
slot count and the cache can hold; their prompts run in one step, then one
token each per step; a sequence that meets a stop token or its length limit
leaves at once and its slot and blocks go back; when the batch has drained the
next one starts on the same cache.

The loop's decisions need no GPU: it talks to a ``Backend`` (admit / release /
fits / run), which in tests is a fake.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterator, List, Optional, Sequence, Tuple


@dataclass
class Request:
    prompt: List[int]
    max_new_tokens: int
    temperature: float = 0.0
    stop_token_ids: Tuple[int, ...] = ()
    request_id: int = 0

    def __post_init__(self):
        if len(self.prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")


@dataclass
class Result:
    request_id: int
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""          # "stop" (a stop token, kept in tokens) or "length"


class Backend:
    """What the loop needs from an engine."""

    def capacity(self) -> Tuple[int, int]:
        """(slots, tokens) that a batch may hold when nothing else is live."""
        raise NotImplementedError

    def tokens_held(self, n_tokens: int) -> int:
        """Cache tokens a sequence of ``n_tokens`` occupies (rounded to blocks)."""
        raise NotImplementedError

    def admit(self) -> int:
        raise NotImplementedError

    def release(self, slot: int) -> None:
        raise NotImplementedError

    def run(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], requests: Sequence[Request],
            steps: Sequence[int]) -> List[int]:
        """Feed ``tokens[i]`` to ``slots[i]`` and sample one next token each."""
        raise NotImplementedError


def plan_batch(waiting: Sequence[Request], max_batch: int, slots: int, tokens: int, held) -> int:
    """How many requests from the head of the queue start together: at most
    ``max_batch`` and ``slots``, and their worst-case lengths (prompt + all new
    tokens, as the cache rounds them) must fit ``tokens``.  A request that
    cannot fit even alone is an error, not a wait."""
    n, used = 0, 0
    for r in waiting:
        need = held(len(r.prompt) + r.max_new_tokens)
        if need > tokens:
            raise ValueError(f"request {r.request_id}: {len(r.prompt)} prompt + {r.max_new_tokens} new tokens "
                             f"need {need} cache tokens, the cache holds {tokens}")
        if n >= max_batch or n >= slots or used + need > tokens:
            break
        n, used = n + 1, used + need
    return n


class GenerationLoop:
    def __init__(self, backend: Backend, max_batch: int = 64):
        if max_batch < 1:
            raise ValueError("max_batch must be >= 1")
        self.backend = backend
        self.max_batch = max_batch

    def events(self, requests: Sequence[Request]) -> Iterator[List[Tuple[int, int, Optional[str]]]]:
        """One list per step: (index of the request, its new token, finish
        reason or None) for every sequence that was live in that step."""
        waiting = list(enumerate(requests))
        slots_cap, tokens_cap = self.backend.capacity()
        while waiting:
            n = plan_batch([r for _, r in waiting], self.max_batch, slots_cap, tokens_cap,
                           self.backend.tokens_held)
            batch, waiting = waiting[:n], waiting[n:]
            live = [(idx, req, self.backend.admit()) for idx, req in batch]
            produced = {idx: 0 for idx, _, _ in live}
            feed = [list(req.prompt) for _, req, _ in live]
            try:
                while live:
                    new = self.backend.run([s for _, _, s in live], feed, [r for _, r, _ in live],
                                           [produced[i] for i, _, _ in live])
                    step_events, still, feed = [], [], []
                    for (idx, req, slot), tok in zip(live, new):
                        produced[idx] += 1
                        reason = None
                        if tok in req.stop_token_ids:
                            reason = "stop"
                        elif produced[idx] >= req.max_new_tokens:
                            reason = "length"
                        step_events.append((idx, tok, reason))
                        if reason is None:
                            still.append((idx, req, slot))
                            feed.append([tok])
                        else:
                            self.backend.release(slot)
                    live = still
                    yield step_events
            finally:
                for _, _, slot in live:          # only on an error or an abandoned iterator
                    self.backend.release(slot)

    def run(self, requests: Sequence[Request]) -> List[Result]:
        results = [Result(r.request_id) for r in requests]
        for step in self.events(requests):
            for idx, tok, reason in step:
                results[idx].tokens.append(tok)
                if reason:
                    results[idx].finish_reason = reason
        return results
