"""Decode steps replayed from CUDA graphs.

A decode step of this model is a few hundred small kernels; launched one by
one from Python their launch cost exceeds their run time (the finding of
davidjoyme/flashdecode-cuda, README.md:105-111: ~93 us per eager op call, "the
levers are launch count and graph capture").  Here a whole step - embedding,
every layer, final norm, output head and the sampler - is captured once per
batch-size bucket and replayed; per step the host only reserves cache blocks,
uploads one small index array and launches the graph.

A graph is tied to fixed device buffers (its own workspace) and to grid sizes,
so it is keyed by the padded batch size, a bound on the longest sequence (a
power of two; it sizes the split of the keys) and whether the step samples or
takes the argmax; temperatures, request ids, step counters and the seed are
read from device memory.  Padding rows carry slot -1; every kernel skips them,
so padding changes no result.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels as K
from ..cache.allocator import PoolExhausted
from ..cache.paged import PagedCache
from .model import Model, StepContext, Workspace

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
KV_BOUND_MIN = 1024      # the length bound of a graph is a power of two from here on (or the cache's longest sequence)


def bucket_of(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    return -(-n // 64) * 64


class _Graph:
    def __init__(self, ws: Workspace):
        self.ws = ws
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.ctx: Optional[StepContext] = None
        self.sampled: Optional[torch.Tensor] = None
        self.temp = self.req = self.step = self.seed = None
        self.seed_value: Optional[int] = None
        self.launches = 0
        self.sample_scratch = None
        self.n_rows_real = 0
        self.logits: Optional[torch.Tensor] = None   # [bucket, vocab] float32: the step's logits, in the graph's workspace
        self.host: Optional[np.ndarray] = None       # the step's index array; only a few slices change per step
        self.meta: Optional[torch.Tensor] = None     # its device copy (fixed address)


class GraphDecoder:
    """One-token-per-sequence steps of ``model`` over ``cache`` with sampling,
    through captured graphs.  ``run`` takes host tokens and returns the device
    tensor of sampled tokens; with ``tokens=None`` it feeds the previous step's
    sampled tokens without leaving the device."""

    def __init__(self, model: Model, cache: PagedCache):
        self.model, self.cache = model, cache
        self.graphs: Dict[Tuple, _Graph] = {}
        self.last: Optional[_Graph] = None
        self.last_n = 0
        self.launches_per_step = 0
        self._host_out: Optional[torch.Tensor] = None
        self._host_view: Optional[np.ndarray] = None
        # (graph, slots, the cache's lengths_version): the next step's slots and lengths are in that graph's index
        # array already; void as soon as any sequence of the cache has started, ended or grown since
        self._ahead: Optional[Tuple] = None

    # ------------------------------------------------------------------
    def _key(self, n: int, longest: int, greedy: bool, seed: int) -> Tuple:
        # powers of two: a sequence that grows from 1,000 to 4,000 tokens passes three bounds, not four, and a process
        # that captures fewer graphs stays clear of the slower replay that set in after the fourth capture (the same
        # graph 1.25 or 1.33 ms a step; which one changed with captures and large allocations, nothing else)
        bound = KV_BOUND_MIN
        while bound < longest:
            bound *= 2
        bound = min(bound, self.cache.max_len)
        return (bucket_of(n), bound, greedy, 0)       # the seed lives in device memory: one graph serves every seed

    def _prepare(self, g: _Graph, key: Tuple, slots: Sequence[int], tokens: Sequence[int]) -> StepContext:
        B, bound = key[0], key[1]
        return self.model.make_context(self.cache, slots, [[int(t)] for t in tokens], "all",
                                       pad_rows=B - len(slots), kv_len_bound=bound, ws=g.ws)

    def _body(self, g: _Graph, ctx: StepContext, key: Tuple) -> None:
        logits = self.model.forward(ctx)
        g.logits = logits
        if key[2]:
            K.sample(logits, g.sampled, scratch=g.sample_scratch)
        else:
            K.sample(logits, g.sampled, g.temp, g.req, g.step, 0, scratch=g.sample_scratch, seed_tensor=g.seed)

    def _refill(self, g: _Graph, key: Tuple, slots: Sequence[int], tokens: Sequence[int]) -> None:
        """Re-upload the index array of a captured graph for a new step: the batch-shape parts
        (rows of tokens, counts, wanted rows) never change; tokens, slots and lengths do."""
        B, n = key[0], len(slots)
        if min(tokens) < 0 or max(tokens) >= self.model.vocab_size:       # plain integers: cheaper than array reductions
            raise ValueError(f"token ids must lie in [0, {self.model.vocab_size})")
        h = g.host
        h[0:n] = tokens
        ahead, self._ahead = self._ahead, None
        if ahead is None or ahead[0] is not g or ahead[1] != tuple(slots) or ahead[2] != self.cache.lengths_version:
            self._fill_lengths(g, B, slots)     # else: written while the GPU ran the step before, and still true
        self.model._staging.upload(h, g.meta)

    def _fill_lengths(self, g: _Graph, B: int, slots: Sequence[int]) -> None:
        """The slots and lengths of the next step into a graph's index array."""
        n, cache = len(slots), self.cache
        lens = [cache.length(s) for s in slots]
        if max(lens) + 1 > cache.max_len:
            raise ValueError(f"a sequence would grow beyond the cache's longest sequence {cache.max_len}")
        h = g.host
        h[2 * B:2 * B + n] = lens               # positions of the new tokens
        h[3 * B:3 * B + n] = slots
        h[3 * B + n:4 * B] = -1
        h[6 * B:6 * B + n] = lens               # tokens cached before the step

    def _graph_for(self, key: Tuple, slots, tokens) -> Tuple[_Graph, StepContext]:
        g = self.graphs.get(key)
        if g is not None and len(slots) == g.n_rows_real:
            self._refill(g, key, slots, tokens)
            return g, g.ctx
        if g is not None:
            ctx = self._prepare(g, key, slots, tokens)      # same bucket, another number of real rows
            g.host, g.n_rows_real = self.model.last_meta_host.copy(), len(slots)
            return g, ctx
        B = key[0]
        dev = self.model.device
        g = _Graph(Workspace(dev))
        g.sampled = torch.zeros(B, dtype=torch.int32, device=dev)
        g.temp = torch.zeros(B, dtype=torch.float32, device=dev)
        g.req = torch.zeros(B, dtype=torch.int64, device=dev)
        g.step = torch.zeros(B, dtype=torch.int32, device=dev)
        g.seed = torch.zeros(1, dtype=torch.int64, device=dev)
        g.sample_scratch = torch.zeros(max(1, K.sample_scratch_words(B, self.model.vocab_size)),
                                       dtype=torch.int32, device=dev)
        ctx = self._prepare(g, key, slots, tokens)
        g.host, g.n_rows_real = self.model.last_meta_host.copy(), len(slots)
        g.meta = g.ws.get("step_meta", (g.host.size,), torch.int32)
        # One eager run before the capture, which allocates the workspace.  It runs on padding rows only (every
        # slot -1, which every kernel skips): the real step is the graph's first replay, so neither the cache
        # nor a mixer's per-sequence state sees this step twice.
        warm = g.host.copy()
        warm[3 * B:4 * B] = -1
        self.model._staging.upload(warm, g.meta)
        self._body(g, ctx, key)
        torch.cuda.synchronize()
        self.model._staging.upload(g.host, g.meta)
        graph = torch.cuda.CUDAGraph()
        before = K.launch_count()
        with torch.cuda.graph(graph):
            self._body(g, ctx, key)
        g.launches = K.launch_count() - before          # this library's kernels in one replay
        g.graph, g.ctx = graph, ctx
        self.graphs[key] = g
        return g, ctx

    # ------------------------------------------------------------------
    def run(self, slots: Sequence[int], tokens: Optional[Sequence[int]], temperatures: Optional[Sequence[float]] = None,
            request_ids: Optional[Sequence[int]] = None, steps: Optional[Sequence[int]] = None,
            seed: int = 0) -> torch.Tensor:
        """Feed one token to each slot, sample one next token each.  Returns an
        int32 device tensor whose first ``len(slots)`` entries are the tokens
        (valid until the next call).  ``tokens`` None: use the tokens sampled by
        the previous call (same slots, in the same order)."""
        cache, n = self.cache, len(slots)
        greedy = temperatures is None or not any(t > 0.0 for t in temperatures)
        cache.reserve([(s, 1) for s in slots])
        cache.sync()
        longest = max(cache.length(s) for s in slots) + 1
        key = self._key(n, longest, greedy, seed)
        device_fed = tokens is None
        if device_fed:
            if self.last is None or self.last_n != n:
                raise ValueError("no previous step with the same slots to take tokens from")
            prev = self.last.sampled[:n]
            tokens = [0] * n
        g, ctx = self._graph_for(key, slots, tokens)
        if device_fed:
            ctx.tokens[:n].copy_(prev)
        if not greedy:
            B = key[0]
            pad = B - n
            g.temp.copy_(torch.tensor(list(temperatures) + [0.0] * pad, dtype=torch.float32), non_blocking=False)
            g.req.copy_(torch.tensor(list(request_ids) + [0] * pad, dtype=torch.int64))
            g.step.copy_(torch.tensor(list(steps) + [0] * pad, dtype=torch.int32))
            if g.seed_value != seed:
                bits = seed & 0xFFFFFFFFFFFFFFFF
                g.seed.fill_(bits - (1 << 64) if bits >= (1 << 63) else bits)       # the same 64 bits, as int64
                g.seed_value = seed
        g.graph.replay()
        for s in slots:
            cache.advance(s, 1)
        self.last, self.last_n = g, n
        self.launches_per_step = g.launches
        # While the GPU runs this step: the blocks of the next one.  If every sequence goes on, the next call's
        # reserve and sync find nothing to do; one that ends gives the block back with its slot.  A refusal
        # here (a full pool, a sequence at its longest) is the next call's to report, if it still applies.
        # The same for the index array: everything but the tokens, in case the same sequences go on with this graph.
        self._ahead = None
        try:
            cache.reserve([(s, 1) for s in slots])
            cache.sync()
            if g.host is not None and n == g.n_rows_real:
                self._fill_lengths(g, key[0], slots)
                self._ahead = (g, tuple(slots), cache.lengths_version)
        except (ValueError, PoolExhausted):
            pass
        return g.sampled

    def last_logits(self, n: int) -> torch.Tensor:
        """float32 logits [n, vocab] of the last step's first ``n`` sequences (a view of the graph's workspace,
        valid until the next call)."""
        return self.last.logits[:n]

    def read_tokens(self, n: int) -> List[int]:
        """The first ``n`` tokens of the last step as host integers (one copy into pinned memory)."""
        src = self.last.sampled
        if self._host_out is None or self._host_out.numel() < src.numel():
            self._host_out = torch.empty(max(src.numel(), 256), dtype=torch.int32).pin_memory()
            self._host_view = self._host_out.numpy()
        if src.is_cuda:
            K.copy_d2h_sync(self._host_out, src, n)
        else:
            self._host_out[:n].copy_(src[:n])
        return self._host_view[:n].tolist()
