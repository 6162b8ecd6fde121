"""A model built from a blueprint, and its one step function.

``Model.step`` takes a batch of sequences (cache slots) with the new tokens of
each, which may differ in number: whole prompts of unequal lengths in one step,
then one token each.  It runs only those tokens, as one packed batch, against
what earlier steps left in the cache, and returns float32 logits at the wanted
places only.  It replaces the pair ``prefill`` (equal lengths, empty cache) /
``decode_step`` of davidjoyme/flashdecode-cuda (engine/model.py:142-312).

Host work per step: reserve cache blocks, build the step's index arrays, one
small upload; lengths live on the host, nothing is read back.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .. import kernels as K
from ..cache.paged import DEFAULT_BLOCK_SIZE, KVGroupSpec, PagedCache, StateSpec
from ..parts.base import KVRequest, LayerCache, Runtime
from ..registry import architecture, part_class
from ..weights import loader as W
from .blueprint import ModelBlueprint, PartSpec

Want = Union[str, None, Sequence[Sequence[int]]]


class Workspace:
    """Named scratch tensors that persist between steps (grown on demand), so
    a step allocates nothing once shapes have been seen."""

    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[Tuple, torch.Tensor] = {}      # (name, dtype, shape) -> view; dropped when its buffer grows

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        key = (name, dtype, shape)
        view = self._views.get(key)
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        buf = self._bufs.get((name, dtype))
        if buf is None or buf.numel() < n:
            buf = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[(name, dtype)] = buf
            for k in [k for k in self._views if k[0] == name and k[1] == dtype]:
                del self._views[k]
        if len(self._views) > 4096:
            self._views.clear()
        view = buf[:n].view(shape)
        self._views[key] = view
        return view


@dataclass
class StepContext:
    """Everything the parts see of one step.  Index arrays are int32 on the
    device; ``h_*`` are their host mirrors for parts written in Python."""
    rt: Runtime
    ws: Workspace
    cache: PagedCache
    T: int                      # tokens in the step (padding included)
    n_rows: int                 # sequences in the step (padding included)
    tokens: torch.Tensor        # [T] token ids
    tok_row: torch.Tensor       # [T] batch row of each token
    tok_pos: torch.Tensor       # [T] position of each token in its sequence
    row_slot: torch.Tensor      # [n] cache slot of each row; -1 marks a padding row
    row_q_start: torch.Tensor   # [n] first token of the row
    row_q_len: torch.Tensor     # [n] new tokens of the row
    row_ctx_len: torch.Tensor   # [n] tokens cached before the step
    want_rows: Optional[torch.Tensor]   # [n_want] tokens whose logits are wanted
    n_want: int
    max_q_len: int
    kv_len_bound: int           # >= longest sequence after the step; sizes grids only
    h_slots: List[int] = field(default_factory=list)
    h_q_len: List[int] = field(default_factory=list)
    h_ctx_len: List[int] = field(default_factory=list)
    # set for every schedule entry: whoever consumes the block's output takes float partial sums [parts, T, H]
    delta_parts_ok: bool = False
    # set for every schedule entry, and by a block for each of its parts: the weights the step streams first after
    # the part that runs now (``Part.first_weights`` of what follows), or None; a part may have its last kernel ask
    # L2 for their beginning
    upcoming: Optional[torch.Tensor] = None


class _Staging:
    """Ring of pinned host buffers for the per-step index upload; a buffer is
    reused only after the copy that read it has completed.  The numpy views of
    the buffers and the events are made once: this runs between two decode steps,
    while the GPU has nothing to do."""

    def __init__(self, n: int = 4):
        self.bufs: List[Optional[torch.Tensor]] = [None] * n
        self.views: List[Optional[np.ndarray]] = [None] * n
        self.events: List[Optional[torch.cuda.Event]] = [None] * n
        self.used = [False] * n
        self.i = 0

    def upload(self, host: np.ndarray, dst: torch.Tensor) -> None:
        if dst.device.type != "cuda":
            dst.copy_(torch.from_numpy(host))
            return
        i = self.i
        self.i = (i + 1) % len(self.bufs)
        if self.used[i]:
            self.events[i].synchronize()
        n = host.size
        buf = self.bufs[i]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1024), dtype=torch.int32).pin_memory()
            self.bufs[i], self.views[i] = buf, buf.numpy()
            if self.events[i] is None:
                self.events[i] = torch.cuda.Event()
        self.views[i][:n] = host
        K.copy_h2d_async(dst, buf, n)
        self.events[i].record()
        self.used[i] = True


class Model:
    """Parts built from a blueprint; ``bind`` gives them weights; ``new_cache``
    and ``step`` run them."""

    def __init__(self, config, blueprint: ModelBlueprint, dtype: torch.dtype = torch.bfloat16, device="cuda"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be torch.float32 or torch.bfloat16, got {dtype}")
        blueprint.validate()
        self.config = config
        self.blueprint = blueprint
        self.dtype = dtype
        self.device = torch.device(device)
        self.hidden_size = blueprint.hidden_size
        self.vocab_size = blueprint.vocab_size
        self.positions = {name: self._build(spec) for name, spec in blueprint.positions.items()}
        self.embedding = self._build(blueprint.embedding)
        self.blocks = []
        for ls in blueprint.layers:
            block_cls = part_class("block", ls.block)
            self.blocks.append(block_cls(**{name: self._build(spec) for name, spec in ls.parts.items()}))
        self.final_norm = self._build(blueprint.final_norm)
        self.head = self._build(blueprint.head)
        self.schedule = list(blueprint.schedule)
        self._layout = self._cache_layout()
        self.rt: Optional[Runtime] = None
        self.ws: Optional[Workspace] = None
        self._staging = _Staging()
        self.trace: Optional[Dict[str, torch.Tensor]] = None    # set to {} to record per-layer activations
        self.last_meta_host: Optional[np.ndarray] = None        # the index array of the last prepared step
        self.bound = False

    # ------------------------------------------------------------------ build
    @classmethod
    def from_config(cls, config, dtype: torch.dtype = torch.bfloat16, device="cuda") -> "Model":
        arch = architecture(config.architecture)
        return cls(config, arch.blueprint(config), dtype, device)

    def _build(self, spec: PartSpec):
        cls = part_class(spec.kind, spec.name)
        params = dict(spec.params)
        if isinstance(params.get("position"), str):
            params["position"] = self.positions[params["position"]]
        if spec.kind == "position":
            return cls(**params)
        return cls(prefix=spec.prefix, **params)

    def all_parts(self) -> list:
        parts = list(self.positions.values()) + [self.embedding]
        for b in self.blocks:
            parts += [b] + list(b.parts())
        return parts + [self.final_norm, self.head]

    def tensor_specs(self) -> List[W.TensorSpec]:
        specs, seen = [], set()
        for p in self.all_parts():
            for s in p.tensor_specs():
                if s.name in seen:
                    raise ValueError(f"tensor {s.name} is declared by two parts")
                seen.add(s.name)
                specs.append(s)
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> "Model":
        """Check ``tensors`` (by checkpoint name, any device) against what the
        parts declare, move them to the device in their storage dtype, and hand
        them to the parts."""
        if self.device.type != "cuda" and not getattr(self, "_allow_cpu", False):
            raise K.KernelError("flashdecode_cuda_b200 models run on a CUDA device only; there is no CPU path")
        specs = self.tensor_specs()
        tensors = dict(tensors)
        head = self.blueprint.head
        tied = head.params.get("tied_to")
        head_name = f"{head.prefix}.weight"
        if tied and head_name in tensors and tied in tensors and tensors[head_name].shape == tensors[tied].shape \
                and torch.equal(tensors[head_name].cpu(), tensors[tied].cpu()):
            del tensors[head_name]          # a tied checkpoint that stores its head twice
        W.check(specs, tensors)
        if self.device.type == "cuda":
            K.require_device()
        status = torch.zeros(1, dtype=torch.int32, device=self.device)
        sms = K.sm_count() if self.device.type == "cuda" else 1
        self.rt = Runtime(self.device, self.dtype, status, sms)
        self.ws = Workspace(self.device)
        by_name = {s.name: s for s in specs}
        on_dev = {n: W.cast(by_name[n], t, self.dtype, self.device) for n, t in tensors.items()}
        for p in self.all_parts():
            p.bind(on_dev, self.rt)
        self.bound = True
        return self

    @property
    def graph_safe(self) -> bool:
        """Whether decode steps may be captured into CUDA graphs (every part says so)."""
        return all(getattr(p, "graph_safe", True) for p in self.all_parts())

    def weight_bytes(self, include_embedding: bool = False) -> int:
        """Bytes of weights a decode step reads once: every layer's matrices
        and vectors and the output head; the embedding table only by rows."""
        total = sum(p.weight_bytes() for p in self.all_parts() if p is not self.embedding)
        if include_embedding:
            total += self.embedding.table.numel() * self.embedding.table.element_size()
        return total

    # ------------------------------------------------------------------ cache
    def _cache_layout(self):
        groups: List[dict] = []          # {"key": (n_kv, d, window), "n_layers": int}
        states: List[StateSpec] = []
        runs = []                        # per schedule entry: (group index or None, layer in group, writes, {name: state key})
        for i, run in enumerate(self.schedule):
            mixer = getattr(self.blocks[run.layer], "mixer", None)
            req: Optional[KVRequest] = mixer.kv_request() if mixer is not None else None
            if run.cache_from is not None:
                owner = self.schedule[run.cache_from]
                omixer = getattr(self.blocks[owner.layer], "mixer", None)
                oreq = omixer.kv_request() if omixer is not None else None
                if (req is None) != (oreq is None) or (req is not None and
                                                       (req.n_kv_heads, req.head_dim, req.window) !=
                                                       (oreq.n_kv_heads, oreq.head_dim, oreq.window)):
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {run.cache_from}: "
                                     f"their mixers keep different things")
                g, l, _, st = runs[run.cache_from]
                runs.append((g, l, False, st))
                continue
            gi, li = None, 0
            if req is not None:
                key = (req.n_kv_heads, req.head_dim, req.window)
                for j, g in enumerate(groups):
                    if g["key"] == key:
                        gi = j
                        break
                else:
                    groups.append({"key": key, "n_layers": 0})
                    gi = len(groups) - 1
                li = groups[gi]["n_layers"]
                groups[gi]["n_layers"] += 1
            st = {}
            for s in (mixer.state_requests() if mixer is not None else []):
                key = f"run{i}.{s.name}"
                states.append(StateSpec(key, tuple(s.shape), s.dtype))
                st[s.name] = key
            runs.append((gi, li, True, st))
        specs = [KVGroupSpec(g["n_layers"], *g["key"]) for g in groups]
        return specs, states, runs

    def cache_groups(self) -> List[KVGroupSpec]:
        return list(self._layout[0])

    def new_cache(self, max_tokens: Optional[int] = None, *, batch_size: Optional[int] = None,
                  max_len: Optional[int] = None, block_size: int = DEFAULT_BLOCK_SIZE, max_slots: Optional[int] = None,
                  slack_blocks: int = 0) -> PagedCache:
        """A cache sized either by ``max_tokens`` (the most tokens that live
        sequences hold at any time, each sequence rounded up to a multiple of
        64) or, in the manner of ``new_paged_cache(batch_size, max_len,
        block_size)`` of davidjoyme/flashdecode-cuda (engine/model.py:115-135),
        by a batch size and a longest sequence."""
        limit = self.blueprint.max_positions
        if max_tokens is not None:
            units = max(1, -(-max_tokens // 64))
            per_unit = -(-64 // block_size)
            num_blocks = units * per_unit if block_size <= 64 else -(-max_tokens // block_size) + units
            slots = max_slots or units
            longest = min(max_len or max_tokens, limit, -(-max_tokens // 64) * 64)
        elif batch_size is not None and max_len is not None:
            if max_len > limit:
                raise ValueError(f"max_len {max_len} exceeds the configuration's max_position_embeddings {limit}")
            longest = max_len
            slots = max_slots or batch_size
            num_blocks = -(-max_len // block_size) * batch_size
        else:
            raise ValueError("new_cache needs max_tokens, or batch_size and max_len")
        num_blocks += slack_blocks
        groups, states, _ = self._layout
        for pos in self.positions.values():
            pos.prepare(longest, self.rt)
        cache = PagedCache(groups, states, num_blocks, slots, -(-longest // block_size), block_size,
                           self.dtype, self.device)
        cache.max_len = longest
        return cache

    def _layer_caches(self, cache: PagedCache) -> List[LayerCache]:
        out = []
        for gi, li, writes, st in self._layout[2]:
            out.append(LayerCache(cache.groups[gi] if gi is not None else None, li, writes,
                                  {name: cache.states[key] for name, key in st.items()}))
        return out

    # ------------------------------------------------------------------- step
    def _wanted(self, counts: List[int], want: Want) -> List[int]:
        starts = np.concatenate(([0], np.cumsum(counts)))[:-1]
        if want is None:
            return []
        if isinstance(want, str):
            if want == "last":
                return [int(s + c - 1) for s, c in zip(starts, counts)]
            if want == "all":
                return list(range(int(sum(counts))))
            raise ValueError(f"want must be 'last', 'all', None or a list of positions per sequence, got {want!r}")
        if len(want) != len(counts):
            raise ValueError(f"want lists positions for {len(want)} sequences, the step has {len(counts)}")
        rows = []
        for s, c, w in zip(starts, counts, want):
            for p in w:
                if not (0 <= p < c):
                    raise ValueError(f"wanted position {p} is outside the {c} tokens the sequence brings")
                rows.append(int(s + p))
        return rows

    def make_context(self, cache: PagedCache, slots: Sequence[int], tokens: Sequence[Sequence[int]],
                     want: Want = "last", pad_rows: int = 0, kv_len_bound: Optional[int] = None,
                     ws: Optional[Workspace] = None) -> StepContext:
        """Index arrays of a step.  ``pad_rows``: rows to add that hold no
        sequence (slot -1, one dummy token each), for fixed-size batches."""
        n = len(slots)
        counts = [len(t) for t in tokens]
        if n == 0 or len(tokens) != n or min(counts) < 1:
            raise ValueError("a step needs at least one sequence and at least one new token for each")
        if len(set(slots)) != n:
            raise ValueError(f"a slot appears twice in one step: {list(slots)}")
        ctx_len = [cache.length(s) for s in slots]
        for s, c, l in zip(slots, counts, ctx_len):
            if l + c > cache.max_len:
                raise ValueError(f"slot {s}: {l} cached + {c} new tokens exceed the cache's longest sequence "
                                 f"{cache.max_len}")
        flat = np.fromiter((t for seq in tokens for t in seq), dtype=np.int64, count=sum(counts))
        if flat.size and (flat.min() < 0 or flat.max() >= self.vocab_size):
            raise ValueError(f"token ids must lie in [0, {self.vocab_size}); got {int(flat.min())}..{int(flat.max())}")
        T, N = int(flat.size) + pad_rows, n + pad_rows
        # "all" on a padded batch includes the padding rows: the count of wanted rows is then fixed
        wanted = list(range(T)) if (pad_rows and want == "all") else self._wanted(counts, want)
        counts_p = np.asarray(counts + [1] * pad_rows, dtype=np.int32)
        starts = (np.cumsum(counts_p) - counts_p).astype(np.int32)
        ctx_p = np.asarray(ctx_len + [0] * pad_rows, dtype=np.int32)
        tok_row = np.repeat(np.arange(N, dtype=np.int32), counts_p)
        tok_pos = (np.arange(T, dtype=np.int32) - starts[tok_row] + ctx_p[tok_row]).astype(np.int32)
        host = np.concatenate([
            np.concatenate([flat.astype(np.int32), np.zeros(pad_rows, np.int32)]), tok_row, tok_pos,
            np.asarray(list(slots) + [-1] * pad_rows, dtype=np.int32), starts, counts_p, ctx_p,
            np.asarray(wanted, dtype=np.int32)])
        ws = ws or self.ws
        meta = ws.get("step_meta", (host.size,), torch.int32)
        self.last_meta_host = host
        self._staging.upload(host, meta)
        o = 0

        def take(k):
            nonlocal o
            v = meta[o:o + k]
            o += k
            return v
        tok, trow, tpos = take(T), take(T), take(T)
        rslot, rstart, rlen, rctx = take(N), take(N), take(N), take(N)
        wrows = take(len(wanted)) if wanted else None
        longest = max(l + c for l, c in zip(ctx_len, counts))
        return StepContext(self.rt, ws, cache, T, N, tok, trow, tpos, rslot, rstart, rlen, rctx, wrows,
                           len(wanted), int(max(counts)), int(kv_len_bound or longest),
                           list(slots), counts, ctx_len)

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Run the parts over a prepared step.  Returns logits [n_want, V]
        (float32, a view of workspace memory that the next step overwrites)."""
        resid = ctx.ws.get("resid", (ctx.T, self.hidden_size), torch.float32)
        self.embedding.forward(ctx, resid)
        if self.trace is not None:
            self.trace["embed"] = resid.detach().float().cpu().clone()
        caches = self._layer_caches(ctx.cache)
        delta = None
        for i, run in enumerate(self.schedule):
            # whoever norms next - the next entry's block or the final norm - says whether it takes float
            # partial sums [parts, T, H] for a delta; a block hands that on to its last sub-layer
            nxt = self.blocks[self.schedule[i + 1].layer] if i + 1 < len(self.schedule) else self.final_norm
            ctx.delta_parts_ok = bool(getattr(nxt, "accepts_parts", False))
            ctx.upcoming = (nxt if i + 1 < len(self.schedule) else self.head).first_weights()
            delta = self.blocks[run.layer].forward(ctx, resid, delta, caches[i])
            if self.trace is not None:
                d = delta.float().sum(0) if delta.dim() == 3 else delta.float()
                self.trace[f"layer.{i}"] = (resid + d).cpu()
        if ctx.n_want == 0:
            return None
        xn = ctx.ws.get("final_normed", (ctx.n_want, self.hidden_size), self.dtype)
        self.final_norm.forward(ctx, delta, resid, xn, rows=ctx.want_rows, n_out=ctx.n_want, write_resid=False)
        return self.head.forward(ctx, xn)

    def step(self, cache: PagedCache, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Want = "last") -> Optional[torch.Tensor]:
        """Feed ``tokens[i]`` (one or more new tokens) to the sequence in
        ``slots[i]``; return float32 logits [n_want, vocab] at the wanted places
        in the order of the sequences and of ``want``.

        ``want``: "last" (the last new token of each sequence), "all", None, or
        for each sequence a list of places among its new tokens."""
        if not self.bound:
            raise RuntimeError("the model has no weights yet: call bind() or use load_model()")
        counts = [len(t) for t in tokens]
        cache.reserve(list(zip(slots, counts)))
        cache.sync()
        ctx = self.make_context(cache, slots, tokens, want)
        logits = self.forward(ctx)
        for s, c in zip(slots, counts):
            cache.advance(s, c)
        return logits

    def check_status(self) -> None:
        """Read the kernels' status word (a device synchronisation) and raise
        if any kernel met an index it had to skip."""
        word = int(self.rt.status.item())
        if word:
            self.rt.status.zero_()
            raise RuntimeError(f"a kernel reported: {K.status_message(word)}")
