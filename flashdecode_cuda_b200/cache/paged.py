"""The cache of a batch: a slot per sequence, paged keys and values per layer
group, and fixed-size state per sequence.

What it keeps from ``PagedKVCache`` of davidjoyme/flashdecode-cuda
(engine/paged_cache.py:122-377): pools of blocks ``[num_blocks, n_kv,
block_size, head_dim]`` per layer, a block table with -1 for "no block", a
host mirror that the allocator reasons about, and "reserve before any layer
writes, advance once after all layers" (:220-241, engine/model.py:163-165,245-250).

What is different:

* lengths live on the host only; nothing is read back from the device;
* a sequence is a *slot record* (state, length, blocks); slots come from a
  LIFO free list and go back when a sequence ends, so batch after batch reuses
  slots and blocks;
* layers are gathered into *groups* with the same needs (all keys, or a window
  of them; KV heads; head size).  Each group has its own pool, allocator and
  block table; a window group gives blocks back as they fall behind the window;
* beside the paged storage there is per-sequence state of fixed size, indexed
  by slot, for mixers that carry a recurrent state instead of keys.

All decisions are taken on the host; the device holds the pools, the block
tables and the state buffers.  The class works with ``device="cpu"`` too, which
is how its bookkeeping is tested without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .allocator import IdAllocator, PoolExhausted

FREE, ACTIVE = 0, 1

# Tokens of a cache block unless the caller says otherwise.  64 is one key tile of the prompt attention kernel
# (one TMA copy per tile, head half and K or V; with 16-token blocks its copies are four times as many and
# a 2,048-token prompt's attention takes 42 instead of 33 us) and the unit in which requests are counted.
DEFAULT_BLOCK_SIZE = 64


@dataclass(frozen=True)
class KVGroupSpec:
    """Layers that share one kind of key/value storage.  ``window`` None: all
    keys are kept; a number: only blocks that still hold one of the last
    ``window`` positions."""
    n_layers: int
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state per sequence: ``[max_slots, *shape]`` of ``dtype``."""
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class SlotRecord:
    state: int = FREE
    length: int = 0
    blocks: List[List[int]] = field(default_factory=list)      # per group: block id per table column (-1: none)


class KVGroup:
    """Pool, allocator and block table of one layer group."""

    def __init__(self, spec: KVGroupSpec, num_blocks: int, max_slots: int, max_blocks_per_seq: int,
                 block_size: int, dtype: torch.dtype, device):
        self.spec = spec
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.max_blocks_per_seq = max_blocks_per_seq
        # [layer, k|v, block, kv head, token in block, dim]
        self.pool = torch.zeros((spec.n_layers, 2, num_blocks, spec.n_kv_heads, block_size, spec.head_dim),
                                dtype=dtype, device=device)
        self.alloc = IdAllocator(num_blocks, "block")
        self.table_host = np.full((max_slots, max_blocks_per_seq), -1, dtype=np.int32)
        self.table = torch.full((max_slots, max_blocks_per_seq), -1, dtype=torch.int32, device=device)
        self._pending: Dict[Tuple[int, int], int] = {}     # (slot, column) -> block, not yet on the device
        self._ring: List[Optional[torch.Tensor]] = [None] * 4          # pinned staging buffers
        self._ring_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self._ring_i = 0
        self._dev_updates: Optional[torch.Tensor] = None

    def k_pool(self, layer: int) -> torch.Tensor:
        return self.pool[layer, 0]

    def v_pool(self, layer: int) -> torch.Tensor:
        return self.pool[layer, 1]

    def set_entry(self, slot: int, col: int, block: int) -> None:
        self.table_host[slot, col] = block
        self._pending[(slot, col)] = block       # a later value for the same entry replaces the earlier

    def sync(self) -> None:
        """Bring the device table up to date with one small copy: [indices | values] from a ring
        of pinned buffers (a buffer is reused only after the copy that read it has completed)."""
        if not self._pending:
            return
        n = len(self._pending)
        width = self.max_blocks_per_seq
        flat = np.empty(2 * n, dtype=np.int32)
        flat[:n] = [s * width + c for s, c in self._pending]
        flat[n:] = list(self._pending.values())
        self._pending.clear()
        dev = self.table.device
        if dev.type != "cuda":
            t = torch.from_numpy(flat)
            self.table.view(-1).index_copy_(0, t[:n].long(), t[n:])
            return
        i = self._ring_i
        self._ring_i = (i + 1) % len(self._ring)
        if self._ring_events[i] is not None:
            self._ring_events[i].synchronize()
        buf = self._ring[i]
        if buf is None or buf.numel() < 2 * n:
            buf = torch.empty(max(2 * n, 512), dtype=torch.int32).pin_memory()
            self._ring[i] = buf
        buf[:2 * n].numpy()[:] = flat
        if self._dev_updates is None or self._dev_updates.numel() < 2 * n:
            self._dev_updates = torch.empty(max(2 * n, 512), dtype=torch.int32, device=dev)
        self._dev_updates[:2 * n].copy_(buf[:2 * n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._ring_events[i] = ev
        self.table.view(-1).index_copy_(0, self._dev_updates[:n].long(), self._dev_updates[n:2 * n])

    def bytes_per_token(self) -> int:
        s = self.spec
        return 2 * s.n_layers * s.n_kv_heads * s.head_dim * self.pool.element_size()


class PagedCache:
    def __init__(self, groups: Sequence[KVGroupSpec], states: Sequence[StateSpec], num_blocks: int,
                 max_slots: int, max_blocks_per_seq: int, block_size: int = DEFAULT_BLOCK_SIZE,
                 dtype: torch.dtype = torch.bfloat16, device="cuda"):
        if block_size <= 0 or max_slots <= 0 or max_blocks_per_seq <= 0:
            raise ValueError("block_size, max_slots and max_blocks_per_seq must be positive")
        self.block_size = block_size
        self.max_slots = max_slots
        self.max_blocks_per_seq = max_blocks_per_seq
        self.num_blocks = num_blocks
        self.max_len = max_blocks_per_seq * block_size      # longest sequence; a model may set it lower
        self.dtype = dtype
        self.device = torch.device(device)
        self.groups = [KVGroup(g, num_blocks, max_slots, max_blocks_per_seq, block_size, dtype, self.device)
                       for g in groups]
        self.states: Dict[str, torch.Tensor] = {
            s.name: torch.zeros((max_slots, *s.shape), dtype=s.dtype, device=self.device) for s in states}
        self.slot_alloc = IdAllocator(max_slots, "slot")
        self.slots = [SlotRecord() for _ in range(max_slots)]
        self.lengths_version = 0        # grows whenever a slot's sequence or its length changes (admit, release, advance)

    # ------------------------------------------------------------------ slots
    def admit(self) -> int:
        """Take a free slot for a new sequence of length 0; its state is zeroed."""
        (slot,) = self.slot_alloc.allocate(1)
        rec = self.slots[slot]
        rec.state, rec.length = ACTIVE, 0
        self.lengths_version += 1
        rec.blocks = [[] for _ in self.groups]
        for st in self.states.values():
            st[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        """Give the slot and everything it holds back."""
        rec = self._record(slot)
        for g, blocks in zip(self.groups, rec.blocks):
            held = [b for b in blocks if b >= 0]
            if held:
                g.alloc.free(held)
            for col, b in enumerate(blocks):
                if b >= 0:
                    g.set_entry(slot, col, -1)
        rec.state, rec.length, rec.blocks = FREE, 0, []
        self.lengths_version += 1
        self.slot_alloc.free([slot])

    def _record(self, slot: int) -> SlotRecord:
        if not (0 <= slot < self.max_slots) or self.slots[slot].state != ACTIVE:
            raise ValueError(f"slot {slot} holds no sequence")
        return self.slots[slot]

    def length(self, slot: int) -> int:
        return self._record(slot).length

    def active_slots(self) -> List[int]:
        return [i for i, r in enumerate(self.slots) if r.state == ACTIVE]

    # ------------------------------------------------------------- capacity
    def blocks_needed(self, n_tokens: int) -> int:
        return (n_tokens + self.block_size - 1) // self.block_size

    def reserve(self, wants: Sequence[Tuple[int, int]]) -> None:
        """For every (slot, extra tokens): make sure blocks exist for positions
        up to length + extra, in every group.  Nothing changes if any group
        cannot serve the whole request."""
        listed = [slot for slot, _ in wants]
        if len(set(listed)) != len(listed):
            raise ValueError(f"a slot appears twice in one reservation: {listed}")
        plan = []
        need_per_group = [0] * len(self.groups)
        for slot, extra in wants:
            rec = self._record(slot)
            cols = self.blocks_needed(rec.length + extra)
            if cols > self.max_blocks_per_seq:
                raise ValueError(f"slot {slot}: {rec.length + extra} tokens need {cols} blocks, "
                                 f"the table holds {self.max_blocks_per_seq} per sequence")
            for gi, blocks in enumerate(rec.blocks):
                if cols > len(blocks):
                    need_per_group[gi] += cols - len(blocks)
                    plan.append((slot, gi, len(blocks), cols))
        for gi, g in enumerate(self.groups):
            if need_per_group[gi] > g.alloc.num_free:
                raise PoolExhausted(f"paged cache exhausted: group {gi} needs {need_per_group[gi]} more blocks, "
                                    f"{g.alloc.num_free} free of {g.num_blocks}")
        for slot, gi, have, cols in plan:
            g = self.groups[gi]
            new = g.alloc.allocate(cols - have)
            self.slots[slot].blocks[gi].extend(new)
            for c, b in zip(range(have, cols), new):
                g.set_entry(slot, c, b)

    def advance(self, slot: int, n: int) -> None:
        """The step's tokens are in the cache: lengthen, and let window groups
        give back blocks that no later query can see."""
        rec = self._record(slot)
        if self.blocks_needed(rec.length + n) > min((len(b) for b in rec.blocks), default=1 << 30):
            raise ValueError(f"slot {slot}: advancing by {n} beyond the reserved blocks")
        rec.length += n
        self.lengths_version += 1
        for gi, g in enumerate(self.groups):
            w = g.spec.window
            if w is None:
                continue
            # the next query sits at position `length` and sees keys > length - w
            first_needed = max(0, rec.length - w + 1)
            dead_cols = first_needed // self.block_size
            blocks = rec.blocks[gi]
            freed = []
            for c in range(min(dead_cols, len(blocks))):
                if blocks[c] >= 0:
                    freed.append(blocks[c])
                    blocks[c] = -1
                    g.set_entry(slot, c, -1)
            if freed:
                g.alloc.free(freed)

    def sync(self) -> None:
        for g in self.groups:
            g.sync()

    # ----------------------------------------------------------- diagnostics
    def slot_of(self, slot: int, position: int, group: int = 0) -> Tuple[int, int]:
        """(block id, offset in block) of a cached position
        (engine/paged_cache.py:257-262 of the reference)."""
        rec = self._record(slot)
        return rec.blocks[group][position // self.block_size], position % self.block_size

    def gather(self, slot: int, group: int, layer: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Keys and values of a slot as [length, n_kv, d] (positions whose block
        was given back read as zero).  For tests and debugging."""
        rec = self._record(slot)
        g = self.groups[group]
        s = g.spec
        k = torch.zeros((rec.length, s.n_kv_heads, s.head_dim), dtype=g.pool.dtype, device=g.pool.device)
        v = torch.zeros_like(k)
        for pos in range(rec.length):
            b = rec.blocks[group][pos // self.block_size]
            if b >= 0:
                k[pos] = g.pool[layer, 0, b, :, pos % self.block_size]
                v[pos] = g.pool[layer, 1, b, :, pos % self.block_size]
        return k, v

    def kv_bytes(self, slots: Optional[Sequence[int]] = None) -> int:
        """Bytes of keys and values that a decode step over ``slots`` has to
        read: valid tokens only, a window group at most its window
        (engine/paged_cache.py:352-364 of the reference counts the same way)."""
        slots = self.active_slots() if slots is None else slots
        total = 0
        for g in self.groups:
            for s in slots:
                n = self._record(s).length
                if g.spec.window is not None:
                    n = min(n, g.spec.window)
                total += n * g.bytes_per_token()
        return total

    def fragmentation(self) -> float:
        """Share of the allocated token places that hold no token: the unused tails of the sequences' last
        blocks (engine/paged_cache.py:366-371 of the reference).  0.0 for an empty cache; window groups count
        the blocks they still hold."""
        places = tokens = 0
        for gi, g in enumerate(self.groups):
            for rec in self.slots:
                if rec.state != ACTIVE:
                    continue
                held = sum(1 for b in rec.blocks[gi] if b >= 0)
                places += held * self.block_size
                first = len(rec.blocks[gi]) - held                 # columns a window group has given back
                tokens += max(0, rec.length - first * self.block_size)
        return 0.0 if places == 0 else 1.0 - tokens / places

    def blocks_in_use(self) -> List[int]:
        return [g.alloc.num_used for g in self.groups]

    def check_invariants(self) -> None:
        """No block lost, held twice or free while held; slots likewise."""
        for gi, g in enumerate(self.groups):
            held: Dict[int, int] = {}
            for si, rec in enumerate(self.slots):
                if rec.state != ACTIVE:
                    if rec.blocks:
                        raise AssertionError(f"free slot {si} still lists blocks")
                    continue
                for b in rec.blocks[gi]:
                    if b < 0:
                        continue
                    if b in held:
                        raise AssertionError(f"group {gi}: block {b} held by slots {held[b]} and {si}")
                    if not g.alloc.in_use(b):
                        raise AssertionError(f"group {gi}: block {b} of slot {si} is on the free list")
                    held[b] = si
            if len(held) != g.alloc.num_used:
                raise AssertionError(f"group {gi}: {g.alloc.num_used} blocks marked used, {len(held)} held by slots")
            if g.alloc.num_free + g.alloc.num_used != g.num_blocks:
                raise AssertionError(f"group {gi}: free + used != pool size")
        n_active = sum(r.state == ACTIVE for r in self.slots)
        if n_active != self.slot_alloc.num_used:
            raise AssertionError(f"{self.slot_alloc.num_used} slots marked used, {n_active} active records")

    def __repr__(self) -> str:
        used = ", ".join(f"{g.alloc.num_used}/{g.num_blocks}" for g in self.groups)
        return (f"PagedCache(slots {self.slot_alloc.num_used}/{self.max_slots}, blocks used [{used}], "
                f"block_size {self.block_size}, fragmentation {self.fragmentation():.1%}, {self.dtype})")
