"""The cache: a slot per sequence, keys and values per cache line in pages of 64
tokens, and beside them a per-sequence state of fixed size.

The reference allocates, per ``generate`` call and for its single sequence, two
``(prompt + n_new, nkv*hd)`` arrays per layer (src/minimax.rs:395-398).  Here many
sequences of unequal, growing lengths share one store, so the store is cut into
pages: a sequence holds ``ceil(length / 64)`` pages per group and a table maps
(slot, position // 64) to a page.  Cache lines whose needs are the same (number
of key/value heads, head size, all keys or a window of them) form a *group* with
a store, a page pool and a table of its own; a windowed group gives a page back
as soon as every key on it lies outside the window.  What is cached is K after
norm and rotary and V as projected (src/minimax.rs:262-268).

The state area holds, per cache line that asks for one, a tensor of a fixed
shape and type per slot, zeroed when the slot is given out.  MiniMax-M2 has no such
state; mixers with a recurrence use it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from .pools import CacheFull, IndexPool

PAGE_TOKENS = 64
_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass(frozen=True)
class CacheNeed:
    """What one cache line needs.  ``kv_heads == 0`` means no keys and values."""

    kv_heads: int = 0
    head_dim: int = 0
    window: int | None = None            # None: every earlier key stays visible
    state_shape: tuple[int, ...] = ()    # state per sequence; () for none
    state_dtype: str = "float32"         # "float32" | "bfloat16" | "int32"

    @property
    def group_key(self) -> tuple[int, int, int | None] | None:
        return (self.kv_heads, self.head_dim, self.window) if self.kv_heads else None


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclass
class LineView:
    """What a mixer sees of its cache line."""

    keys: torch.Tensor | None            # [num_pages, kv_heads, PAGE_TOKENS, head_dim]
    values: torch.Tensor | None          # [num_pages, kv_heads, head_dim, PAGE_TOKENS]
    page_table: torch.Tensor | None      # int32 [num_slots, max_pages]; -1 where no page is held
    window: int | None
    state: torch.Tensor | None           # [num_slots, *state_shape] in the need's state_dtype


class _Group:
    def __init__(self, key, lines, num_pages, num_slots, dtype, device, allocate):
        self.kv_heads, self.head_dim, self.window = key
        self.lines = list(lines)
        self.num_pages = num_pages
        self.pool = IndexPool(num_pages, "page")
        self.table = np.full((num_slots, num_pages), -1, dtype=np.int32)
        self.first_page = np.zeros(num_slots, dtype=np.int64)        # first page index still held
        self.end_page = np.zeros(num_slots, dtype=np.int64)          # one past the last page held
        self.dirty: list[tuple[int, int, int]] = []
        self.fresh: list[int] = []           # pages given out since the last sync whose old contents may be read
        shape = (len(self.lines), num_pages, self.kv_heads, PAGE_TOKENS, self.head_dim)
        if allocate:
            self.keys = torch.zeros(shape, dtype=dtype, device=device)
            # within a page the values lie transposed, [head_dim, PAGE_TOKENS]: the product P @ V then reads
            # runs of neighbouring keys
            self.values = torch.zeros(shape[:3] + (self.head_dim, PAGE_TOKENS), dtype=dtype, device=device)
            self.table_dev = torch.full((num_slots, num_pages), -1, dtype=torch.int32, device=device)
        else:
            self.keys = self.values = self.table_dev = None

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, pages_for(new_len) - int(self.end_page[slot]))

    def grow(self, slot: int, new_len: int) -> None:
        lo, hi = int(self.end_page[slot]), pages_for(new_len)
        if hi <= lo:
            return
        for index in range(lo, hi):
            self.table[slot, index] = self.pool.alloc()
        self.end_page[slot] = hi
        self.dirty.append((slot, lo, hi))
        # A page that the new tokens do not fill keeps, beyond them, what an earlier sequence left there.  The
        # attention kernels give such keys no weight, but 0 x NaN is NaN: whatever was there must be finite.
        # So the last page handed out is cleared unless the sequence's tokens fill it to the end.
        if new_len % PAGE_TOKENS:
            self.fresh.append(int(self.table[slot, hi - 1]))

    def release_outside_window(self, slot: int, length: int) -> None:
        if self.window is None:
            return
        # the next query sits at position >= length and sees keys j > position - window
        first_needed = max(0, length - self.window + 1) // PAGE_TOKENS
        lo = int(self.first_page[slot])
        hi = min(first_needed, int(self.end_page[slot]))
        if hi <= lo:
            return
        for index in range(lo, hi):
            self.pool.free(int(self.table[slot, index]))
            self.table[slot, index] = -1
        self.first_page[slot] = hi
        self.dirty.append((slot, lo, hi))

    def release_all(self, slot: int) -> None:
        lo, hi = int(self.first_page[slot]), int(self.end_page[slot])
        for index in range(lo, hi):
            self.pool.free(int(self.table[slot, index]))
            self.table[slot, index] = -1
        if hi > lo:
            self.dirty.append((slot, lo, hi))
        self.first_page[slot] = 0
        self.end_page[slot] = 0

    def sync(self) -> None:
        if self.table_dev is not None:
            for slot, lo, hi in self.dirty:
                self.table_dev[slot, lo:hi].copy_(torch.from_numpy(self.table[slot, lo:hi]))
            if len(self.fresh) == 1:
                self.keys[:, self.fresh[0]].zero_()
                self.values[:, self.fresh[0]].zero_()
            elif self.fresh:
                pages = torch.tensor(self.fresh, dtype=torch.int64).to(self.keys.device)
                self.keys.index_fill_(1, pages, 0)
                self.values.index_fill_(1, pages, 0)
        self.dirty.clear()
        self.fresh.clear()


class SequenceCache:
    """Slots, pages and state for the sequences an engine is running."""

    def __init__(self, needs: Sequence[CacheNeed], *, max_tokens: int, num_slots: int | None = None,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device | str = "cpu",
                 allocate: bool = True):
        if max_tokens <= 0:
            raise ValueError(f"a cache for {max_tokens} tokens cannot hold a sequence")
        self.needs = list(needs)
        self.num_pages = pages_for(max_tokens)
        self.max_tokens = self.num_pages * PAGE_TOKENS
        self.num_slots = num_slots if num_slots is not None else min(self.num_pages, 2048)
        if self.num_slots <= 0:
            raise ValueError("a cache needs at least one slot")
        self.dtype, self.device = dtype, torch.device(device)
        self.slots = IndexPool(self.num_slots, "slot")
        self.lengths = np.zeros(self.num_slots, dtype=np.int64)
        by_key: dict[tuple, list[int]] = {}
        for line, need in enumerate(self.needs):
            if need.group_key is not None:
                by_key.setdefault(need.group_key, []).append(line)
        self.groups = [_Group(key, lines, self.num_pages, self.num_slots, dtype, self.device, allocate)
                       for key, lines in by_key.items()]
        self._line_group: dict[int, tuple[_Group, int]] = {}
        for group in self.groups:
            for index, line in enumerate(group.lines):
                self._line_group[line] = (group, index)
        self.states: dict[int, torch.Tensor] = {}
        for line, need in enumerate(self.needs):
            if need.state_shape:
                if need.state_dtype not in _STATE_DTYPES:
                    raise ValueError(f"cache line {line}: a state of type {need.state_dtype!r}; "
                                     f"known: {sorted(_STATE_DTYPES)}")
                self.states[line] = torch.zeros((self.num_slots, *need.state_shape),
                                                dtype=_STATE_DTYPES[need.state_dtype],
                                                device=self.device if allocate else "cpu")

    # -- slots ------------------------------------------------------------------------------------
    def alloc(self) -> int:
        """A free slot for a new sequence: length 0, no pages, state zeroed."""
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        for state in self.states.values():
            state[slot].zero_()
        return slot

    def free(self, slot: int) -> None:
        """Give a sequence's slot and pages back."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is freed twice (or was never given out)")
        for group in self.groups:
            group.release_all(slot)
        self.lengths[slot] = 0
        self.slots.free(slot)

    def length(self, slot: int) -> int:
        return int(self.lengths[slot])

    # -- one step ---------------------------------------------------------------------------------
    def begin_step(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """Make room for ``new_tokens[i]`` more tokens of sequence ``slots[i]``; all or nothing."""
        if len(set(slots)) != len(slots):
            raise ValueError("a sequence appears twice in one step")
        for slot in slots:
            if not self.slots.is_held(slot):
                raise ValueError(f"slot {slot} is not held by a sequence")
        for group in self.groups:
            want = sum(group.pages_needed(s, self.length(s) + n) for s, n in zip(slots, new_tokens))
            if want > group.pool.num_free:
                raise CacheFull(
                    f"the step needs {want} more pages of {PAGE_TOKENS} tokens, {group.pool.num_free} of "
                    f"{group.num_pages} are free (cache sized for {self.max_tokens} tokens)")
        for group in self.groups:
            for slot, n in zip(slots, new_tokens):
                group.grow(slot, self.length(slot) + n)
            group.sync()

    def end_step(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """Record the new lengths; windowed groups give back pages no later query can see."""
        for slot, n in zip(slots, new_tokens):
            self.lengths[slot] += n
        for group in self.groups:
            if group.window is not None:
                for slot in slots:
                    group.release_outside_window(slot, self.length(slot))
                group.sync()

    # -- views ------------------------------------------------------------------------------------
    def line(self, line: int) -> LineView:
        need = self.needs[line]
        state = self.states.get(line)
        if line in self._line_group:
            group, index = self._line_group[line]
            keys = group.keys[index] if group.keys is not None else None
            values = group.values[index] if group.values is not None else None
            return LineView(keys, values, group.table_dev, need.window, state)
        return LineView(None, None, None, None, state)

    def check(self) -> None:
        """No slot or page is lost or held twice, and tables agree with the pools."""
        self.slots.check()
        for group in self.groups:
            group.pool.check()
            in_tables = group.table[group.table >= 0]
            if len(set(in_tables.tolist())) != len(in_tables):
                raise AssertionError("a page is held by two sequences")
            if len(in_tables) != group.pool.num_held:
                raise AssertionError(
                    f"{group.pool.num_held} pages are held but the tables name {len(in_tables)}")
            for slot in range(self.num_slots):
                if not self.slots.is_held(slot) and (group.table[slot] >= 0).any():
                    raise AssertionError(f"free slot {slot} still holds pages")

    @property
    def tokens_held(self) -> int:
        """Tokens the live sequences hold, each rounded up to whole pages (the largest group counts)."""
        return max((g.pool.num_held for g in self.groups), default=0) * PAGE_TOKENS
