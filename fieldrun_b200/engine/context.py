"""What one step knows besides its rows: who each token belongs to and where it sits.

A step is a batch of sequences; sequence ``b`` brings ``q_len[b]`` new tokens that
continue at position ``start[b]`` of cache slot ``slot[b]``.  The tokens of all
sequences lie flat, one after another.  Row ``i`` of a sequence is absolute
position ``start + i`` (src/minimax.rs:265-266, 276-278).  The same tables exist on
the host (for decisions) and on the device (for the kernels).
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch


class Workspace:
    """Named scratch tensors that are kept and reused from step to step."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._store: dict[tuple[str, torch.dtype], torch.Tensor] = {}

    def buffer(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        flat = self._store.get(key)
        if flat is None or flat.numel() < count:
            flat = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._store[key] = flat
        return flat[:count].view(*shape)

    def bytes_held(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._store.values())

    def send_ints(self, values: np.ndarray) -> torch.Tensor:
        """``values`` (int32) on the device, by one asynchronous copy out of a pinned buffer that is kept.  The
        result is this workspace's buffer of step inputs: it holds until the next call."""
        count = int(values.shape[0])
        staged = getattr(self, "_pinned", None)
        if staged is None or staged.numel() < count:
            if staged is not None:
                self._pinned_free.synchronize()
            staged = self._pinned = torch.empty(max(2 * count, 1024), dtype=torch.int32).pin_memory()
            self._pinned_free = torch.cuda.Event()
        else:
            self._pinned_free.synchronize()                # the copy before this one has left the buffer
        staged[:count] = torch.from_numpy(values)
        dev = self.buffer("step.inputs", (count,), torch.int32)
        dev.copy_(staged[:count], non_blocking=True)
        self._pinned_free.record()
        return dev


def pack_tables(slots: Sequence[int], starts: Sequence[int], q_lens: Sequence[int]) -> np.ndarray:
    """The step's tables as one int32 array: per token position, slot and sequence; per sequence slot, start
    and number of new tokens; then the running sum of the new tokens."""
    q = np.asarray(q_lens, dtype=np.int64)
    cu = np.concatenate([[0], np.cumsum(q)])
    seq_of_tok = np.repeat(np.arange(len(q)), q)
    within = np.arange(int(q.sum())) - np.repeat(cu[:-1], q)
    pos = np.repeat(np.asarray(starts, dtype=np.int64), q) + within
    slot_of_tok = np.repeat(np.asarray(slots, dtype=np.int64), q)
    return np.concatenate([pos, slot_of_tok, seq_of_tok, np.asarray(slots, dtype=np.int64),
                           np.asarray(starts, dtype=np.int64), q, cu]).astype(np.int32)


# Tiles of these many query rows come to the device with a prompt step's tables (the attention kernels' tile sizes);
# tiles of another size are made, and sent, when they are first asked for.
QUERY_TILE_ROWS = (128, 16)


def _tiles_of(q_lens: Sequence[int], rows: int) -> tuple[list[int], list[int]]:
    seqs, firsts = [], []
    for b, n in enumerate(q_lens):
        for q0 in range(0, n, rows):
            seqs.append(b)
            firsts.append(q0)
    return seqs, firsts


class StepContext:
    def __init__(self, workspace: Workspace, dtype: torch.dtype, slots: Sequence[int], starts: Sequence[int],
                 q_lens: Sequence[int], *, tables: torch.Tensor | None = None, max_kv_len: int | None = None,
                 tokens: np.ndarray | None = None, rows: Sequence[int] | None = None):
        """``tables`` (optional) is a device buffer that already holds, or will hold before the kernels run,
        what :func:`pack_tables` makes for this step; it is used instead of a fresh transfer, so that a
        recorded step can be run again with other positions and slots.  ``max_kv_len`` then bounds the
        lengths the recorded step may be run with.  Without ``tables`` everything the step's kernels need from
        the host goes to the device in one copy: the tables, the step's ``tokens`` and wanted ``rows`` if given
        (then ``tokens_dev`` and ``rows_dev``), and a prompt's query tiles."""
        self.workspace = workspace
        self.device = workspace.device
        self.dtype = dtype
        self.seq_slots = [int(s) for s in slots]
        self.seq_starts = [int(s) for s in starts]
        self.seq_q_lens = [int(q) for q in q_lens]
        self.num_seqs = len(self.seq_slots)
        self.num_tokens = int(sum(self.seq_q_lens))
        self.max_q_len = max(self.seq_q_lens, default=0)
        self.max_kv_len = max((s + q for s, q in zip(self.seq_starts, self.seq_q_lens)), default=0)
        if max_kv_len is not None:
            self.max_kv_len = max(self.max_kv_len, int(max_kv_len))
        self.is_decode = self.max_q_len == 1 and self.num_tokens == self.num_seqs
        t, b = self.num_tokens, self.num_seqs
        self._tiles: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        self.tokens_dev = self.rows_dev = None
        if tables is None:
            # one transfer for all of it
            parts = [pack_tables(self.seq_slots, self.seq_starts, self.seq_q_lens)]
            if tokens is not None:
                parts.append(np.asarray(tokens, dtype=np.int32))
            if rows is not None:
                parts.append(np.asarray(rows, dtype=np.int32))
            tiles = {}
            if self.max_q_len > 1:
                for size in QUERY_TILE_ROWS:
                    seqs, firsts = _tiles_of(self.seq_q_lens, size)
                    tiles[size] = len(seqs)
                    parts.append(np.asarray(seqs + firsts, dtype=np.int32))
            dev = workspace.send_ints(np.concatenate(parts))
            at = 3 * t + 4 * b + 1
            if tokens is not None:
                self.tokens_dev = dev[at:at + t]
                at += t
            if rows is not None and len(rows):
                self.rows_dev = dev[at:at + len(rows)]
                at += len(rows)
            for size, count in tiles.items():
                self._tiles[size] = (dev[at:at + count], dev[at + count:at + 2 * count])
                at += 2 * count
        else:
            dev = tables
            if dev.numel() != 3 * t + 4 * b + 1 or dev.dtype != torch.int32:
                raise ValueError("the step's table buffer has the wrong size")
        self.tok_pos = dev[0:t]
        self.tok_slot = dev[t:2 * t]
        self.tok_seq = dev[2 * t:3 * t]
        o = 3 * t
        self.seq_slot = dev[o:o + b]
        self.seq_start = dev[o + b:o + 2 * b]
        self.seq_q_len = dev[o + 2 * b:o + 3 * b]
        self.cu_q_len = dev[o + 3 * b:o + 4 * b + 1]

    def buffer(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.buffer(name, shape, dtype)

    def query_tiles(self, rows: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Tiles of ``rows`` consecutive new tokens that never span two sequences: (sequence of each tile,
        first row of each tile among its sequence's new tokens), on the device."""
        if rows not in self._tiles:
            seqs, firsts = _tiles_of(self.seq_q_lens, rows)
            both = torch.tensor([seqs, firsts], dtype=torch.int32).to(self.device)
            self._tiles[rows] = (both[0].contiguous(), both[1].contiguous())
        return self._tiles[rows]
