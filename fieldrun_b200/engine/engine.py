"""The step function: a batch of sequences, their next tokens, logits at the wanted places.

``Engine.step`` runs exactly the tokens it is given, as one batch, from what
earlier steps left in the cache, and returns float32 logits for the wanted
positions.  Sequences of a step either all bring their prompt (each from its
first token) or all bring one more token; they may have unequal lengths.  The
reference's counterpart handles one sequence: ``forward_block(emb, cur, kc, vc)``
runs m new rows at position cur (src/minimax.rs:250-287) and ``head_argmax``
projects the last row (src/minimax.rs:373-376).
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..cache import SequenceCache
from ..csrc import ops
from .context import StepContext, Workspace, pack_tables
from .model import DecoderModel

RECORD_KV_STEP = 1024          # a recorded step serves lengths up to the next multiple of this
RECORDED_STEPS_KEPT = 24       # recorded steps kept; beyond that the one unused for longest goes
# batch sizes that steps are recorded for; a step of another size runs in the next larger one (see _recorded_step)
RECORD_BATCHES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)


def record_batch(batch: int) -> int:
    """The batch size of the recorded step that a decode step of ``batch`` sequences runs in."""
    for size in RECORD_BATCHES:
        if size >= batch:
            return size
    return (batch + 255) // 256 * 256


class StepError(ValueError):
    """A step was asked for that cannot be run (bad token id, unknown slot, wanted place out of range)."""


class _RecordedStep:
    """One decode step (one token for each of ``batch`` sequences) recorded as a CUDA graph.

    Its inputs live in fixed device buffers: the tokens, and the step's tables (positions, slots).  Running
    it again means copying new tokens and tables into those buffers and launching the graph; the page
    tables are the cache's own device tensors, which the cache keeps up to date.  Launch overhead of the
    step's many small kernels disappears, which is most of a small batch's step time."""

    def __init__(self, engine: "Engine", batch: int, kv_cap: int):
        self.batch, self.kv_cap = batch, kv_cap
        count = 3 * batch + 4 * batch + 1
        self.host = torch.empty(batch + count, dtype=torch.int32).pin_memory()
        self.inputs = torch.zeros(batch + count, dtype=torch.int32, device=engine.device)
        self.tokens = self.inputs[:batch]
        self.tables = self.inputs[batch:]
        self.rows = torch.arange(batch, dtype=torch.int32, device=engine.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels = 0                                   # kernels of this library inside the graph
        self.logits: Optional[torch.Tensor] = None
        # scratch of its own: the graph holds the addresses, so no other step may ever move these buffers
        self.workspace = Workspace(engine.device)
        self.ctx = StepContext(self.workspace, engine.model.dtype, [0] * batch, [0] * batch, [1] * batch,
                               tables=self.tables, max_kv_len=kv_cap)
        self.copied = torch.cuda.Event()

    def load(self, tokens, slots: Sequence[int], starts: Sequence[int]) -> None:
        """New inputs: ``tokens`` from the host (numpy) or already on the device (tensor).  Fewer sequences
        than the recorded batch: the last one is repeated in the rows left over.  A repeated row computes what
        its original computes, bit for bit, writes the same key and value to the same place, picks the same
        experts (so no weight is read that the step would not read anyway) and its logits are never looked at."""
        real = len(slots)
        pad = self.batch - real
        if pad:
            slots = list(slots) + [slots[-1]] * pad
            starts = list(starts) + [starts[-1]] * pad
        self.copied.synchronize()                          # the last copy out of the pinned buffer is done
        self.host[self.batch:] = torch.from_numpy(pack_tables(slots, starts, [1] * self.batch))
        if isinstance(tokens, torch.Tensor):
            self.tables.copy_(self.host[self.batch:], non_blocking=True)
            if tokens.data_ptr() != self.tokens.data_ptr():
                self.tokens[:real].copy_(tokens)
            if pad:
                self.tokens[real:].copy_(self.tokens[real - 1:real].expand(pad))
        else:
            flat = np.asarray(tokens).astype(np.int32)
            self.host[:real] = torch.from_numpy(flat)
            if pad:
                self.host[real:self.batch] = int(flat[-1])
            self.inputs.copy_(self.host, non_blocking=True)
        self.copied.record()


class Engine:
    def __init__(self, model: DecoderModel, *, max_tokens: int, num_slots: Optional[int] = None, device="cuda",
                 record_steps: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("fieldrun_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.model = model
        self.device = torch.device(device)
        ops.library()                                   # build or load the kernels now, and fail here if that fails
        self.cache: SequenceCache = model.new_cache(max_tokens, num_slots, self.device)
        self.workspace = Workspace(self.device)
        self.vocab_size = model.plan.vocab_size
        self.steps_run = 0
        self.record_steps = record_steps and model.replayable
        self._recorded: dict[tuple[int, int], _RecordedStep] = {}      # in order of last use, oldest first
        self.steps_replayed = 0
        self.steps_recorded = 0
        # most prompt tokens that the generation loop puts into one step (a step's buffers grow with its tokens)
        self.prompt_tokens_per_step = 16384

    # -- sequences -------------------------------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.alloc()

    def release(self, slot: int) -> None:
        self.cache.free(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    @property
    def max_tokens(self) -> int:
        return self.cache.max_tokens

    @property
    def num_slots(self) -> int:
        return self.cache.num_slots

    # -- the step ----------------------------------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Run ``tokens[b]`` as the next tokens of sequence ``slots[b]``.

        ``want[b]`` lists places among ``tokens[b]`` whose logits are returned (default: the last place of
        each sequence).  Returns float32 ``[sum(len(want[b])), vocab]`` in the order of the sequences and of
        ``want``, or None when nothing is wanted.
        """
        if len(slots) != len(tokens):
            raise StepError(f"{len(slots)} sequences but {len(tokens)} token lists")
        if not slots:
            return None
        q_lens = [len(t) for t in tokens]
        if min(q_lens) == 0:
            raise StepError("a sequence of the step brings no token")
        flat = np.concatenate([np.asarray(t, dtype=np.int64) for t in tokens])
        if flat.min() < 0 or flat.max() >= self.vocab_size:
            bad = int(flat[(flat < 0) | (flat >= self.vocab_size)][0])
            raise StepError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
        if want is None:
            want = [[n - 1] for n in q_lens]
        if len(want) != len(slots):
            raise StepError(f"{len(slots)} sequences but {len(want)} lists of wanted places")
        rows: list[int] = []
        offset = 0
        for n, places in zip(q_lens, want):
            for place in places:
                if not 0 <= place < n:
                    raise StepError(f"wanted place {place} is outside the {n} tokens its sequence brings")
                rows.append(offset + int(place))
            offset += n
        starts = [self.cache.length(s) for s in slots]
        longest = max(s + n for s, n in zip(starts, q_lens))
        if longest > self.cache.max_tokens:
            raise StepError(f"a sequence would reach position {longest}, the position tables end at "
                            f"{self.cache.max_tokens}")

        self.cache.begin_step(slots, q_lens)               # raises before anything is launched
        if self.record_steps and max(q_lens) == 1 and rows == list(range(len(slots))):
            logits = self._recorded_step(slots, flat, starts)
            self.cache.end_step(slots, q_lens)
            self.steps_run += 1
            return logits
        ctx = StepContext(self.workspace, self.model.dtype, slots, starts, q_lens, tokens=flat, rows=rows)
        logits = self.model.forward(ctx, self.cache, ctx.tokens_dev, ctx.rows_dev)
        self.cache.end_step(slots, q_lens)
        self.steps_run += 1
        if ctx.num_tokens > len(slots):
            ops.tc_status_check(self.device)          # a kernel that gave up on a wait must not pass for a result
        return logits

    def step_on_device(self, slots: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """One more token for each sequence, the tokens being an int32 tensor on the device (the previous
        step's picks, say): no token crosses to the host.  Returns the logits of every sequence."""
        if tokens.dtype != torch.int32 or tokens.numel() != len(slots) or not tokens.is_cuda:
            raise StepError("step_on_device takes one int32 token per sequence, on the device")
        ones = [1] * len(slots)
        starts = [self.cache.length(s) for s in slots]
        if max(starts) + 1 > self.cache.max_tokens:
            raise StepError(f"a sequence would pass position {self.cache.max_tokens}, where the position tables end")
        self.cache.begin_step(slots, ones)
        if self.record_steps:
            logits = self._recorded_step(slots, tokens, starts, keep=False)[:len(slots)]
        else:
            ctx = StepContext(self.workspace, self.model.dtype, slots, starts, ones)
            rows = torch.arange(len(slots), dtype=torch.int32, device=self.device)
            logits = self.model.forward(ctx, self.cache, tokens.contiguous(), rows)
        self.cache.end_step(slots, ones)
        self.steps_run += 1
        return logits

    def check(self) -> None:
        """Raise if a kernel's bounded wait gave up since the last check (its results are then not valid).
        This reads one int from the device, so it waits for the work before it.  ``step`` checks after a
        prompt and ``pick`` with every token it brings to the host; a loop that stays on the device
        (``step_on_device``/``pick_on_device``) or reads logits only calls this once it is through."""
        ops.tc_status_check(self.device)

    def pick_on_device(self, logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The largest logit of every row, as an int32 tensor on the device."""
        if out is None:
            out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        ops.sample_rows(logits, None, None, out)
        return out

    def _recorded_step(self, slots: Sequence[int], tokens, starts: Sequence[int], keep: bool = True) -> torch.Tensor:
        """A step of one token per sequence with the logits of every sequence wanted, run from a recording.

        Steps are recorded per (batch size, length range): batch sizes come from ``RECORD_BATCHES`` and a
        step of another size runs in the next larger recording with its last sequence repeated, so a batch
        whose sequences end one after another goes through a dozen recordings, not one per size.  A
        recording is made at its key's first occurrence; ``RECORDED_STEPS_KEPT`` are kept, by last use.
        With ``keep`` the logits are copied out of the recorded step's own buffer, which the next replay
        overwrites."""
        batch = len(slots)
        longest = max(starts) + 1
        kv_cap = min((longest + RECORD_KV_STEP - 1) // RECORD_KV_STEP * RECORD_KV_STEP, self.cache.max_tokens)
        key = (record_batch(batch), kv_cap)
        step = self._recorded.pop(key, None)
        if step is None:
            while len(self._recorded) >= RECORDED_STEPS_KEPT:
                self._recorded.pop(next(iter(self._recorded)))
            step = _RecordedStep(self, key[0], kv_cap)
        self._recorded[key] = step                          # the most recently used is last
        step.load(tokens, slots, starts)
        if step.graph is None:
            # run it directly this once (this also sizes every scratch buffer), then record it for the next times
            logits = self.model.forward(step.ctx, self.cache, step.tokens, step.rows)[:batch].clone()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launches()
            with torch.cuda.graph(graph):
                step.logits = self.model.forward(step.ctx, self.cache, step.tokens, step.rows)
            step.kernels = ops.launches() - before
            ops.count_launches(-step.kernels)              # recorded, not run
            step.graph = graph
            self.steps_recorded += 1
            return logits
        step.graph.replay()
        ops.count_launches(step.kernels)
        self.steps_replayed += 1
        return step.logits[:batch].clone() if keep else step.logits[:batch]

    # -- picking tokens ------------------------------------------------------------------------------------
    def pick(self, logits: torch.Tensor, temperatures: Optional[Sequence[float]] = None,
             uniforms: Optional[Sequence[float]] = None, top_ks: Optional[Sequence[int]] = None,
             top_ps: Optional[Sequence[float]] = None) -> list[int]:
        """One token per row of logits: the largest logit where the temperature is 0, else a sample with the
        row's uniform number, among the row's ``top_ks`` largest logits (0: all) and the smallest set of them
        that holds ``top_ps`` of the probability (1: all)."""
        rows = logits.shape[0]
        # one more int: the kernels' status word comes to the host in the same copy as the tokens
        out = torch.empty(rows + 1, dtype=torch.int32, device=logits.device)
        temp_dev = uni_dev = floor = None
        logits = logits.contiguous()
        if temperatures is not None and any(t > 0 for t in temperatures):
            if uniforms is None or len(uniforms) != rows or len(temperatures) != rows:
                raise StepError("sampling needs one temperature and one uniform number per row")
            ks = list(top_ks) if top_ks is not None else [0] * rows
            ps = list(top_ps) if top_ps is not None else [1.0] * rows
            if len(ks) != rows or len(ps) != rows:
                raise StepError("sampling needs one top_k and one top_p per row")
            both = torch.tensor([list(temperatures), list(uniforms), ps], dtype=torch.float32).to(logits.device)
            temp_dev, uni_dev = both[0], both[1]
            if any(k > 0 for k in ks) or any(p < 1.0 for p in ps):
                floor = torch.empty(rows, dtype=torch.float32, device=logits.device)
                ops.sample_floor(logits, temp_dev, torch.tensor(ks, dtype=torch.int32).to(logits.device), both[2], floor)
        ops.sample_rows(logits, temp_dev, uni_dev, out[:rows], floor)
        out[rows:].copy_(ops.tc_status(self.device))
        picked = out.tolist()
        ops.tc_status_raise(self.device, picked.pop())     # a kernel that gave up on a wait must not pass for a result
        return picked
