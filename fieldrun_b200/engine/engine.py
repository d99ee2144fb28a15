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
from .context import StepContext, Workspace
from .model import DecoderModel


class StepError(ValueError):
    """A step was asked for that cannot be run (bad token id, unknown slot, wanted place out of range)."""


class Engine:
    def __init__(self, model: DecoderModel, *, max_tokens: int, num_slots: Optional[int] = None, device="cuda"):
        if not torch.cuda.is_available():
            raise RuntimeError("fieldrun_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.model = model
        self.device = torch.device(device)
        ops.library()                                   # build or load the kernels now, and fail here if that fails
        self.cache: SequenceCache = model.new_cache(max_tokens, num_slots, self.device)
        self.workspace = Workspace(self.device)
        self.vocab_size = model.plan.vocab_size
        self.steps_run = 0

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
        ctx = StepContext(self.workspace, self.model.dtype, slots, starts, q_lens)
        tokens_dev = torch.from_numpy(flat.astype(np.int32)).to(self.device)
        rows_dev = torch.tensor(rows, dtype=torch.int32, device=self.device) if rows else None
        logits = self.model.forward(ctx, self.cache, tokens_dev, rows_dev)
        self.cache.end_step(slots, q_lens)
        self.steps_run += 1
        return logits

    # -- picking tokens ------------------------------------------------------------------------------------
    def pick(self, logits: torch.Tensor, temperatures: Optional[Sequence[float]] = None,
             uniforms: Optional[Sequence[float]] = None) -> list[int]:
        """One token per row of logits: the largest logit where the temperature is 0, else a sample with the
        row's uniform number."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        temp_dev = uni_dev = None
        if temperatures is not None and any(t > 0 for t in temperatures):
            if uniforms is None or len(uniforms) != rows or len(temperatures) != rows:
                raise StepError("sampling needs one temperature and one uniform number per row")
            both = torch.tensor([list(temperatures), list(uniforms)], dtype=torch.float32).to(logits.device)
            temp_dev, uni_dev = both[0], both[1]
        ops.sample_rows(logits.contiguous(), temp_dev, uni_dev, out)
        return out.tolist()
