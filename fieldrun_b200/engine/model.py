"""A decoder put together from a plan: embedding, the runs of the run order, final norm, head.

The model owns the parts and their tensors; it knows nothing of requests.  One
call of :meth:`DecoderModel.forward` runs the rows of one step through every run
of the plan and returns float32 logits for the rows that were asked for
(the reference projects only a sequence's last row, src/minimax.rs:373-376; the
final norm and the head run here on the asked rows only, too).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed, SequenceCache
from ..config.plan import ModelPlan
from ..parts import build_block, build_part
from ..parts.linear import require_true_float32
from ..weights.loader import TensorNeed, TensorSource
from .context import StepContext

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the model runs in bfloat16 or float32, not {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r} is neither bfloat16 nor float32") from None


class DecoderModel:
    def __init__(self, plan: ModelPlan, dtype):
        plan.check()
        self.plan = plan
        self.dtype = parse_dtype(dtype)
        self.embedding = build_part("embedding", plan.embedding, self.dtype)
        self.blocks = []
        for layer in plan.layers:
            self.blocks.append(build_block(
                layer.block,
                build_part("mixer", layer.mixer, self.dtype),
                build_part("feed_forward", layer.feed_forward, self.dtype),
                build_part("norm", layer.mixer_norm, self.dtype),
                build_part("norm", layer.feed_forward_norm, self.dtype)))
        self.final_norm = build_part("norm", plan.final_norm, self.dtype)
        self.head = build_part("head", plan.head, self.dtype)
        self.head_is_tied = plan.head.tensors.get("weight") == plan.embedding.tensors.get("weight")
        self.loaded = False

    # -- tensors -------------------------------------------------------------------------------------
    def all_parts(self):
        parts = [self.embedding]
        for block in self.blocks:
            parts.extend(block.parts())
        parts.append(self.final_norm)
        parts.append(self.head)
        return parts

    def tensor_needs(self) -> list[TensorNeed]:
        needs: list[TensorNeed] = []
        for part in self.all_parts():
            needs.extend(part.tensor_needs())
        return needs

    def load(self, source: TensorSource) -> None:
        if self.dtype == torch.float32:
            require_true_float32()
        self.embedding.load(source)
        for block in self.blocks:
            for part in block.parts():
                part.load(source)
        self.final_norm.load(source)
        if self.head_is_tied:
            self.head.load(source, shared=self.embedding.weight)
        else:
            self.head.load(source)
        self.loaded = True

    @property
    def replayable(self) -> bool:
        """Whether a step of this model can be recorded once and run again (see ``Part.replayable``)."""
        return all(part.replayable for part in self.all_parts())

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for part in self.all_parts():
            for value in vars(part).values():
                if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
                    seen.add(value.data_ptr())
                    total += value.numel() * value.element_size()
        return total

    # -- cache ---------------------------------------------------------------------------------------
    def cache_needs(self) -> list[CacheNeed]:
        """What each cache line needs, indexed by line id."""
        lines = max((run.cache_line for run in self.plan.run_order), default=-1) + 1
        needs: list[Optional[CacheNeed]] = [None] * lines
        for run in self.plan.run_order:
            need = self.blocks[run.layer].mixer.cache_need()
            if run.writes_cache:
                needs[run.cache_line] = need
            elif needs[run.cache_line] != need:
                raise ValueError(
                    f"layer {run.layer} reads cache line {run.cache_line}, whose writer needs {needs[run.cache_line]}, "
                    f"but itself needs {need}")
        return [n if n is not None else CacheNeed() for n in needs]

    def new_cache(self, max_tokens: int, num_slots: Optional[int] = None, device="cuda") -> SequenceCache:
        cache = SequenceCache(self.cache_needs(), max_tokens=max_tokens, num_slots=num_slots, dtype=self.dtype,
                              device=device)
        for block in self.blocks:
            block.mixer.prepare(cache.max_tokens, device)
        return cache

    # -- one step --------------------------------------------------------------------------------------
    def forward(self, ctx: StepContext, cache: SequenceCache, tokens: torch.Tensor,
                logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if not self.loaded:
            raise RuntimeError("the model has no weights yet")
        x = self.embedding.forward(ctx, tokens)
        pending = None
        for run in self.plan.run_order:
            x, pending = self.blocks[run.layer].forward(ctx, x, pending, cache.line(run.cache_line), run.writes_cache)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        act, _ = self.final_norm.forward(ctx, x, delta=pending, rows=logit_rows, write_back=False)
        return self.head.forward(ctx, act)
