"""The description of a model as data: which parts make each layer, in which
order the layers run and whose cache each run reads.

An architecture turns its typed configuration into a :class:`ModelPlan`; the
engine builds the parts from it without knowing the architecture.  The
reference writes one file per architecture and repeats norm, rotary, attention
and experts in each (src/minimax.rs:31-126 beside src/rope.rs:26-108); here they
are parts chosen layer by layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: a registered kind, its constants, and the checkpoint
    names of its tensors (local name -> name in the safetensors file; a name
    may hold ``{e}`` where the part enumerates experts)."""

    kind: str
    args: Mapping[str, Any] = field(default_factory=dict)
    tensors: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A layer: a block arrangement over a mixer and a feed-forward, each behind its norm."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class RunSpec:
    """One entry of the run order.  ``layer`` indexes :attr:`ModelPlan.layers`
    (the same layer may run twice).  ``cache_line`` names the line of the cache
    this run reads; ``writes_cache`` is false for a run that reads a line which
    an earlier run wrote."""

    layer: int
    cache_line: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    run_order: tuple[RunSpec, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_id: tuple[int, ...] = ()

    def check(self) -> None:
        written: set[int] = set()
        for step, run in enumerate(self.run_order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"run order entry {step} names layer {run.layer}, the plan has {len(self.layers)}")
            if run.writes_cache:
                if run.cache_line in written:
                    raise ValueError(f"run order entry {step} writes cache line {run.cache_line} a second time")
                written.add(run.cache_line)
            elif run.cache_line not in written:
                raise ValueError(
                    f"run order entry {step} reads cache line {run.cache_line} before any entry wrote it")


def default_run_order(num_layers: int) -> tuple[RunSpec, ...]:
    """Each layer once, in order, each with a cache line of its own."""
    return tuple(RunSpec(layer=i, cache_line=i) for i in range(num_layers))
