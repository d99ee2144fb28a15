"""The Python entry point, in the manner of the reference's ``Model`` trait.

The reference offers, per model: ``predict(ids) -> next id`` (src/model.rs:260),
``generate(prompt, n_new) -> ids`` (exactly n_new greedy tokens, no stop check;
src/model.rs:516, src/minimax.rs:391-414) and ``generate_stream(prompt, max_tokens,
eos, emit)`` (src/model.rs:497, src/minimax.rs:416-462); its HTTP face wraps the
same calls (``POST /generate {"prompt", "n"}``, ``/predict {"ids"}``,
src/api.rs:580-605).  The same names and meanings here, plus what a batch engine
adds: several prompts at once, a temperature and a seed.

    import fieldrun_b200 as fr
    lm = fr.load("model_dir", dtype="bfloat16", max_tokens=8192)
    lm.generate([5, 17, 3], 16)                       # -> 16 token ids
    lm.generate_batch([[5, 17, 3], [9]], max_tokens=16, eos=[2], temperature=0.8, seed=1)
"""
from __future__ import annotations

import os
from typing import Callable, Optional, Sequence

import torch

from .config import ModelConfig, load_config
from .config.registry import Architecture, architecture_for
from .engine.engine import Engine
from .engine.generate import Generated, Request, generate as run_requests
from .engine.model import DecoderModel, parse_dtype
from .sampling import SamplingParams
from .weights import FolderSource, MemorySource, RandomInit, write_model_folder


def build_model(arch: Architecture, config: ModelConfig, dtype) -> DecoderModel:
    return DecoderModel(arch.plan(config), dtype)


def write_random_model(folder: str, config: ModelConfig | dict, init: RandomInit = RandomInit()) -> None:
    """Write ``config.json`` and ``model.safetensors`` of a randomly initialised model of ``config``."""
    if isinstance(config, dict):
        arch = architecture_for(config, "config")
        config = arch.config_from_dict(config, "config")
    else:
        arch = architecture_for({"architectures": [config.architecture]}, "config")
    model = DecoderModel(arch.plan(config), torch.float32)
    write_model_folder(folder, config.to_json_dict(), model.tensor_needs(), init)


class LanguageModel:
    """A loaded model with its cache and step function."""

    def __init__(self, model: DecoderModel, config: ModelConfig, *, max_tokens: int = 8192,
                 num_slots: Optional[int] = None, device="cuda", max_batch: int = 64):
        self.model, self.config = model, config
        self.engine = Engine(model, max_tokens=max_tokens, num_slots=num_slots, device=device)
        self.max_batch = max_batch

    @property
    def eos_token_id(self) -> tuple[int, ...]:
        return tuple(self.config.eos_token_id)

    # -- the reference's calls ---------------------------------------------------------------------------
    def predict(self, ids: Sequence[int]) -> int:
        """The most likely next token after ``ids`` (src/minimax.rs:380-385)."""
        return self.generate(ids, 1)[0]

    def generate(self, prompt: Sequence[int], n_new: int) -> list[int]:
        """Exactly ``n_new`` greedy tokens; no stop token is checked (src/minimax.rs:391-414)."""
        request = Request(tuple(int(t) for t in prompt), int(n_new), ignore_eos=True)
        return run_requests(self.engine, [request], max_batch=1)[0].tokens

    def generate_stream(self, prompt: Sequence[int], max_tokens: int, eos: Sequence[int] = (),
                        emit: Optional[Callable[[int], Optional[bool]]] = None) -> list[int]:
        """Greedy tokens until a stop token (not put out), ``emit`` returning False, or ``max_tokens``
        (src/minimax.rs:441-461)."""
        request = Request(tuple(int(t) for t in prompt), int(max_tokens), eos=tuple(int(e) for e in eos))
        callback = (lambda _index, token: emit(token)) if emit is not None else None
        return run_requests(self.engine, [request], max_batch=1, emit=callback)[0].tokens

    # -- batches -------------------------------------------------------------------------------------------
    def generate_batch(self, prompts: Sequence[Sequence[int]], max_tokens: int, *, eos: Optional[Sequence[int]] = None,
                       temperature: float = 0.0, seed: int = 0, ignore_eos: bool = False,
                       emit: Optional[Callable[[int, int], Optional[bool]]] = None,
                       return_reasons: bool = False, top_k: int = 0, top_p: float = 1.0):
        """Generate for many prompts of unequal lengths; ``eos`` defaults to the configuration's stop tokens.
        With a temperature above 0 tokens are sampled, among the ``top_k`` largest logits (0: all) and the
        smallest set of them that holds ``top_p`` of the probability (1: all)."""
        SamplingParams(temperature=temperature, seed=seed, top_k=top_k, top_p=top_p)        # checks the values
        stops = tuple(int(e) for e in (self.eos_token_id if eos is None else eos))
        requests = [Request(tuple(int(t) for t in p), int(max_tokens), float(temperature), int(seed), stops,
                            ignore_eos, index, int(top_k), float(top_p)) for index, p in enumerate(prompts)]
        results: list[Generated] = run_requests(self.engine, requests, max_batch=self.max_batch, emit=emit)
        if return_reasons:
            return [r.tokens for r in results], [r.finish_reason for r in results]
        return [r.tokens for r in results]

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        """float32 logits [len(ids), vocab] of every position of one sequence run whole."""
        slot = self.engine.new_sequence()
        try:
            out = self.engine.step([slot], [list(ids)], [list(range(len(ids)))])
            self.engine.check()                 # a kernel that gave up on a wait must not pass for a result
            return out
        finally:
            self.engine.release(slot)


def load(model_dir: str, *, dtype="bfloat16", max_tokens: int = 8192, num_slots: Optional[int] = None,
         device="cuda", max_batch: int = 64) -> LanguageModel:
    """Load a model folder (config.json + safetensors); the model class is chosen by config.json."""
    if not os.path.isdir(model_dir):
        raise FileNotFoundError(f"{model_dir}: no such model folder")
    arch, config = load_config(model_dir)
    model = build_model(arch, config, dtype)
    source = FolderSource(model_dir, model.tensor_needs(), parse_dtype(dtype), device)
    try:
        model.load(source)
    finally:
        source.close()
    return LanguageModel(model, config, max_tokens=max_tokens, num_slots=num_slots, device=device, max_batch=max_batch)


def random_model(config: ModelConfig | dict, init: RandomInit = RandomInit(), *, dtype="bfloat16", max_tokens: int = 8192,
                 num_slots: Optional[int] = None, device="cuda", max_batch: int = 64) -> LanguageModel:
    """A model of ``config`` with random weights drawn on the device (nothing is written)."""
    if isinstance(config, dict):
        arch = architecture_for(config, "config")
        config = arch.config_from_dict(config, "config")
    else:
        arch = architecture_for({"architectures": [config.architecture]}, "config")
    model = build_model(arch, config, dtype)
    source = MemorySource(lambda need: init.draw(need, device), init.stored, parse_dtype(dtype), device)
    model.load(source)
    return LanguageModel(model, config, max_tokens=max_tokens, num_slots=num_slots, device=device, max_batch=max_batch)
