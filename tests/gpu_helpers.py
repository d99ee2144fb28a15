"""Shared pieces of the GPU tests: model folders in temporary places, plain logits, comparisons."""
import functools
import json
import os
import tempfile

import numpy as np

import fieldrun_b200 as fr
import plain_model as pm
from tiny_configs import ALL, WRITTEN_AS_IS

# largest allowed |engine - plain| as a share of the largest |plain logit| of the compared rows
TOLERANCE = {"float32": 2e-5, "bfloat16": 2.5e-2}

_ROOT = tempfile.mkdtemp(prefix="fieldrun_b200_tests_")


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    config, init = ALL[name]
    folder = os.path.join(_ROOT, name)
    fr.write_random_model(folder, config, init)
    if name in WRITTEN_AS_IS:
        with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
            json.dump(WRITTEN_AS_IS[name], handle, indent=1)
    return folder


@functools.lru_cache(maxsize=None)
def plain_weights(name: str):
    return pm.read_model_folder(model_folder(name))


def request_tokens(name: str, length: int, seed: int) -> list[int]:
    vocab = ALL[name][0]["vocab_size"]
    return np.random.default_rng(1000 * seed + length).integers(0, vocab, size=length).tolist()


@functools.lru_cache(maxsize=None)
def _plain_run(name: str, length: int, seed: int):
    config, weights = plain_weights(name)
    s = pm.sizes_from_config(config)
    hidden, margins = pm.hidden_states(config, weights, request_tokens(name, length, seed), return_margins=True)
    head = weights["model.embed_tokens.weight"] if s["tied"] else weights["lm_head.weight"]
    return hidden @ head.astype(np.float64).T, margins.min(axis=0)


def plain_logits(name: str, length: int, seed: int) -> np.ndarray:
    return _plain_run(name, length, seed)[0]


def plain_margins(name: str, length: int, seed: int) -> np.ndarray:
    """Per token, the smallest gap over the layers between the last picked expert's choice value and the
    first one left out.  Where it is tiny, rounding may pick another expert: the router is not continuous."""
    return _plain_run(name, length, seed)[1]


def worst(got, ref) -> float:
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), "the engine produced a non-finite logit"
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


# A token whose router margin is below this may get another expert under bfloat16 rounding (the noise of a
# choice value there is about 2e-4); its row, and only its row, is then held to NEAR_TIE_FACTOR x the tolerance.
NEAR_TIE_MARGIN = {"float32": 1e-6, "bfloat16": 1.5e-3}
NEAR_TIE_FACTOR = 4.0


# with the engine's expert picks forced on the plain model the comparison is one of continuous functions: tighter
FORCED_ROUTES_TOLERANCE = 1e-2


def assert_close(got, ref, dtype: str, what: str = "", margins=None, tolerance=None) -> None:
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    worst(got, ref)
    per_row = np.abs(got - ref).max(axis=-1) / max(np.abs(ref).max(), 1e-30)
    limit = np.full(len(per_row), TOLERANCE[dtype] if tolerance is None else tolerance)
    if margins is not None:
        limit[np.asarray(margins) < NEAR_TIE_MARGIN[dtype]] *= NEAR_TIE_FACTOR
    bad = per_row > limit
    if bad.any():
        first = int(np.argmax(bad))
        margin = f", router margin there {margins[first]:.2e}" if margins is not None else ""
        raise AssertionError(f"{what}: relative error {per_row[first]:.3e} exceeds {limit[first]:.1e} ({dtype}); "
                             f"first wrong row {first} of {len(per_row)}{margin}; row errors {np.round(per_row[:40], 6)}")


@functools.lru_cache(maxsize=None)
def loaded(name: str, dtype: str, max_tokens: int = 2048, num_slots=None):
    return fr.load(model_folder(name), dtype=dtype, max_tokens=max_tokens, num_slots=num_slots)


# --------------------------------------------------------------------------- schedules of steps, with the experts picked

class RouteRecorder:
    """Records which experts the engine picks for every token of every step.  Each routed feed-forward copies
    its picks into a log on the device (``route_log``); the copy is part of a recorded step too, so decode steps
    keep running from their recordings while the picks are read.  Recordings made before the logs existed are
    dropped on the way in, those made with them on the way out."""

    def __init__(self, lm):
        self.lm = lm
        self.routes: dict = {}

    def __enter__(self):
        import torch
        engine = self.lm.engine
        engine._recorded.clear()
        self.parts = [block.feed_forward for block in self.lm.model.blocks]
        for part in self.parts:
            part.route_log = torch.zeros((engine.max_tokens, part.top_k), dtype=torch.int32, device=engine.device)
        return self

    def __exit__(self, *exc):
        self.lm.engine._recorded.clear()
        for part in self.parts:
            part.route_log = None
        return False

    def assign(self, rows):
        """``rows``: (request, position) of every token of the step just run, in the step's order."""
        logs = {id(part): part.route_log[:len(rows)].cpu().numpy().copy() for part in self.parts}
        for run, spec in enumerate(self.lm.model.plan.run_order):
            ids = logs[id(self.lm.model.blocks[spec.layer].feed_forward)]
            for t, (key, position) in enumerate(rows):
                self.routes.setdefault(key, {}).setdefault(run, {})[position] = ids[t]

    def of(self, key, length):
        per_run = self.routes[key]
        return np.stack([np.stack([per_run[run][pos] for pos in range(length)]) for run in sorted(per_run)])


def run_schedule(lm, requests, steps, recorder=None):
    """Runs ``steps``: each a list of (request, first position, end position) whose tokens go through one
    Engine.step with every place wanted.  A request gets a slot at its first step and gives it back after
    the step that brings its last token.  Returns request -> logits [length, vocab]."""
    engine = lm.engine
    slots, rows_of = {}, {key: [] for key in requests}
    for step in steps:
        for key, lo, hi in step:
            if key not in slots:
                slots[key] = engine.new_sequence()
        out = engine.step([slots[k] for k, _, _ in step], [requests[k][lo:hi] for k, lo, hi in step],
                          [list(range(hi - lo)) for _, lo, hi in step]).float().cpu().numpy()
        if recorder is not None:
            recorder.assign([(k, pos) for k, lo, hi in step for pos in range(lo, hi)])
        at = 0
        for key, lo, hi in step:
            rows_of[key].append(out[at:at + hi - lo])
            at += hi - lo
            if hi == len(requests[key]):
                engine.release(slots.pop(key))
    assert not slots, "a request of the schedule never got its last token"
    engine.cache.check()
    return {key: np.concatenate(parts) for key, parts in rows_of.items()}


ROUTE_MARGIN = 5e-3     # the engine may pick another expert than the plain model only where the choice is this close


def check_request(name, dtype, ids, logits, routes=None, what=""):
    """float32: the logits against the plain model.  bfloat16 (``routes`` given): the logits against the plain
    model made to pick the experts the engine picked -- a continuous function, so the full tolerance holds on
    every row -- and the engine's picks against the plain model's own, which may differ only at near ties."""
    config, weights = plain_weights(name)
    if routes is None:
        assert_close(logits, pm.logits_all_positions(config, weights, ids), dtype, what)
        return
    sizes = pm.sizes_from_config(config)
    hidden, margins, own = pm.hidden_states(config, weights, ids, forced_routes=routes, return_routes=True)
    head = weights["model.embed_tokens.weight"] if sizes["tied"] else weights["lm_head.weight"]
    assert_close(logits, hidden @ head.astype(np.float64).T, dtype, what,
                 tolerance=FORCED_ROUTES_TOLERANCE if dtype == "bfloat16" else None)
    differs = np.sort(own, axis=-1) != np.sort(np.asarray(routes), axis=-1)
    clear = margins > ROUTE_MARGIN
    bad = differs.any(axis=-1) & clear
    assert not bad.any(), (f"{what}: the engine picked other experts than the plain model at (layer, token) "
                           f"{np.argwhere(bad)[:5].tolist()} where the margins are {margins[bad][:5]}")
