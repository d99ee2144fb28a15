#!/usr/bin/env python3
"""Decode and prefill throughput of fieldrun_b200 at MiniMax-M2 layer sizes, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

Prints one JSON line.  A step is one decode step of a batch of --batch sequences (default 8) whose
prompts of 2,048 tokens were run first; `value` is decoded tokens a second with the tokens staying on the
device, `e2e` the same through the Python entry point with host tokens in and out every step, `e2e_loop`
whole calls of `generate_batch` (prompts included).  It also times a prefill of one 2,048-token prompt, decode
steps at batch 1 and 64 (their prompts are run too; beside the device-stepped figure the same with host tokens in
and out every step, `_e2e`), all three batch sizes again in mid-run (contexts of 3,072),
each with the bytes its step has to read and the fraction of the memory roofline, and (`long_cache`) a batch of
8 sequences of 8,192 to 65,536 tokens: their prompts and decode steps over those caches.  With --gpus above 1
it says that it is a single-GPU program and exits with 2.  `--impl reference` reports that the reference cannot
run here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# MiniMax-M2 layer sizes, 16 layers: the configuration the headline numbers are quoted on
M2 = dict(
    architectures=["MiniMaxM2ForCausalLM"], model_type="minimax_m2", hidden_size=3072, num_attention_heads=48,
    num_key_value_heads=8, head_dim=128, rotary_dim=64, rope_theta=5000000.0, use_qk_norm=True, num_local_experts=256,
    num_experts_per_tok=8, intermediate_size=1536, vocab_size=200064, rms_norm_eps=1e-6, tie_word_embeddings=False)
FULL_LAYERS = 16
PROMPT = 2048
CONTEXT = 4096
MID_RUN = 3072                                   # context of the mid-run points (decoding runs from 2,048 to 4,096)
LONG_PROMPTS = tuple(8192 * i for i in range(1, 9))   # the long-cache batch: 8,192 to 65,536 tokens
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                data = json.load(handle)
            out = dict(FALLBACK_PEAKS)
            found = 0
            for key in out:
                if isinstance(data.get(key), (int, float)) and data[key] > 0:
                    out[key] = float(data[key])
                    found += 1
            if found:
                return out, "measured" if found == len(out) else "measured where given, else fallback"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi; `window` reports the samples of a time span."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.proc = None
        self.samples: list[tuple[float, float, float, list[str]]] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clock, top = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            active = [n for n, flag in zip(self.NAMES, parts[2:6]) if flag.lower().startswith("active")]
            self.samples.append((time.time(), clock, top, active))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def window(self, begin: float, end: float) -> dict:
        if self.proc is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi gave no sample"], "samples": 0}
        inside = [s for s in self.samples if begin <= s[0] <= end]
        if not inside:                                   # a region shorter than the sampling period: the nearest sample
            inside = [min(self.samples, key=lambda s: min(abs(s[0] - begin), abs(s[0] - end)))]
        clocks = sorted(s[1] for s in inside)
        reasons = sorted({r for s in inside for r in s[3]})
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": inside[0][2], "reasons": reasons, "samples": len(inside)}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="fieldrun_b200")
    parser.add_argument("--layers", type=int, default=FULL_LAYERS)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--skip-points", action="store_true", help="leave out prefill and the batch 1/64 points")
    parser.add_argument("--skip-long-cache", action="store_true", help="leave out the batch of 8,192 to 65,536 tokens")
    parser.add_argument("--skip-loop", action="store_true", help="leave out the generate_batch timings")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust program; this image has no "
                          "cargo/rustc and no network for its crates, so it cannot be built or installed offline"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: fieldrun_b200 is a single-GPU library; --gpus {args.gpus} is not supported (run with --gpus 1)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch

    import fieldrun_b200 as fr
    from fieldrun_b200.csrc import ops

    torch.cuda.set_device(0)
    sampler = ClockSampler()
    sampler.start()
    peak, peak_source = peaks()
    config = dict(M2, num_hidden_layers=args.layers)
    largest = max(args.batch, 1 if args.skip_points else 64)
    max_tokens = largest * CONTEXT + 2 * CONTEXT
    if not args.skip_long_cache:
        max_tokens = max(max_tokens, sum(LONG_PROMPTS) + len(LONG_PROMPTS) * 512)
    t0 = time.time()
    lm = fr.random_model(config, fr.RandomInit(seed=2, matrix_std=0.02, norm_std=0.1, bias_std=0.01), dtype="bfloat16",
                         max_tokens=max_tokens, num_slots=largest + 2, max_batch=largest)
    engine = lm.engine
    model = lm.model
    cfg = lm.config
    load_s = time.time() - t0
    rng = np.random.default_rng(0)

    def prompts(n, length):
        return [rng.integers(0, cfg.vocab_size, size=length).tolist() for _ in range(n)]

    def fill(batch, length=PROMPT):
        """Sequences holding ``length`` tokens each, by running their prompts (16,384 prompt tokens a step)."""
        slots = [engine.new_sequence() for _ in range(batch)]
        first = torch.empty(batch, dtype=torch.int32, device="cuda")
        per_step = max(1, 16384 // length)
        for at in range(0, batch, per_step):
            part = slots[at:at + per_step]
            logits = engine.step(part, prompts(len(part), length))
            ops.sample_rows(logits.contiguous(), None, None, first[at:at + len(part)])
        return slots, first

    def device_step(slots, tokens_dev):
        """One decode step whose tokens come from and go to the device (the engine's recorded step)."""
        return engine.pick_on_device(engine.step_on_device(slots, tokens_dev))

    def time_decode(slots, first, steps, warmup):
        tokens = first
        for _ in range(warmup):
            tokens = device_step(slots, tokens)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = ops.launches()
        start.record()
        for _ in range(steps):
            tokens = device_step(slots, tokens)
        stop.record()
        torch.cuda.synchronize()
        engine.check()                                   # no kernel of the timed steps gave up on a wait
        return start.elapsed_time(stop) / steps, ops.launches() - before, tokens

    def point(batch, length, steps, warmup=3, host=False):
        """Decode at ``batch`` from prompts of ``length``: tokens a second, bytes a step must read, roofline share;
        with ``host`` also tokens a second through ``Engine.step``/``Engine.pick``, host tokens in and out."""
        slots, first = fill(batch, length)
        lo = engine.cache.length(slots[0]) + warmup
        ms, _, tokens = time_decode(slots, first, steps, warmup)
        step_bytes, picked = decode_bytes(slots)
        got = {}
        if host:
            host_tokens = tokens.tolist()
            for _ in range(warmup):
                host_tokens = engine.pick(engine.step(slots, [[t] for t in host_tokens]))
            torch.cuda.synchronize()
            begin = time.perf_counter()
            for _ in range(steps):
                host_tokens = engine.pick(engine.step(slots, [[t] for t in host_tokens]))
            torch.cuda.synchronize()
            got["e2e"] = round(batch * steps / (time.perf_counter() - begin), 2)
        for s in slots:
            engine.release(s)
        gbs = step_bytes / (ms * 1e-3) / 1e9
        got.update({"tok_s": round(batch * 1000.0 / ms, 2), "ms": round(ms, 4), "bytes": step_bytes, "gbs": round(gbs, 1),
                    "frac": round(gbs / peak["hbm_gbs"], 4), "experts": round(sum(picked) / max(len(picked), 1), 1),
                    "contexts": f"{lo}..{lo + steps}"})
        return got

    def decode_bytes(slots):
        """Bytes one decode step has to read: every weight it uses once (the experts actually picked, per
        layer) and the keys and values of the live sequences."""
        picked: list[int] = []
        for block in model.blocks:
            block.feed_forward.on_route = lambda ids: picked.append(int(torch.unique(ids).numel()))
        probe = rng.integers(0, cfg.vocab_size, size=len(slots)).tolist()
        recording, engine.record_steps = engine.record_steps, False        # the count needs a step run directly
        engine.step(slots, [[t] for t in probe])
        engine.record_steps = recording
        torch.cuda.synchronize()
        for block in model.blocks:
            block.feed_forward.on_route = None
        d, hd = cfg.hidden_size, cfg.head_dim
        attn = ((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * hd * d + cfg.num_attention_heads * hd * d) * 2
        router = cfg.num_local_experts * d * 4
        expert = 3 * cfg.intermediate_size * d * 2
        weights = sum(attn + router + n * expert for n in picked) + cfg.vocab_size * d * 2
        kv = sum(engine.cache.length(s) for s in slots) * 2 * cfg.num_key_value_heads * hd * 2 * len(model.blocks)
        return weights + kv, picked

    result: dict = {}

    # ---- the headline: decode at --batch ------------------------------------------------------------------
    slots, first = fill(args.batch)
    timed_contexts = f"{PROMPT + args.warmup}..{PROMPT + args.warmup + args.steps}"
    timed_from = time.time()
    ms_step, launches, tokens = time_decode(slots, first, args.steps, args.warmup)
    clocks = sampler.window(timed_from, time.time())
    value = args.batch * 1000.0 / ms_step
    step_bytes, picked = decode_bytes(slots)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    # ---- end to end: host tokens in and out through Engine.step / Engine.pick ---------------------------------
    host_tokens = tokens.tolist()
    pinned_in = torch.empty(args.batch, dtype=torch.int32).pin_memory()
    for _ in range(args.warmup):
        host_tokens = engine.pick(engine.step(slots, [[t] for t in host_tokens]))
    torch.cuda.synchronize()
    begin = time.perf_counter()
    for _ in range(args.steps):
        pinned_in.copy_(torch.tensor(host_tokens, dtype=torch.int32))
        host_tokens = engine.pick(engine.step(slots, [[t] for t in pinned_in.tolist()]))
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - begin) * 1000.0 / args.steps
    for s in slots:
        engine.release(s)

    result.update({
        "metric": "MiniMax-M2 decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens", "value": round(value, 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random weights", "impl": "fieldrun_b200",
        "config": {
            "model": "MiniMax-M2 layer sizes", "layers": args.layers, "layers_of_config": FULL_LAYERS,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "rotary_dim": cfg.rotary_dim, "experts": cfg.num_local_experts,
            "top_k": cfg.num_experts_per_tok, "expert_width": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single GPU",
            "l2": "weights read per step exceed L2", "peaks": peak_source, "timed_contexts": timed_contexts,
        },
        "e2e": {"value": round(args.batch * 1000.0 / e2e_ms, 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": 4 * args.batch + 4 * (7 * args.batch + 1), "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "bytes_per_step": step_bytes,
                     "experts_per_layer": round(sum(picked) / max(len(picked), 1), 1), "of": peak_source},
        "load_s": round(load_s, 1),
    })

    if not args.skip_points:
        # ---- prefill of one 2,048-token prompt -------------------------------------------------------------
        for attempt in range(2):                                    # the first run warms up
            slot = engine.new_sequence()
            ids = prompts(1, PROMPT)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([slot], ids)
            stop.record()
            torch.cuda.synchronize()
            prefill_ms = start.elapsed_time(stop)
            engine.release(slot)
        d, hd, nh, nkv = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
        per_layer = (2 * PROMPT * d * (nh + 2 * nkv) * hd + 4 * nh * hd * PROMPT * (PROMPT + 1) // 2 + 2 * PROMPT * nh * hd * d
                     + 2 * PROMPT * d * cfg.num_local_experts + 2 * PROMPT * cfg.num_experts_per_tok * 3 * cfg.intermediate_size * d)
        flops = per_layer * args.layers + 2 * d * cfg.vocab_size
        # 2,048 tokens with 8 picks each reach every expert of a layer, so the prompt has to read all weights once:
        # that, not the arithmetic, bounds the step.  "hbm_frac" is those bytes / time / the HBM peak.
        layer_bytes = (((nh + 2 * nkv) * hd * d + nh * hd * d) * 2 + cfg.num_local_experts * d * 4
                       + cfg.num_local_experts * 3 * cfg.intermediate_size * d * 2)
        prefill_bytes = layer_bytes * args.layers + d * cfg.vocab_size * 2
        result["prefill"] = {"value": round(PROMPT * 1000.0 / prefill_ms, 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                             "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4), "flops": flops,
                             "weight_bytes": prefill_bytes,
                             "hbm_frac": round(prefill_bytes / (prefill_ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4)}
        # ---- short prompts: their tokens reach only part of the experts, and what bounds them changes with the length --
        for length in (64, 256):
            best = None
            for attempt in range(3):                                # the first run warms up
                slot = engine.new_sequence()
                ids = prompts(1, length)
                torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                engine.step([slot], ids)
                stop.record()
                torch.cuda.synchronize()
                if attempt:
                    best = start.elapsed_time(stop) if best is None else min(best, start.elapsed_time(stop))
                engine.release(slot)
            result["prefill"][f"ms_{length}_tokens"] = round(best, 3)
            result["prefill"][f"tok_s_{length}_tokens"] = round(length * 1000.0 / best, 1)
        # ---- decode at batch 1 and 64, and every batch size again in mid-run ------------------------------------
        points = {f"decode_b{args.batch}": round(value, 2), f"decode_b{args.batch}_frac": round(achieved / peak["hbm_gbs"], 4),
                  f"decode_b{args.batch}_gbs": round(achieved, 1), f"decode_b{args.batch}_bytes": step_bytes,
                  f"decode_b{args.batch}_experts": round(sum(picked) / max(len(picked), 1), 1),
                  f"decode_b{args.batch}_contexts": timed_contexts}
        half = max(8, args.steps // 2)
        for batch, length, tag in [(1, PROMPT, ""), (64, PROMPT, "")] + [(b, MID_RUN, "_mid") for b in (1, args.batch, 64)]:
            got = point(batch, length, half, host=not tag)
            name = f"decode_b{batch}{tag}"
            points[name] = got["tok_s"]
            for key in ("frac", "gbs", "bytes", "experts", "contexts", "e2e"):
                if key in got:
                    points[f"{name}_{key}"] = got[key]
        result["points"] = points

    if not args.skip_loop:
        # ---- whole calls of generate_batch: prompts, picks and host decisions included ---------------------------
        loop = {}
        for tag, lengths in (("equal", [64] * args.batch), ("ragged", [8 + (56 * i) // max(args.batch - 1, 1) for i in range(args.batch)])):
            from fieldrun_b200.engine.generate import Request, generate
            best = None
            for attempt in range(2):                                  # the first call records the decode steps it needs
                requests = [Request(tuple(p), n, ignore_eos=True, index=i)
                            for i, (p, n) in enumerate(zip(prompts(args.batch, PROMPT), lengths))]
                torch.cuda.synchronize()
                begin = time.perf_counter()
                out = generate(engine, requests, max_batch=args.batch)
                torch.cuda.synchronize()
                best = time.perf_counter() - begin
            made = sum(len(r.tokens) for r in out)
            loop[f"{tag}_tok_s"] = round(made / best, 1)
            loop[f"{tag}_s"] = round(best, 4)
            loop[f"{tag}_new_tokens"] = made
        loop["prompts"] = f"{args.batch} x {PROMPT}"
        loop["what"] = "generate_batch wall time, prompts included; equal: 64 new tokens each; ragged: 8 to 64"
        result["e2e_loop"] = loop

    if not args.skip_long_cache:
        # ---- a batch of long sequences: prompts of 8,192 to 65,536 tokens in steps of 16,384, then decode steps -------
        from fieldrun_b200.engine.generate import prompt_steps
        slots = [engine.new_sequence() for _ in LONG_PROMPTS]
        ids = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in LONG_PROMPTS]
        first = torch.empty(len(slots), dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for pieces in prompt_steps(list(LONG_PROMPTS), engine.prompt_tokens_per_step):
            group = [i for i, _, _ in pieces]
            ends = [end == LONG_PROMPTS[i] for i, _, end in pieces]
            logits = engine.step([slots[i] for i in group], [ids[i][lo:hi] for i, lo, hi in pieces],
                                 [[hi - lo - 1] if last else [] for (_, lo, hi), last in zip(pieces, ends)])
            if logits is not None:
                done = [i for i, last in zip(group, ends) if last]
                picked_now = engine.pick_on_device(logits)
                first[torch.tensor(done, device="cuda")] = picked_now
        stop.record()
        torch.cuda.synchronize()
        engine.check()
        prompt_s = start.elapsed_time(stop) / 1000.0
        long_steps = max(8, args.steps // 2)
        ms, _, _ = time_decode(slots, first, long_steps, 3)
        step_bytes, picked = decode_bytes(slots)
        kv_bytes = sum(engine.cache.length(s) for s in slots) * 2 * cfg.num_key_value_heads * cfg.head_dim * 2 * len(model.blocks)
        for s in slots:
            engine.release(s)
        result["long_cache"] = {
            "batch": len(LONG_PROMPTS), "prompt_tokens": sum(LONG_PROMPTS), "shortest": LONG_PROMPTS[0], "longest": LONG_PROMPTS[-1],
            "layers": args.layers, "layers_of_config": 4, "prompt_s": round(prompt_s, 3),
            "prompt_tok_s": round(sum(LONG_PROMPTS) / prompt_s, 1), "decode_ms": round(ms, 4),
            "decode_tok_s": round(len(LONG_PROMPTS) * 1000.0 / ms, 2), "decode_steps_timed": long_steps,
            "cache_gb": round(kv_bytes / 1e9, 2), "bytes_per_step": step_bytes,
            "gbs": round(step_bytes / (ms * 1e-3) / 1e9, 1), "frac": round(step_bytes / (ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4),
            "experts": round(sum(picked) / max(len(picked), 1), 1)}

    sampler.stop()
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
