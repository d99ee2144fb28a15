"""Command line, with the reference's option names where it has them.

The reference's one-shot path is ``fieldrun --bundle <stem> --ids <ids.json> --ctx N
--generate M`` (src/main.rs:446-450, 3894-3908): the prompt is the first ``--ctx``
ids (default 64) of ``{"holdout_ids": [...]}``; without ``--generate`` it scores
next-token top-1 over ``--n-eval`` positions (default 500) with a sliding context
and ``--dump`` writes the predictions one id per line (src/main.rs:3933-3941,
4096-4104).  Here ``--model`` names a model folder (``--bundle`` is accepted for
it), and ``--temperature``, ``--seed``, ``--top-k``, ``--top-p``, ``--eos``, ``--dtype`` and ``--prompts`` are
what a batch engine with sampling adds; ``--device cpu`` and ``--kv-int8`` are recognised and refused with a reason.  ``random`` writes a model folder with
random weights, the counterpart of the reference's offline ``convert`` step.

    python -m fieldrun_b200 --model DIR --ids ids.json --ctx 64 --generate 32
    python -m fieldrun_b200 --model DIR --prompts prompts.json --generate 32 --temperature 0.8 --seed 1
    python -m fieldrun_b200 random --config config.json --seed 0 -o DIR
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _read_ids(path: str) -> list[int]:
    with open(path, "r", encoding="utf-8") as handle:
        data = json.load(handle)
    if isinstance(data, dict) and "holdout_ids" in data:
        data = data["holdout_ids"]
    if not isinstance(data, list) or not all(isinstance(t, int) for t in data):
        raise SystemExit(f'[fieldrun_b200] {path}: expected {{"holdout_ids": [<token ids>]}} or a list of ids')
    return data


def _random(argv: list[str]) -> int:
    from . import RandomInit, write_random_model
    parser = argparse.ArgumentParser(prog="fieldrun_b200 random", description="write a model folder with random weights")
    parser.add_argument("--config", required=True, help="a config.json of a registered architecture")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--std", type=float, default=0.02, help="std of projections, experts, embedding, head")
    parser.add_argument("--norm-std", type=float, default=0.1, help="norm weights are 1 + N(0, norm-std)")
    parser.add_argument("--bias-std", type=float, default=0.0, help="routing bias is N(0, bias-std)")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="stored dtype of matrices")
    parser.add_argument("-o", "--out", required=True)
    args = parser.parse_args(argv)
    import torch
    with open(args.config, "r", encoding="utf-8") as handle:
        config = json.load(handle)
    init = RandomInit(seed=args.seed, matrix_std=args.std, norm_std=args.norm_std, bias_std=args.bias_std,
                      stored_dtype=torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    write_random_model(args.out, config, init)
    print(f"[fieldrun_b200] wrote {args.out}/config.json and model.safetensors (seed {args.seed})")
    return 0


def main(argv: list[str] | None = None) -> int:
    """Runs the command; an error the user can act on becomes one line and exit status 1, as the reference
    turns its panics into one-line messages (src/main.rs:115-126)."""
    try:
        return _main(argv)
    except (OSError, ValueError, RuntimeError, KeyError) as err:
        print(f"[fieldrun_b200] error: {err}", file=sys.stderr)
        return 1


def _main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "random":
        return _random(argv[1:])
    parser = argparse.ArgumentParser(prog="fieldrun_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", "--bundle", dest="model", required=True, help="model folder (config.json + safetensors)")
    parser.add_argument("--ids", help='token ids: {"holdout_ids": [...]}')
    parser.add_argument("--prompts", help="several prompts: a JSON list of lists of token ids")
    parser.add_argument("--ctx", type=int, default=64, help="prompt = the first N ids / scoring context (default 64)")
    parser.add_argument("--generate", type=int, help="generate M tokens")
    parser.add_argument("--n-eval", type=int, default=500, help="positions to score (default 500)")
    parser.add_argument("--dump", help="write predictions or generated tokens, one id per line")
    parser.add_argument("--logits-dump", help="write the logits of every position of the prompt (the first --ctx ids): "
                        "little-endian float32 [positions, vocab], as the reference's option of this name does")
    parser.add_argument("--max-tokens", type=int, default=0, help="cache size in tokens (default: what the run needs)")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--temperature", type=float, default=0.0, help="0 picks the largest logit")
    parser.add_argument("--seed", type=int, default=0, help="seed of temperature sampling")
    parser.add_argument("--top-k", type=int, default=0, help="sample among the k largest logits only (0: all)")
    parser.add_argument("--top-p", type=float, default=1.0, help="sample among the smallest set of tokens holding this probability")
    parser.add_argument("--eos", default=None, help="stop token ids, comma separated (default: the config's; 'none')")
    parser.add_argument("--batch", type=int, default=64, help="most sequences in one batch")
    parser.add_argument("--device", default="auto", choices=["auto", "gpu", "cpu"],
                        help="the reference's switch (src/main.rs:4036-4094); this library runs on the GPU only")
    parser.add_argument("--kv-int8", action="store_true", help="the reference's 8-bit cache; not part of this library")
    parser.add_argument("--profile", action="store_true",
                        help="time every kernel with CUDA events (steps run directly, slower) and print the sums as JSON lines")
    args = parser.parse_args(argv)
    if args.device == "cpu":
        raise SystemExit("[fieldrun_b200] --device cpu: this library has no CPU path; it runs on one CUDA device (sm_100a)")
    if args.kv_int8:
        raise SystemExit("[fieldrun_b200] --kv-int8: quantized caches are not part of this library; the cache holds the model's dtype")

    import fieldrun_b200 as fr

    if args.prompts:
        with open(args.prompts, "r", encoding="utf-8") as handle:
            prompts = json.load(handle)
        if args.generate is None:
            raise SystemExit("[fieldrun_b200] --prompts needs --generate M")
    elif args.ids:
        ids = _read_ids(args.ids)
        prompts = [ids[:min(args.ctx, len(ids))]]
    else:
        raise SystemExit("[fieldrun_b200] give --ids <ids.json> or --prompts <prompts.json>")

    if args.logits_dump:
        need = (len(prompts[0]) + 63) // 64 * 64
    elif args.generate is not None:
        new = args.generate
        need = sum((len(p) + new + 63) // 64 * 64 for p in prompts[:args.batch])
    else:
        need = min(args.batch, args.n_eval) * ((args.ctx + 64) // 64 * 64)
    lm = fr.load(args.model, dtype=args.dtype, max_tokens=max(args.max_tokens, need, 64), max_batch=args.batch)

    if args.logits_dump:
        # every position's logits of one sequence run whole (src/main.rs:1146-1156 runs each prefix anew)
        logits = lm.logits(prompts[0]).cpu().numpy().astype("<f4")
        logits.tofile(args.logits_dump)
        print(f"[fieldrun_b200] --logits-dump: {logits.shape[0]} positions x {logits.shape[1]} (f32 LE) -> {args.logits_dump}")
        return 0

    if args.generate is not None:
        if args.eos is None:
            eos = None
        elif args.eos.lower() == "none":
            eos = []
        else:
            eos = [int(t) for t in args.eos.split(",") if t]
        if args.profile:
            from .csrc import ops
            lm.engine.record_steps = False                   # a replayed step is one launch: nothing to tell apart
            ops.timing_start()
        started = time.perf_counter()
        outputs = lm.generate_batch(prompts, args.generate, eos=eos, temperature=args.temperature, seed=args.seed,
                                    ignore_eos=(eos == []), top_k=args.top_k, top_p=args.top_p)
        seconds = time.perf_counter() - started
        if args.profile:
            report = ops.timing_report()
            total = sum(ms for _, ms in report.values()) or 1.0
            for name, (launches, ms) in sorted(report.items(), key=lambda item: -item[1][1]):
                print(json.dumps({"kernel": name, "launches": launches, "ms": round(ms, 3), "share": round(ms / total, 4)}),
                      file=sys.stderr)
        total = sum(len(o) for o in outputs)
        for prompt, output in zip(prompts, outputs):
            print(f"[fieldrun_b200] generate {len(output)} tokens from a {len(prompt)}-token prompt")
            print(" ".join(str(t) for t in output))
        print(f"[fieldrun_b200]   {seconds:.2f}s  ({total / max(seconds, 1e-9):.1f} tok/s)")
        if args.dump:
            with open(args.dump, "w", encoding="utf-8") as handle:
                for output in outputs:
                    handle.writelines(f"{t}\n" for t in output)
        return 0

    # scoring: predict ids[i] from ids[i-ctx:i] for n_eval positions
    end = min(args.ctx + args.n_eval, len(ids))
    contexts = [ids[max(0, i - args.ctx):i] for i in range(args.ctx, end)]
    started = time.perf_counter()
    predictions = [o[0] for o in lm.generate_batch(contexts, 1, ignore_eos=True)]
    seconds = time.perf_counter() - started
    correct = sum(int(p == ids[i]) for p, i in zip(predictions, range(args.ctx, end)))
    print(f"[fieldrun_b200] top-1 {correct}/{len(predictions)}")
    print(f"[fieldrun_b200] throughput: {len(predictions) / max(seconds, 1e-9):.1f} forwards/s")
    if args.dump:
        with open(args.dump, "w", encoding="utf-8") as handle:
            handle.writelines(f"{p}\n" for p in predictions)
    return 0
