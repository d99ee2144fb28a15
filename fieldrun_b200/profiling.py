"""Small, self-contained workloads of the hot kernels at MiniMax-M2 layer sizes, for timing and for
profilers.

    python -m fieldrun_b200.profiling <case> [--launches N]

Each case holds between a few hundred MB and 2 GB on the device (more than the L2 cache, far less than a model), runs a few
warm-up launches and N timed ones (CUDA events), and prints the time per launch with the traffic or
arithmetic it stands for.  Cases: ``experts_tc`` (prompt-sized expert products on tcgen05: 64 rows per expert), ``experts_tc_large`` (512 rows
per expert, as in a step of 16k prompt tokens),
``experts_stream`` (decode-sized expert products: the persistent TMA-fed stream; ``experts_stream_mma``: the kernel that
loads weights into registers, kept for inner sizes that are no multiple of 64), ``attention_decode`` (pages by TMA),
``attention_decode_mma`` (pages loaded into registers), ``attention_prefill``
(mma.sync tiles of 16 queries), ``attention_prefill_tc`` (tcgen05 tiles of 128 queries; ``attention_prefill_tc_long``: one prompt of 16,384 tokens),
``decode_small_kernels`` and ``prefill_small_kernels`` (norms, routing, Q/K/V preparation for 8 and 2,048 tokens),
``step_decode`` and ``step_prefill`` (two whole layers through the engine, for launch lists; not part of ``all``),
``step_timeline`` (a replayed decode step's kernels with their start and end times, from the profiler that ships with torch;
not part of ``all``).
The reference has only wall-clock timers around whole runs (src/main.rs:3896-3906); per-kernel numbers are
this library's own.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from .csrc import ops

HIDDEN, WIDTH, HEADS, KV_HEADS, HEAD_DIM = 3072, 1536, 48, 8, 128


def _time(launch, launches: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        launch()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(launches):
        launch()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / launches


def _time_recorded(launch, launches: int) -> float:
    """Milliseconds per launch with the launches recorded into one CUDA graph, so that the host's cost of a
    call (several microseconds from Python) is not what is measured."""
    launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(launches):
            launch()
    graph.replay()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / launches


def _expert_lists(rows_per_expert: list[int], tile_rows: int, device):
    offsets = np.concatenate([[0], np.cumsum(rows_per_expert)]).astype(np.int32)
    tiles = [(e, offsets[e] + r) for e, n in enumerate(rows_per_expert) for r in range(0, n, tile_rows)]
    as_dev = lambda a: torch.tensor(a, dtype=torch.int32, device=device)
    return (as_dev([t[0] for t in tiles]), as_dev([t[1] for t in tiles]), as_dev([len(tiles)]), as_dev(offsets), len(tiles))


def experts(kind: str, launches: int) -> dict:
    dev = torch.device("cuda")
    experts_n = 64
    rows_per = {"tc": [64] * experts_n, "tc_large": [512] * experts_n}.get(kind, [1, 2] * (experts_n // 2))
    tile_rows = {"tc": 128, "tc_large": 256}.get(kind, 8)
    n = sum(rows_per)
    w13 = (torch.randn(experts_n, 2 * WIDTH, HIDDEN, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(experts_n, HIDDEN, WIDTH, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(n, HIDDEN, device=dev).to(torch.bfloat16)
    hidden = torch.empty(n, WIDTH, dtype=torch.bfloat16, device=dev)
    y = torch.empty(n, HIDDEN, dtype=torch.float32, device=dev)
    tile_expert, tile_row0, num_tiles, offsets, tiles = _expert_lists(rows_per, tile_rows, dev)

    def launch():
        if kind.startswith("tc"):
            ops.expert_gemm_tc(w13, x, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, hidden, paired=True)
            ops.expert_gemm_tc(w2, hidden, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, y, paired=False)
        elif kind == "stream_mma":
            ops.expert_gemm_mma(w13, x, None, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, hidden, paired=True,
                                **ops.stream_shape(tiles, WIDTH, HIDDEN, tile_rows, paired=True))
            ops.expert_gemm_mma(w2, hidden, None, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, y, paired=False,
                                **ops.stream_shape(tiles, HIDDEN, WIDTH, tile_rows))
        else:
            ops.weight_stream(w13, x, None, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, hidden, paired=True)
            ops.weight_stream(w2, hidden, None, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, y, paired=False,
                              lists_final=True)

    ms = _time(launch, launches)
    ops.tc_status_check(dev)
    weight_bytes = (w13.numel() + w2.numel()) * 2
    flops = 2 * n * 3 * WIDTH * HIDDEN
    return {"case": f"experts_{kind}", "ms": round(ms, 4), "experts": experts_n, "rows": n,
            "weight_gb_per_s": round(weight_bytes / ms / 1e6, 1), "tflops": round(flops / ms / 1e9, 2)}


def attention(kind: str, launches: int) -> dict:
    dev = torch.device("cuda")
    batch, context = (32, 4096) if kind.startswith("decode") else (1, 16384 if kind.endswith("_long") else 2048)
    pages_per = context // 64
    pages = batch * pages_per
    keys = (torch.randn(pages, KV_HEADS, 64, HEAD_DIM, device=dev) * 0.3).to(torch.bfloat16)
    values = (torch.randn(pages, KV_HEADS, HEAD_DIM, 64, device=dev) * 0.3).to(torch.bfloat16)
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(batch, pages_per).contiguous()
    slots = torch.arange(batch, dtype=torch.int32, device=dev)
    scale = HEAD_DIM ** -0.5
    if kind.startswith("decode"):
        q = torch.randn(batch, HEADS * HEAD_DIM, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        positions = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
        chunks = context // ops.ATTENTION_CHUNK
        part_o = torch.empty(batch, HEADS, chunks, HEAD_DIM, dtype=torch.float32, device=dev)
        part_ml = torch.empty(batch, HEADS, chunks, 2, dtype=torch.float32, device=dev)
        decode = ops.attention_decode_tma if kind == "decode" else ops.attention_decode_mma
        launch = lambda: decode(q, keys, values, table, positions, slots, part_o, part_ml, out, num_heads=HEADS,
                                num_kv_heads=KV_HEADS, head_dim=HEAD_DIM, scale=scale, window=None, max_chunks=chunks)
        ms = _time(launch, launches)
        ops.tc_status_check(dev)
        kv_bytes = (keys.numel() + values.numel()) * 2
        return {"case": "attention_" + kind, "ms": round(ms, 4), "batch": batch, "context": context,
                "kv_gb_per_s": round(kv_bytes / ms / 1e6, 1)}
    q = torch.randn(context, HEADS * HEAD_DIM, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    tiles = context // 16
    tile_seq = torch.zeros(tiles, dtype=torch.int32, device=dev)
    tile_q0 = torch.arange(0, context, 16, dtype=torch.int32, device=dev)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    q_len = torch.tensor([context], dtype=torch.int32, device=dev)
    cu = torch.tensor([0, context], dtype=torch.int32, device=dev)
    if kind.startswith("prefill_tc"):
        tile_seq = torch.zeros(context // 128, dtype=torch.int32, device=dev)
        tile_q0 = torch.arange(0, context, 128, dtype=torch.int32, device=dev)
        launch = lambda: ops.attention_prefill_tc(q, keys, values, table, tile_seq, tile_q0, zero, zero, q_len, cu, out,
                                                  num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM, scale=scale, window=None)
    else:
        launch = lambda: ops.attention_prefill_mma(q, keys, values, table, tile_seq, tile_q0, zero, zero, q_len, cu, out,
                                                   num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM, scale=scale, window=None)
    ms = _time(launch, launches)
    if kind.startswith("prefill_tc"):
        ops.tc_status_check(dev)
    flops = 4 * HEADS * HEAD_DIM * context * (context + 1) // 2
    return {"case": f"attention_{kind}", "ms": round(ms, 4), "tokens": context, "tflops": round(flops / ms / 1e9, 2)}


def small_kernels(launches: int, tokens: int) -> dict:
    """The kernels around the matrix products of a step of `tokens` tokens (8: a decode step of 8 sequences;
    2048: a prompt), each launched back to back from one CUDA graph.  Microseconds per launch."""
    dev = torch.device("cuda")
    launches = max(launches, 200 if tokens <= 64 else 20)   # a replay's own cost, spread over few launches, would show
    experts_n, top_k = 256, 8
    out = {"case": "decode_small_kernels" if tokens <= 64 else "prefill_small_kernels", "tokens": tokens}
    us = lambda launch: round(1000 * _time_recorded(launch, launches), 2)
    x = torch.randn(tokens, HIDDEN, device=dev)
    delta = torch.randn(tokens, HIDDEN, device=dev)
    weight = torch.ones(HIDDEN, device=dev)
    act = torch.empty(tokens, HIDDEN, dtype=torch.bfloat16, device=dev)
    act32 = torch.empty(tokens, HIDDEN, device=dev)
    out["rmsnorm_us"] = us(lambda: ops.rmsnorm(x, weight, 1e-6, act, delta=delta, out32=act32, write_back=True))
    router = torch.randn(experts_n, HIDDEN, device=dev) * 0.02
    bias = torch.zeros(experts_n, device=dev)
    n = tokens * top_k
    i32 = lambda k: torch.zeros(k, dtype=torch.int32, device=dev)
    ids, weights = torch.zeros(tokens, top_k, dtype=torch.int32, device=dev), torch.zeros(tokens, top_k, device=dev)
    lists = [i32(experts_n + 1), i32(n), i32(n), i32(n + experts_n), i32(n + experts_n), i32(1)]
    logits = torch.randn(tokens, experts_n, device=dev)
    if tokens <= ops.ROUTER_SMALL_TOKENS:
        scratch = torch.empty(tokens, experts_n, device=dev)
        out["router_small_us"] = us(lambda: ops.router_small(act32, router, scratch, bias, top_k, True, 1.0, 8, ids, weights, *lists))
    if tokens <= ops.SMALL_ROUTE_TOKENS:
        out["route_plan_small_us"] = us(lambda: ops.route_plan_small(logits, bias, top_k, True, 1.0, 8, ids, weights, *lists))
    out["router_topk_us"] = us(lambda: ops.router_topk(logits, bias, top_k, True, 1.0, ids, weights))
    counts = i32(((n + 1023) // 1024) * experts_n)
    out["expert_plan_us"] = us(lambda: ops.expert_plan(ids, experts_n, 8, counts, *lists))
    qkv = torch.randn(tokens, (HEADS + 2 * KV_HEADS) * HEAD_DIM, device=dev)
    qw, kw = torch.ones(HEADS * HEAD_DIM, device=dev), torch.ones(KV_HEADS * HEAD_DIM, device=dev)
    positions = 4096
    cos, sin = torch.ones(positions, 32, device=dev), torch.zeros(positions, 32, device=dev)
    if tokens <= 64:         # one token each of `tokens` sequences, deep in their contexts
        pos = torch.full((tokens,), 3000, dtype=torch.int32, device=dev)
        slots = torch.arange(tokens, dtype=torch.int32, device=dev)
        pages = tokens * 64
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(tokens, 64).contiguous()
    else:                    # one prompt
        pos = torch.arange(tokens, dtype=torch.int32, device=dev)
        slots = torch.zeros(tokens, dtype=torch.int32, device=dev)
        pages = (tokens + 63) // 64
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages).contiguous()
    keys = torch.zeros(pages, KV_HEADS, 64, HEAD_DIM, dtype=torch.bfloat16, device=dev)
    values = torch.zeros(pages, KV_HEADS, HEAD_DIM, 64, dtype=torch.bfloat16, device=dev)
    q = torch.empty(tokens, HEADS * HEAD_DIM, dtype=torch.bfloat16, device=dev)
    out["qkv_prepare_us"] = us(lambda: ops.qkv_prepare(qkv, qw, kw, 1e-6, cos, sin, pos, slots, table, q, keys, values,
                                                       num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM, rotary_dim=64,
                                                       interleaved=False, write_cache=True))
    y = torch.randn(n, HIDDEN, device=dev)
    rowmap = torch.arange(n, dtype=torch.int32, device=dev)
    out["rmsnorm_with_experts_us"] = us(lambda: ops.rmsnorm(x, weight, 1e-6, act, out32=act32, write_back=True,
                                                            experts=(y, weights.abs() + 0.1, rowmap)))
    return out


def whole_step(kind: str, launches: int, batch: int = 8) -> dict:
    """Two layers of MiniMax-M2's sizes stepped through the engine: ``step_decode`` runs `launches` decode steps
    of 8 sequences over 2,048-token contexts, ``step_prefill`` one prompt of 2,048 tokens `launches` times.  The
    measured steps lie between cudaProfilerStart and cudaProfilerStop, so that
    ``ncu --profile-from-start off --metrics gpu__time_duration.sum`` lists their kernels and nothing else."""
    from . import RandomInit, random_model
    config = {"architectures": ["MiniMaxM2ForCausalLM"], "hidden_size": HIDDEN, "num_hidden_layers": 2,
              "num_attention_heads": HEADS, "num_key_value_heads": KV_HEADS, "head_dim": HEAD_DIM, "rotary_dim": 64,
              "rope_theta": 5e6, "use_qk_norm": True, "num_local_experts": 256, "num_experts_per_tok": 8,
              "intermediate_size": WIDTH, "vocab_size": 200064, "rms_norm_eps": 1e-6, "tie_word_embeddings": False}
    batch, prompt = (batch, 2048) if kind == "decode" else (1, 2048)
    lm = random_model(config, RandomInit(seed=2, bias_std=0.01), dtype="bfloat16", max_tokens=(batch + 1) * (prompt + 128),
                      num_slots=batch + 1)
    engine = lm.engine
    engine.record_steps = False                      # run directly: every kernel is a launch of its own
    rng = np.random.default_rng(0)
    prompts = lambda n: [rng.integers(0, 200064, size=prompt).tolist() for _ in range(n)]
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if kind == "decode":
        slots = [engine.new_sequence() for _ in range(batch)]
        tokens: list[int] = []
        for first in range(0, batch, 8):                   # eight prompts to a step keep its buffers small
            group = slots[first:first + 8]
            tokens += engine.pick(engine.step(group, prompts(len(group))))
        for _ in range(3):
            tokens = engine.pick(engine.step(slots, [[t] for t in tokens]))
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        begin.record()
        for _ in range(launches):
            tokens = engine.pick(engine.step(slots, [[t] for t in tokens]))
        end.record()
    else:
        for _ in range(2):
            slot = engine.new_sequence()
            engine.step([slot], prompts(1))
            engine.release(slot)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        begin.record()
        for _ in range(launches):
            slot = engine.new_sequence()
            engine.step([slot], prompts(1))
            engine.release(slot)
        end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return {"case": f"step_{kind}", "layers": 2, "batch": batch, "context": prompt,
            "ms_per_step_with_host": round(begin.elapsed_time(end) / launches, 3)}


def step_timeline(launches: int, batch: int = 8) -> dict:
    """Three layers of MiniMax-M2's sizes, `batch` sequences over 2,048-token contexts: the start and end of every kernel
    of a decode step that is replayed from its recording, as the profiler that ships with torch records them (CUPTI).
    Kernels that start early overlap; what a kernel costs the step is the time from the end of the kernel before it to
    its own end, which is printed for the middle layer (the first follows the embedding, the last is followed by the
    head).  Times under the profiler run a few percent long."""
    from torch.profiler import ProfilerActivity, profile
    from . import RandomInit, random_model
    layers, prompt = 3, 2048
    config = {"architectures": ["MiniMaxM2ForCausalLM"], "hidden_size": HIDDEN, "num_hidden_layers": layers,
              "num_attention_heads": HEADS, "num_key_value_heads": KV_HEADS, "head_dim": HEAD_DIM, "rotary_dim": 64,
              "rope_theta": 5e6, "use_qk_norm": True, "num_local_experts": 256, "num_experts_per_tok": 8,
              "intermediate_size": WIDTH, "vocab_size": 200064, "rms_norm_eps": 1e-6, "tie_word_embeddings": False}
    lm = random_model(config, RandomInit(seed=2, bias_std=0.01), dtype="bfloat16", max_tokens=(batch + 1) * (prompt + 128),
                      num_slots=batch + 1)
    engine = lm.engine
    rng = np.random.default_rng(0)
    slots = [engine.new_sequence() for _ in range(batch)]
    tokens: list[int] = []
    for first in range(0, batch, 8):
        group = slots[first:first + 8]
        tokens += engine.pick(engine.step(group, [rng.integers(0, 200064, size=prompt).tolist() for _ in group]))
    on_device = torch.tensor(tokens, dtype=torch.int32, device="cuda")
    for _ in range(4):                                     # the first of these records the step
        on_device = engine.pick_on_device(engine.step_on_device(slots, on_device))
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(max(launches, 1)):
            on_device = engine.pick_on_device(engine.step_on_device(slots, on_device))
        torch.cuda.synchronize()
    engine.check()
    kernels = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda e: e.time_range.start)
    last_step = [i for i, e in enumerate(kernels) if "embed_rows" in e.name][-1]
    kernels = kernels[last_step:]
    zero = kernels[0].time_range.start
    by_end = sorted(kernels, key=lambda e: e.time_range.end)
    per_layer = (len(kernels) - 3) // layers               # embedding, head and pick stand outside the layers
    rows, before = [], None
    for index, e in enumerate(by_end):
        end = e.time_range.end - zero
        if 1 + per_layer < index <= 1 + 2 * per_layer:     # the middle layer, from the kernel after its first norm on
            rows.append({"kernel": e.name.split("(")[0].replace("void ", "")[:48], "starts_us": round(e.time_range.start - zero, 1),
                         "ends_us": round(end, 1), "adds_us": round(end - before, 1)})
        before = end
    return {"case": "step_timeline", "layers": layers, "batch": batch, "context": prompt,
            "step_us": round(by_end[-1].time_range.end - zero, 1), "layer_us": round(sum(r["adds_us"] for r in rows), 1),
            "middle_layer": rows}


CASES = {
    "experts_tc": lambda n: experts("tc", n),
    "experts_tc_large": lambda n: experts("tc_large", n),
    "experts_stream": lambda n: experts("stream", n),
    "experts_stream_mma": lambda n: experts("stream_mma", n),
    "attention_decode": lambda n: attention("decode", n),
    "attention_decode_mma": lambda n: attention("decode_mma", n),
    "attention_prefill": lambda n: attention("prefill", n),
    "attention_prefill_tc": lambda n: attention("prefill_tc", n),
    "attention_prefill_tc_long": lambda n: attention("prefill_tc_long", n),
    "step_decode": lambda n, batch=8: whole_step("decode", n, batch),
    "step_prefill": lambda n: whole_step("prefill", n),
    "step_timeline": lambda n, batch=8: step_timeline(n, batch),
    "decode_small_kernels": lambda n: small_kernels(n, 8),
    "prefill_small_kernels": lambda n: small_kernels(n, 2048),
}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("case", choices=sorted(CASES) + ["all"])
    parser.add_argument("--launches", type=int, default=5)
    parser.add_argument("--batch", type=int, default=8, help="sequences of step_decode and step_timeline")
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("fieldrun_b200.profiling needs a CUDA device")
    torch.manual_seed(0)
    for name in ([c for c in sorted(CASES) if not c.startswith("step_")] if args.case == "all" else [args.case]):
        print(json.dumps(CASES[name](args.launches, args.batch) if name in ("step_decode", "step_timeline")
                         else CASES[name](args.launches)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
