"""bin/trace_run driven as a user drives it: a trace on standard input, logits in files.  The same requests
whole, with their last 32 tokens one by one, and in batches of unequal lengths through a small cache, in
float32 and in bfloat16, against the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from gpu_helpers import assert_close, model_folder, plain_logits, plain_margins, request_tokens
from tiny_configs import ALL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = [70, 33, 129, 40, 5]


def replay(name, dtype, steps, out_dir, max_tokens):
    """Runs the steps; returns {step: logits [wanted, vocab]}."""
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folder(name), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)], input=text, capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    vocab = ALL[name][0]["vocab_size"]
    out = {}
    for s in steps:
        path = os.path.join(out_dir, f"{s['step']}.f32")
        wanted = sum(len(e["want"]) for e in s["entries"])
        assert os.path.exists(path) == (wanted > 0)
        if wanted:
            out[s["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
    return out


def rounded(n):
    return (n + 63) // 64 * 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "e"])
def test_three_ways_of_cutting_the_same_requests(tmp_path, name, dtype):
    ids = {i: request_tokens(name, n, 7) for i, n in enumerate(LENGTHS)}
    refs = {i: plain_logits(name, n, 7) for i, n in enumerate(LENGTHS)}
    margins = {i: plain_margins(name, n, 7) for i, n in enumerate(LENGTHS)}

    # 1. each request alone and whole
    steps = [{"step": i, "entries": [{"id": f"r{i}", "tokens": ids[i], "want": list(range(len(ids[i])))}], "end": [f"r{i}"]}
             for i in ids]
    out = replay(name, dtype, steps, tmp_path / "whole", rounded(max(LENGTHS)))
    for i in ids:
        assert_close(out[i], refs[i], dtype, f"{name} request {i} whole", margins[i])

    # 2. the last 32 tokens one by one (requests of at most 32 tokens: from their second token)
    steps, where, step = [], {}, 0
    for i, tokens in ids.items():
        head = max(len(tokens) - 32, 1)
        steps.append({"step": step, "entries": [{"id": f"r{i}", "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        where[i] = [step]
        step += 1
        for j in range(head, len(tokens)):
            steps.append({"step": step, "entries": [{"id": f"r{i}", "tokens": [tokens[j]], "want": [0]}],
                          "end": [f"r{i}"] if j == len(tokens) - 1 else []})
            where[i].append(step)
            step += 1
    out = replay(name, dtype, steps, tmp_path / "tail", rounded(max(LENGTHS)))
    for i in ids:
        assert_close(np.concatenate([out[s] for s in where[i]]), refs[i], dtype, f"{name} request {i}, tail one by one", margins[i])

    # 3. batches of unequal lengths, shorter requests ending earlier, one batch after another in a cache that
    #    holds one batch only, so that slots and pages are used again
    batches = [[0, 1, 2], [3, 4]]
    decoded = {0: 9, 1: 20, 2: 3, 3: 39, 4: 1}
    steps, rows, step = [], {i: [] for i in ids}, 0
    for batch in batches:
        heads = {i: len(ids[i]) - decoded[i] for i in batch}
        steps.append({"step": step, "entries": [{"id": f"r{i}", "tokens": ids[i][:heads[i]], "want": list(range(heads[i]))}
                                                for i in batch], "end": []})
        at = 0
        for i in batch:
            rows[i].append((step, at, at + heads[i]))
            at += heads[i]
        step += 1
        for k in range(max(decoded[i] for i in batch)):
            live = [i for i in batch if k < decoded[i]]
            steps.append({"step": step, "entries": [{"id": f"r{i}", "tokens": [ids[i][heads[i] + k]], "want": [0]} for i in live],
                          "end": [f"r{i}" for i in live if k == decoded[i] - 1]})
            for row, i in enumerate(live):
                rows[i].append((step, row, row + 1))
            step += 1
    capacity = max(sum(rounded(len(ids[i])) for i in batch) for batch in batches)
    out = replay(name, dtype, steps, tmp_path / "batches", capacity)
    for i in ids:
        got = np.concatenate([out[s][a:b] for s, a, b in rows[i]])
        assert_close(got, refs[i], dtype, f"{name} request {i} in a batch", margins[i])


def test_a_step_that_wants_nothing_writes_no_file_and_a_full_cache_is_an_error(tmp_path):
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": [4], "want": [0]}], "end": ["x"]}]
    out = replay("a", "float32", steps, tmp_path / "o", 64)
    assert list(out) == [1]
    # the step that wanted nothing still ran its tokens: position 3's logits are those of the four tokens together
    import plain_model as pm
    from gpu_helpers import plain_weights
    config, weights = plain_weights("a")
    assert_close(out[1], pm.logits_all_positions(config, weights, [1, 2, 3, 4])[3:], "float32", "the token after a silent step")
    text = json.dumps({"step": 0, "entries": [{"id": "y", "tokens": list(range(100)), "want": [99]}], "end": []}) + "\n"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folder("a"), "--dtype", "float32",
                           "--out", str(tmp_path / "p"), "--max-tokens", "64"], input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and ("position tables end" in proc.stderr or "pages" in proc.stderr)
