"""The command line as a user runs it: a model folder written by `random`, token ids in the reference's
{"holdout_ids": [...]} form, `--generate`, scoring with `--dump`, several prompts with a temperature."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_model as pm
from tiny_configs import CONFIG_A

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    proc = subprocess.run([sys.executable, "-m", "fieldrun_b200", *args], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return proc.stdout


def test_random_generate_score_and_dump(tmp_path):
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(CONFIG_A))
    folder = str(tmp_path / "model")
    out = run("random", "--config", str(config_path), "--seed", "3", "--norm-std", "0.1", "-o", folder)
    assert "wrote" in out and os.path.isfile(os.path.join(folder, "model.safetensors"))
    config, weights = pm.read_model_folder(folder)
    ids = np.random.default_rng(5).integers(0, 255, size=40).tolist()
    ids_path = tmp_path / "ids.json"
    ids_path.write_text(json.dumps({"holdout_ids": ids}))

    dump = tmp_path / "gen.txt"
    out = run("--model", folder, "--ids", str(ids_path), "--ctx", "12", "--generate", "6", "--dtype", "float32", "--eos", "none",
              "--dump", str(dump))
    want = pm.generate_greedy(config, weights, ids[:12], 6)
    assert "generate 6 tokens from a 12-token prompt" in out and " ".join(map(str, want)) in out
    assert [int(t) for t in dump.read_text().split()] == want

    dump = tmp_path / "score.txt"
    out = run("--bundle", folder, "--ids", str(ids_path), "--ctx", "8", "--n-eval", "5", "--dtype", "float32", "--dump", str(dump))
    want = [pm.greedy_pick(pm.logits_all_positions(config, weights, ids[i - 8:i])[-1]) for i in range(8, 13)]
    assert [int(t) for t in dump.read_text().split()] == want and "top-1" in out

    dump = tmp_path / "logits.f32"
    out = run("--model", folder, "--ids", str(ids_path), "--ctx", "9", "--dtype", "float32", "--logits-dump", str(dump))
    got = np.fromfile(dump, dtype="<f4").reshape(9, -1)
    want = pm.logits_all_positions(config, weights, ids[:9])
    assert "9 positions" in out and got.shape == want.shape and np.abs(got - want).max() < 2e-5 * np.abs(want).max()

    prompts_path = tmp_path / "prompts.json"
    prompts_path.write_text(json.dumps([ids[:5], ids[5:16], ids[16:17]]))
    first = run("--model", folder, "--prompts", str(prompts_path), "--generate", "5", "--temperature", "0.9", "--seed", "4",
                "--eos", "none")
    again = run("--model", folder, "--prompts", str(prompts_path), "--generate", "5", "--temperature", "0.9", "--seed", "4",
                "--eos", "none")
    tokens = lambda text: [line for line in text.splitlines() if line and line[0].isdigit()]
    assert tokens(first) == tokens(again) and len(tokens(first)) == 3

    proc = subprocess.run([sys.executable, "-m", "fieldrun_b200", "--model", folder, "--ids", str(ids_path), "--ctx", "12",
                           "--generate", "4", "--eos", "none", "--profile"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    kernels = [json.loads(line) for line in proc.stderr.splitlines() if line.startswith("{")]
    assert any(k["kernel"] == "rmsnorm" and k["launches"] > 0 for k in kernels) and abs(sum(k["share"] for k in kernels) - 1) < 0.01


def test_errors_are_one_line_messages(tmp_path):
    proc = subprocess.run([sys.executable, "-m", "fieldrun_b200", "--model", str(tmp_path / "nothing"), "--ids", "x.json"],
                          cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 1 and proc.stderr.startswith("[fieldrun_b200] error:") and "Traceback" not in proc.stderr
    for flag, word in ((["--device", "cpu"], "no CPU path"), (["--kv-int8"], "quantized caches")):
        proc = subprocess.run([sys.executable, "-m", "fieldrun_b200", "--model", str(tmp_path / "nothing"), "--ids", "x.json", *flag],
                              cwd=ROOT, capture_output=True, text=True, timeout=600)
        assert proc.returncode == 1 and word in proc.stderr and "Traceback" not in proc.stderr
