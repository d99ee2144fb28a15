import json
import os

import numpy as np
import pytest
import torch

import fieldrun_b200 as fr
from fieldrun_b200.api import build_model
from fieldrun_b200.config import load_config
from fieldrun_b200.weights import (FolderSource, ModelFolder, TensorNeed, WeightError, WeightFileError, check_needs,
                                   held_dtype, read_header, write_safetensors)
from fieldrun_b200.weights.loader import MATRIX, TABLE, VECTOR
from plain_model import read_safetensors
from tiny_configs import ALL, CONFIG_A, INIT_A


def _folder(tmp_path, name="a"):
    config, init = ALL[name]
    folder = str(tmp_path / f"model_{name}")
    fr.write_random_model(folder, config, init)
    return folder


def _needs(folder):
    arch, cfg = load_config(folder)
    return build_model(arch, cfg, "float32").tensor_needs()


def test_round_trip_and_own_reader_agree(tmp_path):
    tensors = {"x": torch.randn(3, 5), "y": torch.randn(7).to(torch.bfloat16), "z": torch.arange(6, dtype=torch.int32)}
    path = str(tmp_path / "t.safetensors")
    write_safetensors(path, tensors.items())
    plain = read_safetensors(path)
    for entry in read_header(path):
        assert entry.shape == tuple(tensors[entry.name].shape)
    np.testing.assert_array_equal(plain["x"], tensors["x"].numpy())
    np.testing.assert_array_equal(plain["y"], tensors["y"].float().numpy())
    np.testing.assert_array_equal(plain["z"], tensors["z"].numpy())


def test_random_folder_has_exactly_the_needed_tensors(tmp_path):
    for name in ALL:
        folder = _folder(tmp_path, name)
        needs = _needs(folder)
        index = ModelFolder(folder)
        assert set(index.names()) == {n.name for n in needs}
        FolderSource(folder, needs, torch.float32, "cpu").close()


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    a, b, c = str(tmp_path / "a"), str(tmp_path / "b"), str(tmp_path / "c")
    fr.write_random_model(a, CONFIG_A, INIT_A)
    fr.write_random_model(b, CONFIG_A, INIT_A)
    fr.write_random_model(c, CONFIG_A, fr.RandomInit(seed=5))
    wa, wb, wc = (read_safetensors(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert all(np.array_equal(wa[k], wb[k]) for k in wa)
    assert not np.array_equal(wa["lm_head.weight"], wc["lm_head.weight"])
    norm = wa["model.layers.0.input_layernorm.weight"]
    assert abs(norm.mean() - 1.0) < 0.1 and norm.std() > 0.02
    assert np.all(wa["model.layers.0.block_sparse_moe.e_score_correction_bias"] == 0)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = _folder(tmp_path)
    tensors = {k: torch.from_numpy(v) for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    del tensors["model.layers.1.self_attn.k_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.extra"] = torch.zeros(3)
    tensors["lm_head.weight"] = torch.zeros(10, 64)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
    with pytest.raises(WeightError) as err:
        FolderSource(folder, _needs(folder), torch.float32, "cpu")
    e = err.value
    assert sorted(e.missing) == ["model.layers.1.self_attn.k_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.mlp.extra"]
    assert e.wrong_shape == [("lm_head.weight", (256, 64), (10, 64))]
    text = str(e)
    for word in ("missing (2)", "unexpected (1)", "expected [256, 64], found [10, 64]", "model.norm.weight"):
        assert word in text


def test_tensors_the_model_has_no_use_for_are_a_warning_unless_strict(tmp_path, capsys):
    """The reference fetches by name and ignores the rest (src/convert.rs:1231-1257)."""
    folder = _folder(tmp_path)
    tensors = {k: torch.from_numpy(v) for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(4)
    tensors["model.mtp.0.weight"] = torch.zeros(2, 2)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
    source = FolderSource(folder, _needs(folder), torch.float32, "cpu")
    assert sorted(source.unused) == ["model.layers.0.self_attn.rotary_emb.inv_freq", "model.mtp.0.weight"]
    source.close()
    err = capsys.readouterr().err
    assert "warning" in err and "inv_freq" in err and "model.mtp.0.weight" in err
    with pytest.raises(WeightError, match="unexpected \\(2\\)"):
        FolderSource(folder, _needs(folder), torch.float32, "cpu", strict=True)


def test_random_elements_are_a_function_of_seed_name_and_index():
    """Each element restated with Python integers: two rounds of the hash, eight 16-bit fields, one scale."""
    from fieldrun_b200.weights.random_init import _GOLDEN, _MASK, _UNIT, _mix_int, tensor_key, unit_normal
    key = tensor_key(7, "model.layers.3.block_sparse_moe.experts.11.w2.weight")
    assert key != tensor_key(8, "model.layers.3.block_sparse_moe.experts.11.w2.weight")
    assert key != tensor_key(7, "model.layers.3.block_sparse_moe.experts.12.w2.weight")
    drawn = unit_normal(key, (37, 5), "cpu", scale=0.02)

    def element(i):
        a = _mix_int((i * _GOLDEN + key) & _MASK)
        b = _mix_int(a)
        total = sum((word >> shift) & 0xFFFF for word in (a, b) for shift in (0, 16, 32, 48))
        return np.float32(2 * total - 8 * 65535) * np.float32(_UNIT * 0.02)

    for i in (0, 1, 36, 100, 184):
        assert drawn.flatten()[i].item() == float(element(i))
    # a slice is re-made without the rest; chunks do not show
    assert torch.equal(unit_normal(key, (20,), "cpu", scale=0.02, first=100), drawn.flatten()[100:120])
    big = unit_normal(key, (1 << 18,), "cpu")
    assert abs(big.mean().item()) < 0.01 and abs(big.std().item() - 1.0) < 0.01 and big.abs().max().item() < 4.9


def test_integer_tensor_where_a_real_one_is_needed():
    with pytest.raises(WeightError, match="unsupported dtype: w is stored as I32"):
        check_needs("here", [TensorNeed("w", (2,), VECTOR)], {"w": ("I32", (2,))})


def test_held_dtypes():
    assert held_dtype(MATRIX, torch.float32, torch.bfloat16) == torch.bfloat16
    assert held_dtype(MATRIX, torch.bfloat16, torch.float32) == torch.float32
    assert held_dtype(VECTOR, torch.float32, torch.bfloat16) == torch.float32
    assert held_dtype(VECTOR, torch.bfloat16, torch.bfloat16) == torch.float32
    assert held_dtype(TABLE, torch.int64, torch.bfloat16) == torch.int32


def test_fetch_converts_as_documented(tmp_path):
    folder = _folder(tmp_path)
    needs = _needs(folder)
    source = FolderSource(folder, needs, torch.bfloat16, "cpu")
    by_name = {n.name: n for n in needs}
    assert source.fetch(by_name["lm_head.weight"]).dtype == torch.bfloat16
    assert source.fetch(by_name["model.norm.weight"]).dtype == torch.float32
    assert source.fetch(by_name["model.layers.0.block_sparse_moe.gate.weight"]).dtype == torch.float32
    source.close()


def test_broken_files(tmp_path):
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(WeightFileError, match="neither model.safetensors"):
        ModelFolder(str(empty))
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "model.safetensors").write_bytes(b"\xff" * 32)
    with pytest.raises(WeightFileError):
        ModelFolder(str(bad))
    sharded = tmp_path / "sharded"
    sharded.mkdir()
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"w": "part-1.safetensors"}}))
    with pytest.raises(WeightFileError, match="part-1.safetensors"):
        ModelFolder(str(sharded))


def test_sharded_folder(tmp_path):
    folder = tmp_path / "s"
    folder.mkdir()
    write_safetensors(str(folder / "p1.safetensors"), [("a", torch.ones(2))])
    write_safetensors(str(folder / "p2.safetensors"), [("b", torch.zeros(3))])
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "p1.safetensors", "b": "p2.safetensors"}}))
    index = ModelFolder(str(folder))
    assert sorted(index.names()) == ["a", "b"] and index.tensor("b").shape == (3,)
