"""The weight loader (names, shapes, dtypes, one error for everything wrong) and the
random-weights mode."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from inference_engine_b200.config import build_model_spec, config_from_dict
from inference_engine_b200.engine.model import declared_weights
from inference_engine_b200.weights import WeightError, load_weights, write_random_model
from tests import helpers
from tests.tiny_configs import TINY_A, TINY_B


def _expected(cfg):
    return declared_weights(build_model_spec(config_from_dict(cfg)))


def test_declared_names_are_the_checkpoint_names():
    for cfg in (TINY_A, TINY_B):
        want = helpers.llama_tensor_shapes(cfg)
        got = {n: d.shape for n, d in _expected(cfg).items()}
        assert got == want
    assert "lm_head.weight" not in _expected(TINY_A)  # tied: absent from checkpoints


def test_random_model_folder_round_trip(tmp_path):
    folder = write_random_model(TINY_B, tmp_path / "m", seed=3)
    assert json.loads((folder / "config.json").read_text())["num_hidden_layers"] == 3
    tensors = load_weights(folder, _expected(TINY_B), "cpu")
    assert set(tensors) == set(_expected(TINY_B))
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    norm = tensors["model.layers.0.input_layernorm.weight"].float()
    proj = tensors["model.layers.2.mlp.up_proj.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.02 and 0.005 < float(norm.std()) < 0.04
    assert abs(float(proj.mean())) < 0.005 and abs(float(proj.std()) - 0.02) < 0.003
    # the same seed gives the same values; another seed does not; a tensor's values do not
    # depend on which other tensors exist (here: on the number of layers)
    again = load_file(str(write_random_model(TINY_B, tmp_path / "m2", seed=3) / "model.safetensors"))
    other = load_file(str(write_random_model(TINY_B, tmp_path / "m3", seed=4) / "model.safetensors"))
    fewer = load_file(str(write_random_model({**TINY_B, "num_hidden_layers": 1}, tmp_path / "m4", seed=3) / "model.safetensors"))
    name = "model.layers.0.self_attn.q_proj.weight"
    assert torch.equal(again[name], tensors[name]) and not torch.equal(other[name], tensors[name])
    assert torch.equal(fewer[name], tensors[name])
    f32 = load_file(str(write_random_model(TINY_B, tmp_path / "m5", seed=3, dtype="float32") / "model.safetensors"))
    assert f32[name].dtype == torch.float32 and torch.equal(f32[name].bfloat16(), tensors[name])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    weights = helpers.make_weights(TINY_A)
    del weights["model.layers.1.mlp.down_proj.weight"]
    del weights["model.norm.weight"]
    weights["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)  # tied model ships a head
    weights["model.layers.0.extra.bias"] = torch.zeros(3)
    weights["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    folder = helpers.write_model_dir(tmp_path / "bad", TINY_A, weights)
    with pytest.raises(WeightError) as info:
        load_weights(folder, _expected(TINY_A), "cpu")
    err = info.value
    assert err.missing == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["lm_head.weight", "model.layers.0.extra.bias"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (1)",
                  "model.norm.weight", "lm_head.weight", "is [16, 64], expected [32, 64]"):
        assert piece in text


def test_stored_precision_is_kept(tmp_path):
    weights = {k: v.float() for k, v in helpers.make_weights(TINY_A).items()}
    weights["model.norm.weight"] = weights["model.norm.weight"] + 1e-4  # not a bfloat16 value
    weights["model.layers.0.mlp.up_proj.weight"] = weights["model.layers.0.mlp.up_proj.weight"].half()
    folder = helpers.write_model_dir(tmp_path / "f32", TINY_A, weights)
    tensors = load_weights(folder, _expected(TINY_A), "cpu")
    assert tensors["model.norm.weight"].dtype == torch.float32  # stored in 32-bit, stays so
    assert torch.equal(tensors["model.norm.weight"], weights["model.norm.weight"])
    assert tensors["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16  # half -> bfloat16


def test_integer_tables_become_int32():
    from inference_engine_b200.weights import stored_dtype

    assert stored_dtype(torch.int64) == torch.int32 and stored_dtype(torch.uint8) == torch.int32
    assert stored_dtype(torch.float64) == torch.float32


def test_sharded_checkpoints_and_missing_files(tmp_path):
    weights = helpers.make_weights(TINY_A)
    names = sorted(weights)
    folder = tmp_path / "sharded"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_A))
    half = len(names) // 2
    save_file({n: weights[n] for n in names[:half]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({n: weights[n] for n in names[half:]}, str(folder / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {n: f"model-0000{1 if i < half else 2}-of-00002.safetensors" for i, n in enumerate(names)}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    tensors = load_weights(folder, _expected(TINY_A), "cpu")
    assert all(torch.equal(tensors[n], weights[n]) for n in names)
    with pytest.raises(FileNotFoundError, match="no safetensors weights"):
        load_weights(tmp_path, _expected(TINY_A), "cpu")


def test_loaded_model_matches_plain_on_reference_ops(tmp_path):
    """Folder -> registry -> parts -> step function, on the plain PyTorch stand-ins of the
    kernels: tied and untied heads, bfloat16 values computed in 32-bit."""
    from inference_engine_b200.engine.batch import StepEntry
    from inference_engine_b200.engine.loading import load_model
    from inference_engine_b200.engine.runner import make_runner
    from tests import plain_llama
    from tests.ref_ops import RefOps

    for cfg in (TINY_A, TINY_B):
        weights = helpers.make_weights(cfg, seed=5)
        folder = helpers.write_model_dir(tmp_path / f"m{cfg['hidden_size']}", cfg, weights)
        model, _ = load_model(folder, "float32", "cpu", max_positions=64)
        if cfg["tie_word_embeddings"]:
            assert model.head.weight is model.embedding.table  # one buffer
        runner = make_runner(model, RefOps(), "cpu", 8, 16, 2, 64)
        ids = helpers.random_tokens(cfg, 30, 1)
        runner.cache.add_request("a")
        runner.cache.grow("a", 0, 30)
        got = runner.step([StepEntry("a", ids, 0, list(range(30)))])
        helpers.assert_close(got, plain_llama.logits_for(cfg, weights, ids), "float32", "loaded model")
