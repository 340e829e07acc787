"""Configuration, registry, weight loading and its errors (no GPU)."""
import json
import os

import pytest
import torch

from helpers import tiny_config, make_model_dir
from tffinfer_b200 import get_architecture, registered_architectures, RegistryError, ConfigError, WeightError
from tffinfer_b200.config import Qwen3Config, read_config_json, EngineConfig
from tffinfer_b200.parts import Model, MATRIX
from tffinfer_b200.weights import (load_model_weights, write_safetensors, SafetensorsFile,
                                   random_state_dict, held_dtype)


def _cfg_dict(name="B"):
    return tiny_config(name).to_json_dict()


def test_config_round_trip_and_every_field():
    for name in ("A", "B", "C"):
        cfg = tiny_config(name)
        again = Qwen3Config.from_json_dict(json.loads(json.dumps(cfg.to_json_dict())))
        assert again == cfg


def test_configs_differ_in_every_size_and_option():
    a, b = tiny_config("A"), tiny_config("B")
    for f in ("hidden_size", "num_layers", "num_heads", "head_dim", "intermediate_size", "vocab_size",
              "rms_norm_eps", "rope_theta", "max_position", "tie_word_embeddings"):
        assert getattr(a, f) != getattr(b, f), f
    assert a.num_heads // a.num_kv_heads != b.num_heads // b.num_kv_heads
    assert b.num_heads * b.head_dim != b.hidden_size            # q width differs from the model width


def test_head_dim_defaults_to_quotient_only_when_absent():
    d = _cfg_dict("A")
    del d["head_dim"]
    assert Qwen3Config.from_json_dict(d).head_dim == 64 // 4
    d = _cfg_dict("B")
    assert Qwen3Config.from_json_dict(d).head_dim == 32        # 96 / 8 would be 12


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                                 "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta",
                                 "max_position_embeddings"])
def test_missing_required_key_is_named(key):
    d = _cfg_dict()
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_json_dict(d)


def test_unsupported_options_are_refused():
    d = _cfg_dict(); d["attention_bias"] = True
    with pytest.raises(ConfigError, match="attention_bias"):
        Qwen3Config.from_json_dict(d)
    d = _cfg_dict(); d["rope_scaling"] = {"type": "yarn"}
    with pytest.raises(ConfigError, match="rope_scaling"):
        Qwen3Config.from_json_dict(d)
    d = _cfg_dict(); d["num_key_value_heads"] = 3
    with pytest.raises(ConfigError, match="multiple"):
        Qwen3Config.from_json_dict(d)
    d = _cfg_dict(); d["hidden_act"] = "gelu"
    with pytest.raises(ConfigError, match="hidden_act"):
        Qwen3Config.from_json_dict(d)
    d = _cfg_dict(); d["hidden_size"] = "96"
    with pytest.raises(ConfigError, match="hidden_size"):
        Qwen3Config.from_json_dict(d)


def test_window_rules():
    d = _cfg_dict("B")
    d.pop("layer_types"); d["use_sliding_window"] = True; d["sliding_window"] = 8; d["max_window_layers"] = 1
    c = Qwen3Config.from_json_dict(d)
    assert [c.window_of_layer(i) for i in range(3)] == [0, 8, 8]
    c = tiny_config("C")
    assert [c.window_of_layer(i) for i in range(4)] == [0, 24, 0, 24]
    d = _cfg_dict("C"); d["sliding_window"] = None
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen3Config.from_json_dict(d)


def test_registry_names_the_model_and_lists_on_miss():
    assert "Qwen3ForCausalLM" in registered_architectures()
    arch = get_architecture("Qwen3ForCausalLM")
    desc = arch.describe(tiny_config("B"))
    assert len(desc.layers) == 3 and desc.lm_head_name == "lm_head.weight"
    assert arch.describe(tiny_config("A")).lm_head_name is None
    with pytest.raises(RegistryError, match="Qwen3ForCausalLM"):
        get_architecture("NoSuchModel")


def test_engine_config_checks():
    assert EngineConfig(dtype="bf16").normalized().dtype == "bfloat16"
    with pytest.raises(ValueError):
        EngineConfig(dtype="fp8").normalized()
    with pytest.raises(ValueError):
        EngineConfig(page_size=0).normalized()


def test_random_model_folder_and_dtype_policy(tmp_path):
    d = make_model_dir(tmp_path, "B")
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    cfg = Qwen3Config.from_json_dict(read_config_json(d))
    model = Model(get_architecture(cfg.architecture).describe(cfg))
    exp = model.expected_tensors()
    bf = load_model_weights(d, exp, torch.bfloat16, "cpu")
    f32 = load_model_weights(d, exp, torch.float32, "cpu")
    for n, spec in exp.items():
        assert tuple(bf[n].shape) == tuple(spec.shape)
        if spec.role == MATRIX:
            assert bf[n].dtype == torch.bfloat16 and f32[n].dtype == torch.float32
            assert torch.equal(bf[n].float(), f32[n])          # widening changes no value
        else:
            assert bf[n].dtype == torch.float32 and f32[n].dtype == torch.float32
    # the library's own reader sees the same file
    from safetensors.torch import load_file
    lib = load_file(os.path.join(d, "model.safetensors"))
    assert set(lib) == set(exp)
    assert torch.equal(lib["model.norm.weight"].float(), f32["model.norm.weight"])
    # a tensor stored in 32 bits stays in 32 bits, also when serving in bfloat16
    d32 = make_model_dir(tmp_path, "B", store_dtype="float32")
    held = load_model_weights(d32, exp, torch.bfloat16, "cpu")
    assert all(t.dtype == torch.float32 for t in held.values())
    assert held_dtype(torch.float16, MATRIX, torch.bfloat16) == torch.bfloat16


def test_random_weights_depend_on_seed_and_name_only():
    cfg = tiny_config("A")
    a, b, c = random_state_dict(cfg, 1), random_state_dict(cfg, 1), random_state_dict(cfg, 2)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    n = a["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.1 and float(n.std()) > 0.01
    w = a["model.layers.1.mlp.down_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.004


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = tiny_config("B")
    sd = random_state_dict(cfg, 3)
    del sd["model.layers.1.self_attn.k_norm.weight"]
    del sd["lm_head.weight"]
    sd["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(256, dtype=torch.bfloat16)
    sd["model.layers.2.mlp.up_proj.weight"] = torch.zeros(161, 96, dtype=torch.bfloat16)
    d = str(tmp_path / "broken")
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_json_dict(), f)
    write_safetensors(os.path.join(d, "model.safetensors"), sd)
    model = Model(get_architecture(cfg.architecture).describe(cfg))
    with pytest.raises(WeightError) as ei:
        load_model_weights(d, model.expected_tensors(), torch.float32, "cpu")
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.k_norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [(n, tuple(x), tuple(y)) for n, x, y in e.wrong_shape] == \
        [("model.layers.2.mlp.up_proj.weight", (160, 96), (161, 96))]
    msg = str(e)
    for piece in ("missing", "unexpected", "wrong shapes", "k_norm", "q_proj.bias", "[161, 96]"):
        assert piece in msg


def test_tied_model_refuses_a_stray_lm_head(tmp_path):
    cfg = tiny_config("A")
    sd = random_state_dict(cfg, 3)
    sd["lm_head.weight"] = sd["model.embed_tokens.weight"].clone()
    model = Model(get_architecture(cfg.architecture).describe(cfg))
    from tffinfer_b200.weights.loader import check_tensors
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_tensors(sd, model.expected_tensors(), torch.float32, "cpu")


def test_safetensors_reader_rejects_broken_files(tmp_path):
    from tffinfer_b200.weights import SafetensorsError
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"\x05\x00")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    write_safetensors(str(p), {"a": torch.arange(6, dtype=torch.int32).view(2, 3)})
    f = SafetensorsFile(str(p))
    assert f.tensor("a").tolist() == [[0, 1, 2], [3, 4, 5]]


def _write_sharded(tmp_path, cfg, sd, stored_twice=()):
    """A model folder whose tensors are spread over three shard files named by model.safetensors.index.json
    (the layout of checkpoints too large for one file)."""
    d = str(tmp_path / ("sharded_twice" if stored_twice else "sharded"))
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_json_dict(), f)
    names = sorted(sd)
    files = [f"model-0000{i + 1}-of-00003.safetensors" for i in range(3)]
    parts = [dict(), dict(), dict()]
    weight_map = {}
    for i, n in enumerate(names):
        parts[i % 3][n] = sd[n]
        weight_map[n] = files[i % 3]
    for n in stored_twice:
        other = (files.index(weight_map[n]) + 1) % 3
        parts[other][n] = sd[n]
    for fn, part in zip(files, parts):
        write_safetensors(os.path.join(d, fn), part)
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    return d


def test_a_sharded_folder_loads_like_a_single_file_and_a_tensor_stored_twice_is_an_error(tmp_path):
    cfg = tiny_config("B")
    sd = random_state_dict(cfg, 3)
    model = Model(get_architecture(cfg.architecture).describe(cfg))
    expected = model.expected_tensors()
    d = _write_sharded(tmp_path, cfg, sd)
    held = load_model_weights(d, expected, torch.bfloat16, "cpu")
    assert sorted(held) == sorted(sd)
    for n, t in sd.items():
        assert torch.equal(held[n].float(), t.float()), n
    # the whole engine from the sharded folder gives the single-file folder's logits
    from cpu_ops import CpuOps
    from tffinfer_b200.engine import ModelRunner, StepEntry
    single = make_model_dir(tmp_path, "B", seed=3)
    logits = []
    for folder in (d, single):
        r = ModelRunner(folder, EngineConfig(dtype="float32", page_size=8, max_cache_tokens=64, device="cpu"), ops=CpuOps())
        r.add_request("x")
        logits.append(r.step([StepEntry("x", [5, 17, 3, 200, 41], [4])]))
    assert torch.equal(logits[0], logits[1])
    # the same tensor in two shards: one error that names it, beside whatever else is wrong
    twice = ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    sd2 = dict(sd)
    del sd2["model.layers.0.input_layernorm.weight"]
    d2 = _write_sharded(tmp_path, cfg, sd2, stored_twice=twice)
    with pytest.raises(WeightError) as ei:
        load_model_weights(d2, expected, torch.bfloat16, "cpu")
    assert ei.value.duplicates == sorted(twice)
    assert ei.value.missing == ["model.layers.0.input_layernorm.weight"]
    assert "more than one file" in str(ei.value)
    # an index that names no file is refused
    from tffinfer_b200.weights import SafetensorsError
    empty = tmp_path / "empty_index"
    empty.mkdir()
    (empty / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {}}))
    with pytest.raises(SafetensorsError):
        load_model_weights(str(empty), expected, torch.bfloat16, "cpu")
