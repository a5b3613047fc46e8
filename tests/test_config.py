"""Configuration, registry and weight errors (no GPU)."""

from __future__ import annotations

import json

import pytest
import torch

import helpers

from distie_b200.config import ConfigError, EngineConfig, Qwen2Config, get_architecture, known_architectures, read_config
from distie_b200.models import model_tensor_specs, slot_needs
from distie_b200.weights import ModelTensors, WeightsError, open_weights, save_file, write_random_model


def test_typed_config_reads_every_size_from_json():
    cfg = Qwen2Config.from_dict(helpers.TINY_B)
    assert (cfg.head_dim, cfg.num_key_value_groups, cfg.rms_norm_eps, cfg.rope_theta) == (32, 3, 1e-5, 1e6)
    assert Qwen2Config.from_dict(helpers.TINY_A).head_dim == 16
    assert Qwen2Config.from_dict({**helpers.TINY_A, "num_key_value_heads": None}).num_key_value_heads == 4
    nested = {k: v for k, v in helpers.TINY_A.items() if k != "rope_theta"}
    assert Qwen2Config.from_dict({**nested, "rope_parameters": {"rope_theta": 5.0}}).rope_theta == 5.0
    round_trip = Qwen2Config.from_dict(cfg.to_dict())
    assert round_trip == cfg


@pytest.mark.parametrize(
    "change,word",
    [
        ({"num_key_value_heads": 3}, "multiple"),
        ({"hidden_size": 65}, "head_dim"),
        ({"head_dim": 15, "hidden_size": 60}, "even"),
        ({"hidden_act": "gelu"}, "silu"),
        ({"layer_types": ["full_attention", "sliding_attention"]}, "sliding"),
        ({"use_sliding_window": True}, "sliding"),
        ({"rope_parameters": {"rope_type": "yarn"}}, "RoPE"),
        ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ],
)
def test_config_rejections(change, word):
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict({**helpers.TINY_A, **change})


def test_missing_keys_are_named():
    raw = {k: v for k, v in helpers.TINY_A.items() if k not in ("rms_norm_eps", "vocab_size")}
    with pytest.raises(ConfigError, match="vocab_size.*rms_norm_eps|rms_norm_eps.*vocab_size"):
        Qwen2Config.from_dict(raw)


def test_registry_chooses_by_architectures_key(tmp_path):
    assert "Qwen2ForCausalLM" in known_architectures()
    with pytest.raises(KeyError, match="registered: .*Qwen2ForCausalLM"):
        get_architecture("NoSuchModel")
    folder = write_random_model(str(tmp_path / "m"), helpers.TINY_A, seed=0)
    arch, cfg = read_config(folder)
    assert arch.name == "Qwen2ForCausalLM" and cfg.hidden_size == 64
    spec = arch.recipe(cfg)
    assert spec.head_name is None and len(spec.order) == 2 and spec.num_cache_slots == 2
    caches, states = slot_needs(spec)
    assert len(set(caches.values())) == 1 and not states
    untied = get_architecture("Qwen2ForCausalLM").recipe(Qwen2Config.from_dict(helpers.TINY_B))
    assert untied.head_name == "lm_head.weight"


def test_engine_config_env_defaults(monkeypatch):
    monkeypatch.setenv("WORKER_NUM_BLOCKS", "77")
    monkeypatch.setenv("WORKER_DECODE_GRAPHS", "0")
    cfg = EngineConfig.from_env(max_seqs=5, dtype="fp32")
    assert (cfg.num_blocks, cfg.max_seqs, cfg.token_budget, cfg.decode_graphs, cfg.dtype) == (77, 5, 2048, False, "float32")
    monkeypatch.setenv("WORKER_MAX_SEQS", "zero")
    with pytest.raises(ValueError, match="WORKER_MAX_SEQS"):
        EngineConfig.from_env()
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(dtype="fp8")


def test_random_weights_folder_round_trip(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), helpers.TINY_B, seed=1, std=0.1, norm_noise=0.02, dtype="bfloat16")
    again = write_random_model(str(tmp_path / "n"), helpers.TINY_B, seed=1, std=0.1, norm_noise=0.02, dtype="bfloat16")
    a, b = ModelTensors(folder), ModelTensors(again)
    assert sorted(a.keys()) == sorted(b.keys())
    assert all(torch.equal(a.tensor(k), b.tensor(k)) for k in a.keys()), "same seed, same tensors"
    assert a.dtype("model.layers.0.self_attn.q_proj.weight") == torch.bfloat16
    assert a.shape("lm_head.weight") == (384, 96) and a.shape("model.layers.2.self_attn.k_proj.bias") == (32,)
    norm = a.tensor("model.layers.1.input_layernorm.weight").float()
    assert 0.9 < float(norm.mean()) < 1.1 and float(norm.std()) > 0
    assert json.load(open(f"{folder}/config.json"))["rms_norm_eps"] == 1e-5


def test_loader_keeps_32_bit_tensors_and_makes_vectors_float32():
    cfg = Qwen2Config.from_dict(helpers.TINY_A)
    spec = get_architecture("Qwen2ForCausalLM").recipe(cfg)
    specs = model_tensor_specs(spec)
    import plain_qwen2 as plain

    tensors = {k: v.to(torch.bfloat16) for k, v in plain.random_weights(helpers.TINY_A, 0).items()}
    tensors["model.layers.0.mlp.down_proj.weight"] = tensors["model.layers.0.mlp.down_proj.weight"].float()
    store = open_weights(tensors, specs, spec.tolerated, torch.bfloat16, None)
    assert store.matrix("model.layers.0.mlp.up_proj.weight").dtype == torch.bfloat16
    assert store.matrix("model.layers.0.mlp.down_proj.weight").dtype == torch.float32, "stored in 32-bit: stays so"
    assert store.vector("model.layers.0.self_attn.q_proj.bias").dtype == torch.float32
    assert store.vector("model.norm.weight").dtype == torch.float32
    every = open_weights(tensors, specs, spec.tolerated, torch.float32, None)
    assert every.matrix("model.layers.0.mlp.up_proj.weight").dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    import plain_qwen2 as plain

    cfg = Qwen2Config.from_dict(helpers.TINY_B)
    spec = get_architecture("Qwen2ForCausalLM").recipe(cfg)
    tensors = plain.random_weights(helpers.TINY_B, 1)
    del tensors["model.layers.1.self_attn.q_proj.bias"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(10, 96)
    tensors["model.layers.9.extra.weight"] = torch.zeros(2)
    tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightsError) as caught:
        open_weights(str(tmp_path), model_tensor_specs(spec), spec.tolerated, torch.bfloat16, None)
    err = caught.value
    assert sorted(err.missing) == ["lm_head.weight", "model.layers.1.self_attn.q_proj.bias"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert [(n, tuple(h), tuple(w)) for n, h, w in err.wrong_shape] == [("model.layers.0.mlp.gate_proj.weight", (10, 96), (224, 96))]
    assert [n for n, _ in err.wrong_kind] == ["model.norm.weight"]
    text = str(err)
    for word in ("missing", "unexpected", "wrong shapes", "lm_head.weight", "model.layers.9.extra.weight", "(224, 96)"):
        assert word in text


def test_tied_checkpoint_may_carry_a_head(tmp_path):
    import plain_qwen2 as plain

    cfg = Qwen2Config.from_dict(helpers.TINY_A)
    spec = get_architecture("Qwen2ForCausalLM").recipe(cfg)
    tensors = plain.random_weights(helpers.TINY_A, 0)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    open_weights(tensors, model_tensor_specs(spec), spec.tolerated, torch.float32, None)


def test_safetensors_reader_rejects_damage(tmp_path):
    from distie_b200.weights import SafetensorsError, SafetensorsFile

    path = tmp_path / "x.safetensors"
    save_file({"a": torch.arange(6, dtype=torch.int32).view(2, 3), "b": torch.ones(3, dtype=torch.bfloat16)}, str(path))
    handle = SafetensorsFile(str(path))
    assert handle.tensor("a").tolist() == [[0, 1, 2], [3, 4, 5]] and handle.tensor("b").dtype == torch.bfloat16
    path.write_bytes(path.read_bytes()[:-4])
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(path))
    with pytest.raises(FileNotFoundError):
        ModelTensors(str(tmp_path / "nothing"))


def test_a_float32_checkpoint_is_cast_by_a_16_bit_engine_unless_told_otherwise():
    """Every matrix stored in 32-bit: the checkpoint simply is a float32 one, and a bfloat16 engine casts
    it as the reference does (worker/src/inference/torch_engine.py:135-141); vectors stay 32-bit."""
    import plain_qwen2 as plain

    cfg = Qwen2Config.from_dict(helpers.TINY_A)
    spec = get_architecture("Qwen2ForCausalLM").recipe(cfg)
    specs = model_tensor_specs(spec)
    tensors = plain.random_weights(helpers.TINY_A, 0)  # all float32
    name = "model.layers.1.self_attn.o_proj.weight"
    auto = open_weights(tensors, specs, spec.tolerated, torch.bfloat16, None)
    assert auto.matrix(name).dtype == torch.bfloat16 and auto.table("model.embed_tokens.weight").dtype == torch.bfloat16
    assert auto.vector("model.norm.weight").dtype == torch.float32
    keep = open_weights(tensors, specs, spec.tolerated, torch.bfloat16, None, float32_weights="keep")
    assert keep.matrix(name).dtype == torch.float32
    mixed = {k: v.to(torch.bfloat16) for k, v in tensors.items()}
    mixed[name] = tensors[name]
    assert open_weights(mixed, specs, spec.tolerated, torch.bfloat16, None).matrix(name).dtype == torch.float32
    cast = open_weights(mixed, specs, spec.tolerated, torch.bfloat16, None, float32_weights="cast")
    assert cast.matrix(name).dtype == torch.bfloat16
    with pytest.raises(ValueError, match="float32_weights"):
        open_weights(tensors, specs, spec.tolerated, torch.bfloat16, None, float32_weights="sometimes")
    with pytest.raises(ValueError, match="float32_weights"):
        EngineConfig(float32_weights="sometimes")


def test_sharded_checkpoint_round_trip(tmp_path):
    """``model.safetensors.index.json`` with two shards reads like one file; a name in the wrong shard is an error."""
    import plain_qwen2 as plain
    from distie_b200.weights import SafetensorsError

    cfg = Qwen2Config.from_dict(helpers.TINY_B)
    spec = get_architecture("Qwen2ForCausalLM").recipe(cfg)
    tensors = {k: v.to(torch.bfloat16) for k, v in plain.random_weights(helpers.TINY_B, 1).items()}
    names = sorted(tensors)
    shards = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    weight_map = {}
    for shard, members in shards.items():
        save_file({n: tensors[n] for n in members}, str(tmp_path / shard))
        weight_map.update({n: shard for n in members})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    stored = ModelTensors(str(tmp_path))
    assert sorted(stored.keys()) == names
    for name in names:
        assert stored.shape(name) == tuple(tensors[name].shape) and torch.equal(stored.tensor(name), tensors[name])
    store = open_weights(str(tmp_path), model_tensor_specs(spec), spec.tolerated, torch.bfloat16, None)
    assert torch.equal(store.matrix("lm_head.weight"), tensors["lm_head.weight"])
    weight_map[names[0]] = "model-00002-of-00002.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(SafetensorsError, match="not in shard"):
        ModelTensors(str(tmp_path))


def test_cache_sizing_from_a_memory_budget(monkeypatch):
    from distie_b200.cache import pages_that_fit
    from distie_b200.parts import CacheNeed

    # 28 slots of 2 kv heads x 128 in bfloat16, pages of 16: 28,672 bytes a token, 458,752 a page.
    needs = {slot: CacheNeed(2, 128, None) for slot in range(28)}
    assert pages_that_fit(needs, 16, 2, 458_752 * 1001) == 1000, "one page of the budget is the spare page"
    assert pages_that_fit(needs, 16, 4, 458_752 * 1001) == 499
    with pytest.raises(ValueError):
        pages_that_fit({}, 16, 2, 1 << 30)
    assert EngineConfig(gpu_mem_fraction=0.5).sized(77).num_blocks == 77
    assert EngineConfig(gpu_mem_fraction=0.5).sized(77).gpu_mem_fraction is None
    with pytest.raises(ValueError, match="gpu_mem_fraction"):
        EngineConfig(gpu_mem_fraction=1.5)
    monkeypatch.setenv("WORKER_GPU_MEM_FRACTION", "0.25")
    assert EngineConfig.from_env().gpu_mem_fraction == 0.25
    assert EngineConfig.from_env(num_blocks=64).gpu_mem_fraction is None, "an explicit page count wins"
    assert EngineConfig.from_env(num_blocks=64, gpu_mem_fraction=0.5).gpu_mem_fraction == 0.5
