"""Configuration, registry, safetensors reading and the weight checks (no device needed)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from ithaca_b200.config import (ConfigError, LlamaConfig, PartSpec, ScheduleEntry, config_from_dict,
                                config_from_model_dir, register_architecture, registered_architectures,
                                unregister_architecture, validate_schedule)
from ithaca_b200.engine.model import weight_manifest
from ithaca_b200.weights import (SafetensorsError, TensorReq, WeightError, check_tensors, load_checkpoint,
                                 read_file, read_model_tensors, write_file, write_random_model)
from tiny import TINY_A, TINY_B, TINY_C


def test_llama_config_reads_its_keys():
    _, c = config_from_dict(TINY_B)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (192, 3, 6, 2, 32)
    assert c.rope_scaling.rope_type == "llama3" and c.rope_scaling.original_max_position_embeddings == 64
    assert c.eos_token_ids == (3, 5) and c.tie_word_embeddings and c.rms_norm_eps == 1e-6
    _, a = config_from_dict(TINY_A)
    assert a.rope_scaling is None and a.eos_token_ids == (7,) and a.torch_dtype == "float32"


def test_defaults_follow_the_reference():
    d = {"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 1, "num_attention_heads": 4,
         "intermediate_size": 128, "vocab_size": 100}
    _, c = config_from_dict(d)
    assert c.num_key_value_heads == 4 and c.head_dim == 16 and c.rms_norm_eps == 1e-5
    assert c.rope_theta == 10000.0 and c.max_position_embeddings == 4096 and not c.tie_word_embeddings


def test_rotary_numbers_in_one_object_are_read_like_the_separate_keys():
    d = dict(TINY_B)
    separate = config_from_dict(d)[1]
    scaling, theta = d.pop("rope_scaling"), d.pop("rope_theta")
    d["rope_parameters"] = dict(scaling, rope_theta=theta)
    together = config_from_dict(d)[1]
    assert together.rope_theta == separate.rope_theta and together.rope_scaling == separate.rope_scaling
    d["rope_parameters"] = {"rope_type": "default", "rope_theta": 1234.5}
    plain = config_from_dict(d)[1]
    assert plain.rope_theta == 1234.5 and plain.rope_scaling is None
    with pytest.raises(ConfigError):
        config_from_dict(dict(d, rope_parameters=[1, 2]))


@pytest.mark.parametrize("patch,word", [
    ({"hidden_size": None}, "hidden_size"), ({"num_attention_heads": 5, "head_dim": None}, "multiple"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"), ({"rope_scaling": {"rope_type": "yarn", "factor": 2}}, "yarn"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"), ({"vocab_size": 0}, "vocab_size"), ({"head_dim": 15}, "even"),
    ({"eos_token_id": "x"}, "eos_token_id"), ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8}}, "low_freq_factor"),
])
def test_bad_configurations_are_refused(patch, word):
    d = dict(TINY_A)
    for k, v in patch.items():
        if v is None:
            d.pop(k, None)
        else:
            d[k] = v
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_registry_names_what_it_knows():
    with pytest.raises(ConfigError) as e:
        config_from_dict({**TINY_A, "architectures": ["MambaForCausalLM"]})
    assert "MambaForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    register_architecture("ToyLM", LlamaConfig)
    try:
        assert "ToyLM" in registered_architectures()
        arch, c = config_from_dict({**TINY_A, "architectures": ["ToyLM"]})
        assert arch.name == "ToyLM" and c.hidden_size == 64
        with pytest.raises(ValueError):
            register_architecture("ToyLM", LlamaConfig)
    finally:
        unregister_architecture("ToyLM")


def test_model_spec_is_layer_by_layer_data():
    _, c = config_from_dict(TINY_C)
    spec = c.model_spec()
    assert len(spec.layers) == 2 and [e.layer for e in spec.schedule] == [0, 1]
    assert spec.layers[0].mixer.kind == "attention" and spec.layers[0].mixer["window"] == 40
    assert spec.layers[1].feed_forward.weights["down"] == "model.layers.1.mlp.down_proj.weight"
    assert spec.layers[0].position["scaling"]["rope_type"] == "linear"
    m = weight_manifest(spec)
    assert m["model.layers.0.self_attn.q_proj.weight"].shape == (5 * 48, 200)
    assert m["model.layers.0.self_attn.k_proj.weight"].shape == (48, 200)
    assert m["lm_head.weight"].shape == (301, 200)
    _, b = config_from_dict(TINY_B)
    assert "lm_head.weight" not in weight_manifest(b.model_spec())


def test_schedule_validation():
    _, c = config_from_dict(TINY_A)
    spec = c.model_spec()
    import dataclasses
    ok = dataclasses.replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
                                             ScheduleEntry(1, 0, writes_cache=False)))
    validate_schedule(ok)
    for bad in [(ScheduleEntry(2, 0),), (ScheduleEntry(0, 0), ScheduleEntry(1, 0)),
                (ScheduleEntry(0, 1, writes_cache=False), ScheduleEntry(1, 1)), (ScheduleEntry(0, 1),)]:
        with pytest.raises(ValueError):
            validate_schedule(dataclasses.replace(spec, schedule=bad))


def test_safetensors_round_trip_and_other_writer(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "e": torch.empty(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_file(p, t, {"k": "v"})
    back = read_file(p)
    assert set(back) == set(t) and all(torch.equal(back[k], t[k]) and back[k].dtype == t[k].dtype for k in t)
    from safetensors.torch import load_file, save_file
    theirs = load_file(p)                          # the common library reads what this writer wrote
    assert all(torch.equal(theirs[k], t[k]) for k in t)
    p2 = str(tmp_path / "y.safetensors")
    save_file({k: v.contiguous() for k, v in t.items()}, p2)
    back2 = read_file(p2)                          # and this reader reads what the common library wrote
    assert all(torch.equal(back2[k], t[k]) for k in t)


def test_broken_files_are_refused(tmp_path):
    p = str(tmp_path / "m.safetensors")
    write_file(p, {"w": torch.randn(4, 4)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-8])                  # truncated
    with pytest.raises(SafetensorsError, match="outside the file"):
        read_file(p)
    open(p, "wb").write(raw[:4])
    with pytest.raises(SafetensorsError, match="not a safetensors"):
        read_file(p)
    open(p, "wb").write(struct.pack("<Q", 10**12) + raw[8:])
    with pytest.raises(SafetensorsError, match="header length"):
        read_file(p)
    (hl,) = struct.unpack("<Q", raw[:8])
    hdr = json.loads(raw[8:8 + hl])
    hdr["w"]["shape"] = [4, 5]
    h2 = json.dumps(hdr).encode()
    open(p, "wb").write(struct.pack("<Q", len(h2)) + h2 + raw[8 + hl:])
    with pytest.raises(SafetensorsError, match="needs"):
        read_file(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=1)
    _, c = config_from_model_dir(d)
    manifest = weight_manifest(c.model_spec())
    tensors = dict(read_model_tensors(d))
    load_checkpoint(d, manifest)                   # the folder as written is fine
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    with pytest.raises(WeightError) as e:
        check_tensors(tensors, manifest)
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg and "missing tensors (2)" in msg
    assert "rotary_emb.inv_freq" in msg and "unexpected tensors (1)" in msg
    assert "q_proj.weight: expected [64, 64], found [64, 32]" in msg and "lm_head.weight: expected a floating-point" in msg


def test_storage_types_are_kept(tmp_path):
    d = str(tmp_path / "m")
    os.makedirs(d)
    manifest = {"bf": TensorReq((2, 2)), "f32": TensorReq((3,)), "f16": TensorReq((3,)), "table": TensorReq((4,), integer=True)}
    write_file(os.path.join(d, "model.safetensors"), {
        "bf": torch.ones(2, 2, dtype=torch.bfloat16), "f32": torch.ones(3), "f16": torch.ones(3, dtype=torch.float16),
        "table": torch.arange(4, dtype=torch.int64)})
    t = load_checkpoint(d, manifest)
    assert t["bf"].dtype == torch.bfloat16 and t["f32"].dtype == torch.float32
    assert t["f16"].dtype == torch.float32 and t["table"].dtype == torch.int32


def test_random_model_folder(tmp_path):
    d1 = write_random_model(str(tmp_path / "a"), TINY_B, seed=5)
    d2 = write_random_model(str(tmp_path / "b"), TINY_B, seed=5)
    d3 = write_random_model(str(tmp_path / "c"), TINY_B, seed=6)
    t1, t2, t3 = read_model_tensors(d1), read_model_tensors(d2), read_model_tensors(d3)
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    assert all(torch.equal(t1[k], t2[k]) for k in t1) and not torch.equal(t1["model.norm.weight"], t3["model.norm.weight"])
    assert t1["model.embed_tokens.weight"].dtype == torch.bfloat16 and "lm_head.weight" not in t1
    w = t1["model.layers.0.mlp.gate_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(t1["model.norm.weight"].float().mean().item() - 1) < 0.01
    cfg = json.load(open(os.path.join(d1, "config.json")))
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["num_key_value_heads"] == 2
    _, c = config_from_model_dir(d1)
    assert c == config_from_dict(TINY_B)[1]


def test_tensor_in_two_files_and_missing_folder(tmp_path):
    d = str(tmp_path / "m")
    os.makedirs(d)
    with pytest.raises(WeightError, match="no .safetensors"):
        read_model_tensors(d)
    write_file(os.path.join(d, "a.safetensors"), {"w": torch.zeros(2)})
    write_file(os.path.join(d, "b.safetensors"), {"w": torch.zeros(2)})
    with pytest.raises(WeightError, match="appears in both"):
        read_model_tensors(d)
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_model_dir(d)


def test_random_weights_are_a_function_of_seed_name_and_index():
    """Element i of a tensor depends on (seed, name, i) only: a slice made alone equals the slice of the whole,
    another name or seed gives other values, and the law is close to the normal one asked for."""
    from ithaca_b200.weights.random_init import hashed_normal, random_tensor, tensor_key
    k = tensor_key(7, "model.layers.3.mlp.up_proj.weight")
    whole = hashed_normal(k, 300000, 0.02)
    assert np.array_equal(whole[1234:5000], hashed_normal(k, 5000 - 1234, 0.02, first=1234))
    assert not np.array_equal(whole[:100], hashed_normal(tensor_key(8, "model.layers.3.mlp.up_proj.weight"), 100, 0.02))
    assert not np.array_equal(whole[:100], hashed_normal(tensor_key(7, "model.layers.3.mlp.gate_proj.weight"), 100, 0.02))
    assert abs(whole.mean()) < 2e-4 and abs(whole.std() - 0.02) < 2e-4 and np.abs(whole).max() < 0.1
    z = whole / 0.02
    assert abs((z ** 3).mean()) < 0.03 and abs((z ** 4).mean() - 3.0) < 0.2       # skewness 0, fourth moment near 3
    # one value by hand: the two hash words' eight 16-bit fields, centred and scaled in float32
    def mix(v):
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & (2 ** 64 - 1)
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & (2 ** 64 - 1)
        return v ^ (v >> 31)
    i, s = 4321, 0
    for j in (1, 2):
        h = mix((k + (2 * i + j) * 0x9E3779B97F4A7C15) & (2 ** 64 - 1))
        s += sum((h >> sh) & 0xFFFF for sh in (0, 16, 32, 48))
    scale = np.float32(0.02 / np.sqrt(8 * (65536.0 ** 2 - 1) / 12))
    assert whole[i] == np.float32(scale * np.float32(s - 262140))
    ones = random_tensor("n", TensorReq((64,), init="ones"), 1, "float32")
    assert abs(ones.mean().item() - 1.0) < 0.01 and 0.002 < ones.std().item() < 0.02


def test_generation_config_adds_stop_ids(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=1)
    assert config_from_model_dir(d)[1].eos_token_ids == (7,)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [9, 7, 11], "temperature": 0.6}, f)
    cfg = config_from_model_dir(d)[1]
    assert cfg.eos_token_ids == (7, 9, 11) and cfg.model_spec().stop_token_ids == (7, 9, 11)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": "</s>"}, f)
    with pytest.raises(ConfigError, match="generation_config.json"):
        config_from_model_dir(d)


def test_a_window_needs_to_be_switched_on():
    """The reference runs this architecture without a window; a folder that merely carries the number keeps every key."""
    base = dict(TINY_A, sliding_window=40)
    assert config_from_dict(base)[1].sliding_window is None
    on = config_from_dict(dict(base, use_sliding_window=True))[1]
    assert on.sliding_window == 40 and on.model_spec().layers[0].mixer["window"] == 40
    assert on.to_dict()["use_sliding_window"] is True and config_from_dict(on.to_dict())[1] == on
    with pytest.raises(ConfigError, match="use_sliding_window"):
        config_from_dict(dict(base, use_sliding_window="yes"))
