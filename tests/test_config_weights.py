"""Configuration, registry and weight errors (no GPU)."""
import json
import os

import pytest
import torch

from mini_inference_b200.config import ConfigError, EngineArgs, Qwen3Config, load_config, resolve, supported_architectures
from mini_inference_b200.parts.model import DecoderModel
from mini_inference_b200.weights import WeightError, load_into, write_random_model, write_safetensors
from mini_inference_b200.weights.safetensors_io import open_model_tensors
from tests.conftest import TINY_A, TINY_B, TINY_W
from tests.plain import qwen3_plain as plain


def test_typed_config_reads_every_key():
    a, b = Qwen3Config.from_dict(TINY_A), Qwen3Config.from_dict(TINY_B)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 2, 4, 2, 16)
    assert (a.rope_theta, a.rms_norm_eps, a.tie_word_embeddings, a.vocab_size) == (10000.0, 1e-6, True, 256)
    assert (b.rope_theta, b.rms_norm_eps, b.tie_word_embeddings, b.head_dim) == (1e6, 1e-5, False, 32)   # nested rope key
    assert b.num_attention_heads * b.head_dim != b.hidden_size
    w = Qwen3Config.from_dict(TINY_W)
    assert w.layer_windows == (11, None, 11)
    assert Qwen3Config.from_dict(w.to_dict()) == w                       # config.json round trip
    assert a.describe() == {"architecture": "Qwen3ForCausalLM", "qk_norm": "per_head", "moe": False,
                            "heads": 4, "kv_heads": 2, "head_dim": 16}


def test_defaults_follow_the_reference():
    raw = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim")}
    c = Qwen3Config.from_dict(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16              # model_runner.py:78-79


@pytest.mark.parametrize("patch,word", [
    ({"architectures": ["LlamaForCausalLM"]}, "not supported"),
    ({"hidden_size": None}, "lacks hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"rope_parameters": {"rope_theta": 1e4, "rope_type": "yarn"}}, "rope_type"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["sliding_attention", "full_attention"]}, "sliding_window"),
])
def test_config_refusals(patch, word):
    raw = dict(TINY_A, **patch)
    with pytest.raises(ConfigError, match=word):
        arch = resolve(raw)
        arch.config_class.from_dict(raw)


def test_registry_lists_architectures():
    assert "Qwen3ForCausalLM" in supported_architectures()
    with pytest.raises(ConfigError, match="Supported: .*Qwen3ForCausalLM"):
        resolve({"architectures": ["Nope"]})


def test_engine_args_env(monkeypatch):
    monkeypatch.setenv("KV_BLOCK_SIZE", "32")
    monkeypatch.setenv("CHUNKED_PREFILL", "1")
    monkeypatch.setenv("MAX_NUM_SEQS", "7")
    a = EngineArgs(dtype="fp32")
    assert (a.kv_block_size, a.chunked_prefill, a.max_num_seqs, a.dtype) == (32, True, 7, "float32")
    with pytest.raises(ValueError):
        EngineArgs(dtype="int8")


def test_random_model_folder_is_deterministic_and_loads(tmp_path):
    d1, d2 = str(tmp_path / "a"), str(tmp_path / "b")
    write_random_model(TINY_B, d1, seed=3, std=0.05)
    write_random_model(TINY_B, d2, seed=3, std=0.05)
    assert open(os.path.join(d1, "model.safetensors"), "rb").read() == open(os.path.join(d2, "model.safetensors"), "rb").read()
    files = open_model_tensors(d1)
    assert len(files) == 2 + 3 * 11 + 1 and "lm_head.weight" in files           # untied: 25-tensor layout + layer
    assert files["model.layers.0.self_attn.q_proj.weight"].info("model.layers.0.self_attn.q_proj.weight") == (torch.bfloat16, (192, 96))
    cfg, spec = load_config(d1)
    model = DecoderModel(spec)
    info = load_into(model, d1, torch.float32, "cpu")
    assert info["tensors"] == 36
    # the package's reader and the plain reader see the same bytes
    w = plain.read_safetensors(os.path.join(d1, "model.safetensors"))
    assert torch.equal(model.embedding, w["model.embed_tokens.weight"].float())
    assert model.blocks[0].mixer.qkv.shape == (192 + 96 + 96, 96) and model.blocks[0].feed_forward.gate_up.shape == (448, 96)
    # tied model: no lm_head in the file, head aliases the embedding
    d3 = str(tmp_path / "c")
    write_random_model(TINY_A, d3, seed=0)
    assert "lm_head.weight" not in open_model_tensors(d3)
    _, spec3 = load_config(d3)
    m3 = DecoderModel(spec3)
    load_into(m3, d3, torch.bfloat16, "cpu")
    assert m3.lm_head is m3.embedding and m3.embedding.dtype == torch.bfloat16


def test_runtime_dtypes(tmp_path):
    """bf16 run: 16-bit stays bf16, a vector stored in 32 bits stays so, matrices become bf16."""
    d = str(tmp_path / "m")
    write_random_model(TINY_A, d, seed=0, store_dtype="float32")
    _, spec = load_config(d)
    m = DecoderModel(spec)
    load_into(m, d, torch.bfloat16, "cpu")
    assert m.blocks[0].mixer.qkv.dtype == torch.bfloat16
    assert m.blocks[0].norm1.weight.dtype == torch.float32 and m.blocks[0].mixer.q_norm.dtype == torch.float32
    m2 = DecoderModel(spec)
    load_into(m2, d, torch.float32, "cpu")
    assert m2.blocks[0].mixer.qkv.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_shapes(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(TINY_A, d, seed=0)
    w = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    del w["model.layers.1.mlp.up_proj.weight"], w["model.norm.weight"]
    w["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    w["model.layers.0.self_attn.k_norm.weight"] = torch.zeros(32, dtype=torch.bfloat16)
    w["model.layers.0.mlp.down_proj.weight"] = torch.zeros(128, 64, dtype=torch.bfloat16)
    write_safetensors(os.path.join(d, "model.safetensors"), w)
    _, spec = load_config(d)
    with pytest.raises(WeightError) as e:
        load_into(DecoderModel(spec), d, torch.float32, "cpu")
    err = e.value
    assert set(err.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert err.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert {n for n, _, _ in err.wrong_shape} == {"model.layers.0.self_attn.k_norm.weight", "model.layers.0.mlp.down_proj.weight"}
    msg = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape", "[128, 64], expected [64, 128]"):
        assert word in msg
    # a tied model may carry a copy of the head; an untied one must have it
    d2 = str(tmp_path / "u")
    write_random_model(TINY_B, d2, seed=1)
    w2 = plain.read_safetensors(os.path.join(d2, "model.safetensors"))
    del w2["lm_head.weight"]
    write_safetensors(os.path.join(d2, "model.safetensors"), w2)
    _, spec2 = load_config(d2)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_into(DecoderModel(spec2), d2, torch.float32, "cpu")


def test_missing_files(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    with open(tmp_path / "config.json", "w") as f:
        json.dump(TINY_A, f)
    _, spec = load_config(str(tmp_path))
    with pytest.raises(FileNotFoundError):
        load_into(DecoderModel(spec), str(tmp_path), torch.float32, "cpu")


def test_sharded_checkpoint_with_an_index(tmp_path):
    """A folder with model.safetensors.index.json and several shard files loads the same tensors as the single file."""
    single = str(tmp_path / "single")
    write_random_model(TINY_B, single, seed=1, std=0.05)
    files = open_model_tensors(single)
    tensors = {name: f.get(name) for name, f in files.items()}
    next(iter(files.values())).close()
    sharded = tmp_path / "sharded"
    sharded.mkdir()
    with open(os.path.join(single, "config.json")) as f:
        (sharded / "config.json").write_text(f.read())
    names = sorted(tensors)
    shards = {"model-00001-of-00003.safetensors": names[0::3], "model-00002-of-00003.safetensors": names[1::3],
              "model-00003-of-00003.safetensors": names[2::3]}
    weight_map = {}
    for fn, part in shards.items():
        write_safetensors(str(sharded / fn), {n: tensors[n] for n in part})
        weight_map.update({n: fn for n in part})
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    a, b = (DecoderModel(load_config(d)[1]) for d in (single, str(sharded)))
    load_into(a, single, torch.float32, "cpu")
    info = load_into(b, str(sharded), torch.float32, "cpu")
    assert info["tensors"] == len(names)
    assert torch.equal(a.embedding, b.embedding) and torch.equal(a.lm_head, b.lm_head)
    for x, y in zip(a.blocks, b.blocks):
        assert torch.equal(x.mixer.qkv, y.mixer.qkv) and torch.equal(x.feed_forward.down, y.feed_forward.down)
    # a tensor the index names in a shard that lacks it is reported like any missing tensor
    weight_map[names[0]] = "model-00002-of-00003.safetensors"
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(WeightError, match="missing"):
        load_into(DecoderModel(load_config(str(sharded))[1]), str(sharded), torch.float32, "cpu")
