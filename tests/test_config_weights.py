"""Configuration, registry and weight loading: all on the CPU."""
import json
import os
import struct

import pytest
import torch

from abacus_b200.config import (ConfigError, Qwen3Config, architecture_names, get_architecture, load_config)
from abacus_b200.weights import WeightError, load_folder, read_header, save_tensors, write_random_model
from helpers import TINY, make_model_folder, tiny_config


def raw(name="A", **over):
    d = dict(TINY[name]["cfg"], architectures=["Qwen3ForCausalLM"], model_type="qwen3")
    d.update(over)
    return d


def test_keys_and_defaults_follow_export_py():
    c = Qwen3Config.from_dict(raw("A"))
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (64, 4, 2, 16)
    d = raw("A")
    del d["head_dim"]
    assert Qwen3Config.from_dict(d).head_dim == 64 // 4  # tools/export.py:82
    d = raw("A")
    del d["rope_theta"]
    d["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}  # tools/export.py:83
    assert Qwen3Config.from_dict(d).rope_theta == 12345.0
    d = raw("A")
    del d["tie_word_embeddings"]
    assert Qwen3Config.from_dict(d).tie_word_embeddings is False  # tools/export.py:81


def test_spec_carries_every_constant_of_the_config():
    for name in TINY:
        c = tiny_config(name)
        spec = c.to_spec()
        assert len(spec.layers) == c.num_hidden_layers and spec.vocab == c.vocab_size
        assert spec.tied_head == c.tie_word_embeddings and spec.max_positions == c.max_position_embeddings
        for l, b in enumerate(spec.layers):
            m = b.mixer
            assert (m.n_heads, m.n_kv_heads, m.head_dim) == (c.num_attention_heads, c.num_key_value_heads, c.head_dim)
            assert m.scale == pytest.approx(c.head_dim ** -0.5) and m.qk_norm_eps == c.rms_norm_eps
            assert m.position.theta == c.rope_theta and m.position.rotary_dim == c.head_dim
            assert b.mixer_norm.eps == c.rms_norm_eps and b.ffn.inter == c.intermediate_size
            assert m.window == (c.sliding_window if c.layer_types[l] == "sliding_attention" else None)
        assert [e.layer for e in spec.schedule] == list(range(c.num_hidden_layers))
    c = tiny_config("C")
    assert [b.mixer.window for b in c.to_spec().layers] == [None, 24, None, 24]


def test_window_keys_of_older_exporters():
    d = raw("A", sliding_window=16, use_sliding_window=True, max_window_layers=1)
    c = Qwen3Config.from_dict(d)
    assert c.layer_types == ("full_attention", "sliding_attention") and c.sliding_window == 16
    c = Qwen3Config.from_dict(raw("A", sliding_window=16, use_sliding_window=False))
    assert c.sliding_window is None and set(c.layer_types) == {"full_attention"}


@pytest.mark.parametrize("change, word", [
    (dict(model_type="llama"), "qwen3"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope scaling"),
    (dict(layer_types=["full_attention"]), "layer_types"),
    (dict(layer_types=["full_attention", "linear_attention"]), "not built"),
    (dict(layer_types=["full_attention", "sliding_attention"], sliding_window=None), "sliding_window"),
    (dict(hidden_size=0), "hidden_size"),
    (dict(head_dim=15), "head_dim"),
    (dict(rms_norm_eps=-1.0), "rms_norm_eps"),
])
def test_bad_configs_are_refused(change, word):
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(raw("A", **change))


def test_missing_key_is_named():
    d = raw("A")
    del d["intermediate_size"], d["vocab_size"]
    with pytest.raises(ConfigError, match="intermediate_size, vocab_size"):
        Qwen3Config.from_dict(d)


def test_registry(tmp_path):
    assert "Qwen3ForCausalLM" in architecture_names()
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        get_architecture("NoSuchModel")
    folder = make_model_folder(tmp_path, "B")
    arch, cfg = load_config(folder)
    assert arch.name == "Qwen3ForCausalLM" and cfg == tiny_config("B")
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(bad))
    (bad / "config.json").write_text(json.dumps({"hidden_size": 8}))
    with pytest.raises(ConfigError, match="architectures"):
        load_config(str(bad))
    with pytest.raises(ConfigError, match="no such file"):
        load_config(str(tmp_path / "nowhere"))


def test_config_round_trip():
    for name in TINY:
        c = tiny_config(name)
        assert Qwen3Config.from_dict(c.to_dict()) == c


# ------------------------------------------------------------------ weights

def _load(folder):
    arch, cfg = load_config(folder)
    return load_folder(folder, lambda names: arch.tensor_names(cfg.to_spec(), names))


def test_random_model_folder_loads_and_keeps_bfloat16(tmp_path):
    folder = make_model_folder(tmp_path, "B")
    tensors = _load(folder)
    assert len(tensors) == 2 + 11 * 3 + 1  # embedding, final norm, 11 per layer, untied head
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    assert tensors["model.layers.2.self_attn.q_proj.weight"].shape == (6 * 32, 96)
    assert tensors["lm_head.weight"].shape == (389, 96)
    again = _load(make_model_folder(tmp_path / "again", "B"))
    assert all(torch.equal(tensors[n], again[n]) for n in tensors)  # same seed, same weights
    assert "lm_head.weight" not in _load(make_model_folder(tmp_path, "A"))  # tied: no head tensor


def test_float32_and_integer_tensors_stay_as_stored(tmp_path):
    path = str(tmp_path / "x.safetensors")
    save_tensors(path, {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
                        "b": torch.ones(4, dtype=torch.bfloat16), "t": torch.arange(5, dtype=torch.int64)})
    got = load_folder(str(tmp_path), lambda names: ({"a": (2, 3), "b": (4,), "t": (5,)}, set()))
    assert got["a"].dtype == torch.float32 and got["b"].dtype == torch.bfloat16 and got["t"].dtype == torch.int32
    assert got["a"].tolist() == [[0, 1, 2], [3, 4, 5]] and got["t"].tolist() == [0, 1, 2, 3, 4]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    arch, cfg = load_config(folder)
    tensors = dict(_load(folder))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    save_tensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        _load(folder)
    text = str(e.value)
    assert "missing (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in text
    assert "unexpected (1): model.layers.0.self_attn.rotary.inv_freq" in text
    assert "model.layers.0.mlp.down_proj.weight is [64, 64], expected [64, 128]" in text


def test_untied_config_without_head_tensor_is_tied(tmp_path):
    """tools/export.py:81: tied = tie_word_embeddings or no lm_head.weight in the checkpoint."""
    folder = make_model_folder(tmp_path, "B")
    tensors = dict(_load(folder))
    del tensors["lm_head.weight"]
    save_tensors(os.path.join(folder, "model.safetensors"), tensors)
    assert "lm_head.weight" not in _load(folder)
    # and a tied configuration tolerates a head tensor that is there
    folder = make_model_folder(tmp_path, "A")
    tensors = dict(_load(folder))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_tensors(os.path.join(folder, "model.safetensors"), tensors)
    assert "lm_head.weight" not in _load(folder)


def test_broken_files(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    path = os.path.join(folder, "model.safetensors")
    data = open(path, "rb").read()
    open(path, "wb").write(data[:len(data) - 100])
    with pytest.raises(WeightError, match="truncated"):
        read_header(path)
    open(path, "wb").write(struct.pack("<Q", 1 << 40) + data[8:])
    with pytest.raises(WeightError, match="header length"):
        read_header(path)
    open(path, "wb").write(struct.pack("<Q", 5) + b"{{{{{")
    with pytest.raises(WeightError, match="JSON"):
        read_header(path)
    os.remove(path)
    with pytest.raises(WeightError, match="no \\*.safetensors"):
        _load(folder)
    save_tensors(os.path.join(folder, "a.safetensors"), {"w": torch.zeros(2)})
    save_tensors(os.path.join(folder, "b.safetensors"), {"w": torch.zeros(2)})
    with pytest.raises(WeightError, match="both"):
        _load(folder)
    hdr = json.dumps({"w": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}).encode()
    os.remove(os.path.join(folder, "b.safetensors"))
    open(os.path.join(folder, "a.safetensors"), "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(WeightError, match="F16"):
        _load(folder)
