"""Configuration and weight loading, on the CPU."""
import copy
import json
import os

import pytest
import torch

from tiny import CONFIGS, TINY_A, TINY_B, make_folder
from tuff_b200.config import (ConfigError, Lfm2Config, adjusted_ffn_dim, config_from_dict, load_config,
                              registered_architectures)
from tuff_b200.models import Model
from tuff_b200.weights import ModelFiles, SafetensorsError, WeightError, load_checkpoint, write_safetensors


def test_ffn_adjust_table():
    assert adjusted_ffn_dim(8192, True, None, 256) == 5632
    assert adjusted_ffn_dim(6656, True, None, 256) == 4608
    assert adjusted_ffn_dim(10752, True, None, 256) == 7168
    assert adjusted_ffn_dim(8192, False, None, 256) == 8192
    assert adjusted_ffn_dim(384, True, 1.0, 32) == 256
    assert adjusted_ffn_dim(384, True, 1.3, 32) == 352     # int(1.3 * 256) = 332 -> 352


def test_lfm2_config_fields():
    arch, a = config_from_dict(TINY_A)
    _, b = config_from_dict(TINY_B)
    assert arch.name == "Lfm2ForCausalLM" and "Lfm2ForCausalLM" in registered_architectures()
    assert (a.hidden_size, a.head_dim, a.ffn_dim, a.conv_L_cache, a.tie_embedding) == (64, 16, 192, 3, True)
    assert a.layer_types == ("conv", "attention", "conv", "attention") and a.full_attn_idxs == (1, 3)
    assert (b.hidden_size, b.head_dim, b.ffn_dim, b.conv_L_cache, b.tie_embedding) == (96, 24, 256, 4, False)
    assert b.layer_types == ("attention", "conv", "conv", "attention", "conv", "conv")
    assert b.rope_theta == 1e6 and b.norm_eps == 1e-6 and b.num_key_value_heads == 1
    # a written config reads back equal
    assert Lfm2Config.from_dict(a.to_dict()) == a and Lfm2Config.from_dict(b.to_dict()) == b


def test_both_names_of_the_ffn_width():
    same = dict(TINY_A, block_ff_dim=TINY_A["intermediate_size"])
    assert config_from_dict(same)[1].ffn_dim == config_from_dict(TINY_A)[1].ffn_dim
    only = {k: v for k, v in same.items() if k != "intermediate_size"}
    assert config_from_dict(only)[1].ffn_dim == config_from_dict(TINY_A)[1].ffn_dim


def test_lfm2_1p2b_shape():
    raw = dict(architectures=["Lfm2ForCausalLM"], hidden_size=2048, num_hidden_layers=16, num_attention_heads=32,
               num_key_value_heads=8, intermediate_size=8192, block_auto_adjust_ff_dim=True, block_multiple_of=256,
               vocab_size=65536, rope_theta=1e6, norm_eps=1e-5, conv_L_cache=3, full_attn_idxs=[2, 5, 8, 10, 12, 14],
               tie_embedding=True)
    arch, cfg = config_from_dict(raw)
    assert cfg.ffn_dim == 5632 and cfg.head_dim == 64 and len(cfg.conv_idxs) == 10
    import math
    n = sum(math.prod(d.shape) for d in Model(arch.model_spec(cfg)).expected_tensors().values())
    assert n == 918_682_368


@pytest.mark.parametrize("mutate, word", [
    (lambda c: c.pop("hidden_size"), "hidden_size"),
    (lambda c: c.update(num_key_value_heads=3), "multiple"),
    (lambda c: c.update(layer_types=["conv"]), "layer_types"),
    (lambda c: c.update(layer_types=["conv", "full_attention", "conv", "mamba"]), "mamba"),
    (lambda c: c.update(full_attn_idxs=[0, 1]), "disagree"),
    (lambda c: c.update(conv_L_cache=1), "conv_L_cache"),
    (lambda c: c.update(norm_eps="small"), "norm_eps"),
    (lambda c: c.update(vocab_size=0), "vocab_size"),
    (lambda c: c.update(conv_bias=True), "conv_bias"),
    (lambda c: c.update(architectures=["NoSuchModel"]), "not registered"),
    (lambda c: (c.pop("layer_types"),), "layer_types"),
    (lambda c: c.update(hidden_size=66), "head_dim"),
    (lambda c: c.update(block_ff_dim=c["intermediate_size"] + 64), "block_ff_dim"),
])
def test_config_errors(mutate, word):
    c = copy.deepcopy(TINY_A)
    mutate(c)
    with pytest.raises(ConfigError) as e:
        config_from_dict(c)
    assert word in str(e.value)


def test_safetensors_round_trip(tmp_path):
    import safetensors.torch as st
    ts = {"a": torch.randn(3, 5).to(torch.bfloat16), "b.c": torch.arange(7, dtype=torch.int32),
          "z": torch.randn(2, 2, 2), "s": torch.tensor(3.5)}
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, ts.items(), {"k": "v"})
    theirs = st.load_file(p)                      # the library reads what we wrote
    ours = ModelFiles(str(tmp_path))
    for n, t in ts.items():
        assert torch.equal(theirs[n], t) and torch.equal(ours.tensor(n), t) and ours.entries[n].dtype == t.dtype
    st.save_file({k: v.contiguous() for k, v in ts.items()}, p)   # and we read what the library writes
    ours = ModelFiles(str(tmp_path))
    for n, t in ts.items():
        assert torch.equal(ours.tensor(n), t)
    with open(p, "r+b") as f:
        f.write(b"\xff" * 8)
    with pytest.raises(SafetensorsError):
        ModelFiles(str(tmp_path))


def _expected(folder):
    arch, cfg = load_config(folder)
    return Model(arch.model_spec(cfg)).expected_tensors()


def test_weights_kept_dtypes(tmp_path):
    folder = make_folder(tmp_path, "tiny_b")
    exp = _expected(folder)
    w = load_checkpoint(folder, exp, torch.bfloat16, "cpu")
    assert w["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert w["model.layers.0.operator_norm.weight"].dtype == torch.float32          # small vectors in fp32
    assert w["model.layers.1.conv.conv.weight"].shape == (96, 1, 4)
    w32 = load_checkpoint(folder, exp, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["lm_head.weight"], w["lm_head.weight"].float())
    # a matrix stored in 32-bit stays so in the bfloat16 engine
    f32 = make_folder(tmp_path / "f32", "tiny_b", store_dtype=torch.float32)
    w = load_checkpoint(f32, exp, torch.bfloat16, "cpu")
    assert w["lm_head.weight"].dtype == torch.float32


def test_weight_error_lists_everything(tmp_path):
    folder = make_folder(tmp_path, "tiny_a")
    files = ModelFiles(folder)
    ts = {n: files.tensor(n) for n in files.entries}
    files.close()
    del ts["model.layers.1.self_attn.k_proj.weight"]
    del ts["model.embedding_norm.weight"]
    ts["model.layers.0.feed_forward.w1.weight"] = torch.zeros(191, 64, dtype=torch.bfloat16)
    ts["model.layers.2.self_attn.q_proj.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)   # attention tensor on a conv layer
    ts["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)                         # the head is tied
    write_safetensors(os.path.join(folder, "model.safetensors"), ts.items())
    with pytest.raises(WeightError) as e:
        load_checkpoint(folder, _expected(folder), torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["model.embedding_norm.weight", "model.layers.1.self_attn.k_proj.weight"]
    assert err.unexpected == ["lm_head.weight", "model.layers.2.self_attn.q_proj.weight"]
    assert [(n, tuple(a), tuple(b)) for n, a, b in err.wrong_shape] == \
        [("model.layers.0.feed_forward.w1.weight", (192, 64), (191, 64))]
    msg = str(err)
    for word in ("missing", "unexpected", "wrong shape", "k_proj", "lm_head", "[192, 64]", "[191, 64]"):
        assert word in msg


def test_random_weights_are_seeded_per_tensor(tmp_path):
    a = ModelFiles(make_folder(tmp_path / "x", "tiny_a"))
    b = ModelFiles(make_folder(tmp_path / "y", "tiny_a"))
    for n in a.entries:
        assert torch.equal(a.tensor(n), b.tensor(n))
    w = a.tensor("model.layers.0.feed_forward.w1.weight").float()
    g = a.tensor("model.layers.0.ffn_norm.weight").float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(g.mean().item() - 1.0) < 0.03
    cfg = json.load(open(os.path.join(a.model_dir, "config.json")))
    assert cfg["architectures"] == ["Lfm2ForCausalLM"]
