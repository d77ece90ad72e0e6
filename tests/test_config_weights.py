"""Configuration, registry, weight reading/checking and the random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

from conftest import TINY
from mini_inference_engine_b200.config import (ConfigError, EngineConfig, LlamaConfig, architectures, load_config,
                                               register_architecture)
from mini_inference_engine_b200.models.decoder import expected_tensors
from mini_inference_engine_b200.weights import (TensorSpec, WeightError, check_and_bind, read_file,
                                                read_model_folder, write_file, write_model_folder)


def test_llama_config_keys_and_defaults():
    c = load_config(dict(TINY["tiny_a"]))
    assert isinstance(c, LlamaConfig)
    assert (c.num_hidden_layers, c.hidden_size, c.head_dim, c.num_key_value_heads) == (2, 64, 16, 2)
    d = dict(TINY["tiny_b"])
    del d["num_key_value_heads"], d["head_dim"], d["rope_theta"]
    d["eos_token_id"] = [7, 9]
    c = load_config(d)
    assert c.num_key_value_heads == 3 and c.head_dim == 32 and c.rope_theta == 10000.0 and c.eos_token_id == 7
    assert load_config(c.to_dict()) == c                       # config.json round trip


def test_config_errors_name_the_key():
    d = dict(TINY["tiny_a"])
    del d["rms_norm_eps"], d["vocab_size"]
    with pytest.raises(ConfigError, match="rms_norm_eps") as e:
        load_config(d)
    assert "vocab_size" in str(e.value)
    with pytest.raises(ConfigError, match="multiple"):
        load_config(dict(TINY["tiny_a"], num_key_value_heads=3))
    with pytest.raises(ConfigError, match="unknown architecture"):
        load_config(dict(TINY["tiny_a"], architectures=["MambaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        load_config({k: v for k, v in TINY["tiny_a"].items() if k != "architectures"})


def test_registry_takes_another_architecture():
    class Other(LlamaConfig):
        pass
    register_architecture("OtherForCausalLM", Other)
    assert "OtherForCausalLM" in architectures()
    assert isinstance(load_config(dict(TINY["tiny_a"], architectures=["OtherForCausalLM"])), Other)


def test_model_spec_is_data_and_sizes_come_from_config():
    spec = load_config(dict(TINY["tiny_b"])).model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert m.kind == "attention" and m.params["num_heads"] == 3 and m.params["num_kv_heads"] == 1
    assert m.params["position"].params["theta"] == 500000.0
    assert spec.layers[2].feed_forward.params["intermediate_size"] == 256
    assert spec.layers[0].mixer_norm.params["eps"] == 1e-6
    assert spec.head.prefix == "model.embed_tokens."          # tied
    names = expected_tensors(spec)
    assert "lm_head.weight" not in names
    assert names["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    assert names["model.layers.0.mlp.down_proj.weight"].shape == (96, 256)
    assert "lm_head.weight" in expected_tensors(load_config(dict(TINY["tiny_a"])).model_spec())


@pytest.mark.parametrize("key,value,word", [
    ("rope_scaling", {"rope_type": "llama3", "factor": 8.0}, "rope_scaling"),
    ("rope_scaling", {"type": "linear", "factor": 2.0}, "rope_scaling"),
    ("hidden_act", "gelu", "hidden_act"),
    ("mlp_bias", True, "mlp_bias"),
])
def test_keys_that_change_the_arithmetic_and_are_not_honoured_are_refused(key, value, word):
    """The reference reads none of these (inference_engine/config.py:27-42) and would compute something
    else without a word; here such a config.json does not load."""
    with pytest.raises(ConfigError, match=word):
        load_config(dict(TINY["tiny_a"], **{key: value}))


def test_the_same_keys_at_their_neutral_values_load():
    cfg = load_config(dict(TINY["tiny_a"], rope_scaling=None, hidden_act="silu", mlp_bias=False))
    assert cfg == load_config(dict(TINY["tiny_a"]))


def test_what_a_checkpoint_may_hold_beside_the_model_is_named_by_the_spec():
    tied = load_config(dict(TINY["tiny_b"])).model_spec()
    untied = load_config(dict(TINY["tiny_a"])).model_spec()
    assert "lm_head.weight" in tied.ignore and "lm_head.weight" not in untied.ignore
    assert any("inv_freq" in pat for pat in untied.ignore)
    import inspect
    from mini_inference_engine_b200.models import decoder
    src = inspect.getsource(decoder)
    assert "inv_freq" not in src and "lm_head" not in src       # the generic model names no tensor of any architecture


def test_a_layer_is_what_its_block_class_says_it_is_made_of():
    """A block with other parts than Llama's (one norm, mixer and feed-forward side by side) is a new
    registered class, not an edit of the framework: the layer's description is role -> part."""
    from mini_inference_engine_b200.config import LayerSpec, PartSpec
    from mini_inference_engine_b200.models.decoder import _layer_parts
    from mini_inference_engine_b200.parts import register_part
    from mini_inference_engine_b200.parts.block import Block

    class SideBySide(Block):
        roles = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

    register_part("block", "toy_side_by_side_cpu", SideBySide)
    h = 32
    parts = dict(norm=PartSpec("rmsnorm", dict(size=h, eps=1e-5), "n."),
                 mixer=PartSpec("attention", dict(hidden_size=h, num_heads=2, num_kv_heads=1, head_dim=16,
                                                  position=PartSpec("none", dict(head_dim=16, max_position=8))), "a."),
                 feed_forward=PartSpec("swiglu", dict(hidden_size=h, intermediate_size=48), "f."))
    block, named = _layer_parts(LayerSpec("toy_side_by_side_cpu", parts))
    assert [p for p, _ in named] == ["n.", "a.", "f."] and block.parts() == [part for _, part in named]
    assert block.cache_need().num_kv_heads == 1 and block.cache_need().head_dim == 16
    layer = LayerSpec("toy_side_by_side_cpu", parts)
    assert layer.mixer is parts["mixer"] and layer.with_part("norm", parts["norm"]).parts == parts
    with pytest.raises(AttributeError, match="mixer_norm"):
        layer.mixer_norm
    with pytest.raises(ValueError, match="is made of"):
        _layer_parts(LayerSpec("prenorm_residual", parts))


def test_engine_config_overrides():
    c = EngineConfig.from_overrides({"max_num_batched_tokens": 48, "num_blocks": 9})
    assert c.max_num_batched_tokens == 48 and c.num_blocks == 9 and c.block_size == 16
    with pytest.raises(ValueError, match="use_triton_rmsnorm"):
        EngineConfig.from_overrides({"use_triton_rmsnorm": False})
    with pytest.raises(ValueError):
        EngineConfig(block_size=24)


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(6, dtype=torch.int64).view(2, 3),
         "c": torch.randn(4), "e": torch.empty(0, 2)}
    p = str(tmp_path / "x.safetensors")
    write_file(p, t, {"k": "v"})
    back = read_file(p)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    from safetensors.torch import load_file                   # the format is the standard one
    other = load_file(p)
    assert torch.equal(other["a"], t["a"]) and torch.equal(other["b"], t["b"])


def test_storage_dtypes_bf16_kept_f32_kept_ints_int32():
    state = {"w": torch.randn(2, 2).bfloat16(), "n": torch.ones(2), "h": torch.randn(2).half(),
             "t": torch.tensor([1, 2], dtype=torch.int64)}
    out = check_and_bind(state, {k: TensorSpec(tuple(v.shape)) for k, v in state.items()})
    assert out["w"].dtype == torch.bfloat16 and out["n"].dtype == torch.float32
    assert out["h"].dtype == torch.bfloat16 and out["t"].dtype == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = load_config(dict(TINY["tiny_a"]))
    d = write_model_folder(str(tmp_path / "m"), cfg, seed=1)
    state = dict(read_model_folder(d))
    del state["model.layers.1.mlp.up_proj.weight"], state["model.norm.weight"]
    state["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)     # ignorable
    state["model.layers.0.mlp.router.weight"] = torch.zeros(4, 64)
    state["lm_head.weight"] = torch.zeros(255, 64)
    with pytest.raises(WeightError) as e:
        check_and_bind(state, expected_tensors(cfg.model_spec()), ignore=("*rotary_emb.inv_freq",), where="m")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.mlp.router.weight"]
    assert err.wrong_shape == [("lm_head.weight", (255, 64), (256, 64))]
    msg = str(err)
    assert "missing (2)" in msg and "unexpected (1)" in msg and "wrong shape (1)" in msg and "(255, 64)" in msg


def test_no_safetensors_is_an_error(tmp_path):
    with pytest.raises(FileNotFoundError):
        read_model_folder(str(tmp_path))


def test_random_weights_mode_is_seeded_and_writes_a_folder(tmp_path):
    cfg = load_config(dict(TINY["tiny_b"]))
    a = write_model_folder(str(tmp_path / "a"), cfg, seed=5)
    b = write_model_folder(str(tmp_path / "b"), cfg, seed=5)
    c = write_model_folder(str(tmp_path / "c"), cfg, seed=6)
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    with open(os.path.join(a, "config.json")) as f:
        assert load_config(json.load(f)) == cfg
    sa, sb, sc = read_model_folder(a), read_model_folder(b), read_model_folder(c)
    assert set(sa) == set(expected_tensors(cfg.model_spec()))
    assert all(torch.equal(sa[k], sb[k]) for k in sa)
    w = "model.layers.1.self_attn.q_proj.weight"
    assert not torch.equal(sa[w], sc[w])
    assert sa[w].dtype == torch.bfloat16 and abs(sa[w].float().std().item() - 0.02) < 0.004
    assert torch.all(sa["model.layers.0.input_layernorm.weight"] == 1)
    f32 = write_model_folder(str(tmp_path / "f"), cfg, seed=5, dtype=torch.float32)
    assert read_model_folder(f32)[w].dtype == torch.float32
