import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# Two tiny configurations that differ in every size and option (layers, widths, head counts and
# grouping, head size, feed-forward width, vocabulary, rope base, eps, position limit, tying).
TINY = {
    "tiny_a": dict(vocab_size=256, hidden_size=64, intermediate_size=176, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5,
                   rope_theta=10000.0, max_position_embeddings=128, tie_word_embeddings=False,
                   architectures=["LlamaForCausalLM"]),
    # sizes that are multiples of nothing: odd vocabulary, width 100, feed-forward 52, five heads without grouping
    "tiny_c": dict(vocab_size=131, hidden_size=100, intermediate_size=52, num_hidden_layers=1,
                   num_attention_heads=5, num_key_value_heads=5, head_dim=16, rms_norm_eps=1e-4,
                   rope_theta=1000.0, max_position_embeddings=96, tie_word_embeddings=True,
                   architectures=["LlamaForCausalLM"]),
    "tiny_b": dict(vocab_size=384, hidden_size=96, intermediate_size=256, num_hidden_layers=3,
                   num_attention_heads=3, num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-6,
                   rope_theta=500000.0, max_position_embeddings=256, tie_word_embeddings=True,
                   architectures=["LlamaForCausalLM"]),
    # wide enough (five 64-wide K tiles) that single-token steps in bfloat16 split K on the tensor-core
    # product and fold rotation, residual sums and norms into it; a feed-forward width whose doubled
    # size is no multiple of 16, an odd vocabulary, three query heads a key head
    "tiny_d": dict(vocab_size=1031, hidden_size=320, intermediate_size=300, num_hidden_layers=2,
                   num_attention_heads=6, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5,
                   rope_theta=50000.0, max_position_embeddings=192, tie_word_embeddings=False,
                   architectures=["LlamaForCausalLM"]),
}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Model folders (config.json + model.safetensors, bfloat16 weights) of the tiny configurations,
    written by the package's random-weights mode into a temporary folder."""
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.weights import write_model_folder
    out = {}
    for i, (name, c) in enumerate(TINY.items()):
        d = str(tmp_path_factory.mktemp(name))
        write_model_folder(d, load_config(dict(c)), seed=100 + i)
        out[name] = d
    return out


def plain_weights(folder: str) -> dict:
    """The folder's tensors as float32 by name, read without the package's loader."""
    from safetensors.torch import load_file
    return {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def golden(name: str) -> dict:
    with open(os.path.join(os.path.dirname(__file__), "golden", name + ".json")) as f:
        return json.load(f)
