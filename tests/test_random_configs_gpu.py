"""Randomly drawn configurations and engine settings against the plain implementation.

The fixed tiny configurations pin the sizes that matter; this file draws others: every head size the kernels take
(16 .. 128 in steps of 16), head counts and groupings up to 40 query heads, widths and vocabularies that are multiples
of nothing, one to three layers, both dtypes, greedy and seeded sampling, and engine settings that change how a request
is cut and batched (token budget, requests at once, captured graphs or not, steps overlapped or not, a pool so small
that requests are preempted).  Whatever the draw, every generated token must be the plain implementation's choice
for the same prefix (or tie with it within the logits tolerance).  A failure names its seed."""
import random

import pytest
import torch

import plain_llama as pl
from conftest import plain_weights
from test_engine_gpu import assert_tokens_follow_plain, engine_for

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(5000 + seed)
    kv_heads = rng.choice([1, 2, 3, 4])
    max_pos = rng.choice([96, 192, 320])
    cfg = dict(vocab_size=rng.choice([131, 257, 384, 1031, 2050]), hidden_size=rng.choice([64, 100, 136, 200, 320, 328, 520]),
               intermediate_size=rng.choice([52, 96, 150, 176, 300, 344]), num_hidden_layers=rng.choice([1, 2, 3]),
               num_attention_heads=kv_heads * rng.choice([1, 2, 3, 5, 8, 10]), num_key_value_heads=kv_heads,
               head_dim=rng.choice([16, 32, 48, 64, 80, 96, 112, 128]), rms_norm_eps=rng.choice([1e-5, 1e-6, 1e-4]),
               rope_theta=rng.choice([10000.0, 500000.0, 1000.0]), max_position_embeddings=max_pos,
               tie_word_embeddings=rng.random() < 0.5, architectures=["LlamaForCausalLM"])
    num_requests = rng.choice([5, 20, 40, 70])
    max_new = rng.choice([6, 14])
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randrange(1, max_pos - max_new))]
               for _ in range(num_requests)]
    dtype_name = rng.choice(["bfloat16", "bfloat16", "float32"])
    engine = dict(max_num_seqs=rng.choice([4, 16, 48, 80]), max_num_batched_tokens=rng.choice([32, 100, 512, 2048]),
                  use_cuda_graphs=rng.random() < 0.7, overlap_steps=rng.random() < 0.7, max_model_len=max_pos)
    engine["max_num_batched_tokens"] = max(engine["max_num_batched_tokens"], engine["max_num_seqs"])
    if rng.random() < 0.4:                       # a small pool: requests get preempted and recomputed
        engine["num_blocks"] = max(2 * (max_pos // 16 + 2), rng.randrange(20, 120))
    temperature = rng.choice([0.0, 0.0, 0.8])
    checked = rng.sample(range(num_requests), min(num_requests, 6))
    return cfg, prompts, max_new, dtype_name, engine, temperature, checked


@pytest.mark.parametrize("seed", range(200, 216))
def test_a_drawn_configuration_follows_the_plain_implementation(seed, tmp_path):
    from mini_inference_engine_b200 import SamplingParams
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.kernels import gemm_tc, ops
    from mini_inference_engine_b200.weights import write_model_folder
    cfg, prompts, max_new, dtype_name, engine, temperature, checked = draw(seed)
    folder = str(tmp_path / "drawn")
    write_model_folder(folder, load_config(cfg), seed=seed)
    plain_cfg, W = pl.read_config(folder), plain_weights(folder)
    dtype, rnd = (torch.bfloat16, pl.round_bf16) if dtype_name == "bfloat16" else (torch.float32, pl.identity)
    eng = engine_for(folder, dtype, **engine)
    outs = eng.generate(prompts, SamplingParams(max_tokens=max_new, ignore_eos=True, temperature=temperature))
    torch.cuda.synchronize()
    ops.check_range_errors()
    ops.check_tc_errors()
    gemm_tc.check_error()
    what = f"seed {seed}: {dtype_name}, T {temperature}, {cfg}, {engine}"
    assert all(len(o.output_ids) == max_new for o in outs), what
    for i in checked:
        try:
            assert_tokens_follow_plain(plain_cfg, W, rnd, prompts[i], outs[i].output_ids, dtype, temperature=temperature,
                                       seed=eng.cfg.seed, request=outs[i].seq_id)
        except AssertionError as e:
            raise AssertionError(f"{what}; request {i} ({len(prompts[i])} prompt tokens): {e}") from None


def test_the_draws_cover_the_sizes():
    """The seeds above are not all alike: several head sizes, both dtypes, graphs on and off, a preempting pool."""
    draws = [draw(s) for s in range(200, 216)]
    assert len({d[0]["head_dim"] for d in draws}) >= 5
    assert {d[3] for d in draws} == {"bfloat16", "float32"}
    assert {d[4]["use_cuda_graphs"] for d in draws} == {True, False}
    assert any("num_blocks" in d[4] for d in draws) and any(d[5] > 0 for d in draws)
    assert any(len(d[1]) > 32 and d[4]["max_num_seqs"] > 32 for d in draws)
