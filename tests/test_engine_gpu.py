"""Generation through the Python entry point against the plain implementation: greedy and seeded
temperature sampling, the four ways of exercising the engine that the reference's own test uses
(default; a tiny token budget, so prompts go in several portions; no captured graphs; a tiny cache,
with preemptions asserted -- tests/test_correctness.py:41-47 of the reference), long decoding, stop
rules and refusals."""
import random

import pytest
import torch

import plain_llama as pl
from conftest import plain_weights
from helpers import TOL

pytestmark = pytest.mark.gpu
DTYPES = {"float32": (torch.float32, pl.identity), "bfloat16": (torch.bfloat16, pl.round_bf16)}


def engine_for(folder, dtype, **overrides):
    from mini_inference_engine_b200 import EngineConfig, LLMEngine
    return LLMEngine(folder, EngineConfig(**overrides), dtype=dtype, load_tokenizer=False, verbose=False)


def assert_tokens_follow_plain(cfg, W, rnd, prompt, out_ids, dtype, temperature=0.0, seed=0, request=0):
    """Every generated token must be the plain implementation's choice given the same prefix, or
    tie with it within the logits tolerance (the reference accepts ties of 2 bfloat16 ULPs,
    tests/test_correctness.py:95 of the reference).  After a tie the engine's own prefix is followed."""
    ids = list(prompt)
    for n, tok in enumerate(out_ids):
        logits = pl.forward(cfg, W, ids, rnd)[-1]
        if temperature > 0:
            scores = pl.sample_scores(logits, temperature, seed, request, n)
            slack = TOL[dtype] * logits.abs().max().item() / temperature
        else:
            scores = logits
            slack = TOL[dtype] * logits.abs().max().item()
        assert scores[tok] >= scores.max() - slack, (
            f"output {n}: engine chose {tok} (score {scores[tok]:.5f}), plain top {int(scores.argmax())} "
            f"({scores.max():.5f}), slack {slack:.2e}")
        ids.append(tok)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_greedy_generation_tiny_a(dtype_name, model_folders):
    dtype, rnd = DTYPES[dtype_name]
    folder = model_folders["tiny_a"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(0)
    prompts = [[rng.randrange(256) for _ in range(n)] for n in (5, 17, 33)]
    from mini_inference_engine_b200 import SamplingParams
    eng = engine_for(folder, dtype)
    outs = eng.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert [o.prompt_len for o in outs] == [5, 17, 33] and all(len(o.output_ids) == 8 for o in outs)
    assert all(o.ttft is not None and o.latency >= o.ttft for o in outs)
    for p, o in zip(prompts, outs):
        assert_tokens_follow_plain(cfg, W, rnd, p, o.output_ids, dtype)
    if dtype_name == "float32":                       # float32 has no near ties on random weights
        assert [o.output_ids for o in outs] == [pl.generate(cfg, W, p, 8) for p in prompts]
    assert eng.num_graph_steps > 0 and eng.cache.num_free() == eng.cache.pools[0].num_usable


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_seeded_temperature_sampling_tiny_b_in_portions_of_7(dtype_name, model_folders):
    dtype, rnd = DTYPES[dtype_name]
    folder = model_folders["tiny_b"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(1)
    prompts = [[rng.randrange(384) for _ in range(rng.randint(1, 60))] for _ in range(5)]
    from mini_inference_engine_b200 import SamplingParams
    sp = SamplingParams(max_tokens=12, temperature=0.8, ignore_eos=True)
    eng = engine_for(folder, dtype, max_num_batched_tokens=7, seed=99)
    outs = eng.generate(prompts, sp)
    for p, o in zip(prompts, outs):
        assert_tokens_follow_plain(cfg, W, rnd, p, o.output_ids, dtype, 0.8, 99, o.seq_id)
    # a request's tokens do not depend on batching: the same seed and request ids, one by one, no graphs
    if dtype_name == "float32":
        from mini_inference_engine_b200.engine import sequence
        eng2 = engine_for(folder, dtype, use_cuda_graphs=False, seed=99)
        again = []
        for p, o in zip(prompts, outs):
            sequence._ids = iter([o.seq_id])          # the same request id keys the same noise
            again.append(eng2.generate([p], sp)[0].output_ids)
        import itertools
        sequence._ids = itertools.count(10 ** 6)
        assert again == [o.output_ids for o in outs]


def test_four_ways_of_running_give_the_same_tokens(model_folders):
    folder = model_folders["tiny_b"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(2)
    prompts = [[rng.randrange(384) for _ in range(n)] for n in (40, 3, 75, 18, 64, 31)]
    want = [pl.generate(cfg, W, p, 20) for p in prompts]
    from mini_inference_engine_b200 import SamplingParams
    sp = SamplingParams(max_tokens=20, ignore_eos=True)
    ways = {"default": {}, "budget 9": dict(max_num_batched_tokens=9), "no graphs": dict(use_cuda_graphs=False),
            "tiny cache": dict(num_blocks=12), "no chunking": dict(enable_chunked_prefill=False, max_num_batched_tokens=80)}
    for name, ov in ways.items():
        eng = engine_for(folder, torch.float32, **ov)
        got = [o.output_ids for o in eng.generate(prompts, sp)]
        assert got == want, f"{name}: tokens differ from the plain implementation"
        if name == "tiny cache":
            assert eng.scheduler.num_preemptions > 0, "the tiny cache was meant to force preemptions"
        if name == "budget 9":
            assert eng.num_steps > 30
        eng.cache.check()
        assert eng.cache.num_free() == eng.cache.pools[0].num_usable


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_long_decoding_to_the_position_limit(dtype_name, model_folders):
    dtype, rnd = DTYPES[dtype_name]
    folder = model_folders["tiny_b"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    from mini_inference_engine_b200 import SamplingParams
    eng = engine_for(folder, dtype, max_model_len=256)
    out = eng.generate([[7, 8, 9]], SamplingParams(max_tokens=1000, ignore_eos=True))[0]
    assert len(out.output_ids) == 253                 # stops at max_model_len = max_position_embeddings
    assert_tokens_follow_plain(cfg, W, rnd, [7, 8, 9], out.output_ids, dtype)


def test_eos_stops_and_is_kept(model_folders, tmp_path):
    import json
    import os
    import shutil
    folder = model_folders["tiny_a"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    prompt = [3, 1, 4, 1, 5]
    plain = pl.generate(cfg, W, prompt, 10)
    eos = plain[4]
    d = str(tmp_path / "m")
    shutil.copytree(folder, d)
    with open(os.path.join(d, "config.json")) as f:
        c = json.load(f)
    c["eos_token_id"] = eos
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(c, f)
    from mini_inference_engine_b200 import SamplingParams
    eng = engine_for(d, torch.float32)
    stop = plain.index(eos) + 1
    assert eng.generate([prompt], SamplingParams(max_tokens=10))[0].output_ids == plain[:stop]
    assert eng.generate([prompt], SamplingParams(max_tokens=10, ignore_eos=True))[0].output_ids == plain


def test_refusals(model_folders):
    from mini_inference_engine_b200 import SamplingParams
    eng = engine_for(model_folders["tiny_a"], torch.float32, num_blocks=4, use_cuda_graphs=False)
    with pytest.raises(ValueError, match="vocabulary"):
        eng.add_request([1, 256])
    with pytest.raises(ValueError, match="max_model_len"):
        eng.add_request([1] * 129)
    with pytest.raises(ValueError, match="never fit"):
        eng.add_request([1] * 40, SamplingParams(max_tokens=30))     # 3 usable pages, watermark 1: 32 positions
    with pytest.raises(ValueError, match="empty"):
        eng.add_request([])
    with pytest.raises(ValueError, match="tokenizer"):
        eng.add_request("text")
    assert eng.generate([[1] * 20], SamplingParams(max_tokens=12))[0].prompt_len == 20


def test_step_api_and_counters(model_folders):
    from mini_inference_engine_b200 import SamplingParams
    eng = engine_for(model_folders["tiny_a"], torch.bfloat16)
    a = eng.add_request([1, 2, 3], SamplingParams(max_tokens=2, ignore_eos=True))
    b = eng.add_request([4] * 20, SamplingParams(max_tokens=3, ignore_eos=True))
    finished = []
    while eng.has_work():
        finished += eng.step()
    assert finished == [a, b] and a.num_output_tokens == 2 and b.num_output_tokens == 3
    assert eng.num_steps == 3 and eng.h2d_bytes > 0 and eng.d2h_bytes == 4 * 5


@pytest.mark.parametrize("overlap", [True, False])
def test_overlapped_steps_give_the_same_tokens_and_stop_at_eos(overlap, model_folders, tmp_path):
    """With overlapped steps the host launches step N+1 before it reads step N's tokens (they are fed
    back on the device).  Tokens must not change, a request that ends by EOS must not keep the token
    of the step that was already in flight, and the reference's loop over scheduler.has_work() must
    still see every end."""
    import json
    import os
    import shutil
    from mini_inference_engine_b200 import SamplingParams
    folder = model_folders["tiny_a"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(5)
    prompts = [[rng.randrange(256) for _ in range(n)] for n in (9, 30, 2, 17)]
    plain = [pl.generate(cfg, W, p, 14) for p in prompts]
    eos = plain[1][6]                                   # request 1 meets EOS at its 7th token (or earlier)
    d = str(tmp_path / "m")
    shutil.copytree(folder, d)
    with open(os.path.join(d, "config.json")) as f:
        c = json.load(f)
    c["eos_token_id"] = eos
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(c, f)
    want = [o[:o.index(eos) + 1] if eos in o else o for o in plain]
    eng = engine_for(d, torch.float32, overlap_steps=overlap, max_num_batched_tokens=16, num_blocks=9)
    seqs = [eng.add_request(p, SamplingParams(max_tokens=14)) for p in prompts]
    finished = []
    while eng.scheduler.has_work():
        finished += eng.step()
    assert sorted(s.seq_id for s in finished) == sorted(s.seq_id for s in seqs)
    assert [s.output_ids for s in seqs] == want
    assert all(s.finish_time is not None and s.first_token_time is not None for s in seqs)
    eng.cache.check()
    assert eng.cache.num_free() == eng.cache.pools[0].num_usable and not eng.has_work()


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_long_prompts_in_portions_replayed_from_graphs(dtype_name, model_folders):
    """Prompts longer than the token budget go in portions of the budget; a step that is one such
    portion is captured the second time its shape occurs and replayed from then on (tokens, positions
    and block table differ between replays, the shape does not).  The tokens must be the plain
    implementation's, and the same as without those graphs."""
    dtype, rnd = DTYPES[dtype_name]
    folder = model_folders["tiny_c"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    limit, budget = cfg["max_pos"], 32
    n = min(limit - 8, 6 * budget + 21)
    rng = random.Random(3)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)], [rng.randrange(cfg["vocab"]) for _ in range(n - 5)]]
    from mini_inference_engine_b200 import SamplingParams
    outs = {}
    for keep in (4, 0):
        eng = engine_for(folder, dtype, max_num_batched_tokens=budget, max_model_len=limit, graph_prompt_portions=keep)
        eng.PORTION_GRAPH_MIN_TOKENS = 16                  # the tiny model's positions end long before the usual 128
        res = []
        for p in prompts:                                  # one after the other: every prompt step is one portion of one prompt
            res += eng.generate([p], SamplingParams(max_tokens=6, ignore_eos=True))
        outs[keep] = [o.output_ids for o in res]
        full = n // budget + (n - 5) // budget             # steps of exactly `budget` tokens that want no logits
        # the first of those is launched kernel by kernel, the rest replay its graph; the two prompts' last portions
        # (24 and 19 tokens) are padded to the same 32 tokens: the second one replays what the first one left
        assert eng.num_portion_graph_steps == (full - 1 + 1 if keep else 0), (eng.num_portion_graph_steps, full)
        assert eng.cache.num_free() == eng.cache.pools[0].num_usable
    assert outs[4] == outs[0]
    for p, ids in zip(prompts, outs[4]):
        assert_tokens_follow_plain(cfg, W, rnd, p, ids, dtype)


@pytest.mark.parametrize("name", ["tiny_b", "tiny_d"])
def test_a_portion_graph_whose_padding_is_one_token(name, model_folders):
    """A captured portion step holds the portion and a scratch row that pads it to the captured length; how the
    tokens split between the two changes from replay to replay.  With a padding of exactly one token the scratch
    row looks like a decoding row, and the captured step has no decode kernel in it: the kernel for portions must
    serve it.  Last portions of 31, 31, 30 and 32 tokens replay one another's graph of 32 (head sizes 32 and 64:
    the mma.sync and the tcgen05 kernel)."""
    from mini_inference_engine_b200 import SamplingParams
    from mini_inference_engine_b200.kernels import ops
    folder = model_folders[name]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(17)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (63, 95, 62, 64, 127)]
    eng = engine_for(folder, torch.bfloat16, max_num_batched_tokens=32, max_model_len=160)
    eng.PORTION_GRAPH_MIN_TOKENS = 16
    outs = []
    for p in prompts:
        outs += eng.generate([p], SamplingParams(max_tokens=4, ignore_eos=True))
    assert eng.num_portion_graph_steps >= 8, eng.num_portion_graph_steps
    for p, o in zip(prompts, outs):
        assert_tokens_follow_plain(cfg, W, pl.round_bf16, p, o.output_ids, torch.bfloat16)
    ops.check_range_errors()
    ops.check_tc_errors()


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_a_portion_beside_decoding_requests_runs_as_two_graphs(dtype_name, model_folders):
    """Requests arrive while others decode, under a small token budget: most steps hold one prompt portion
    beside decoded tokens.  Such a step replays the decode bucket's graph and a graph of the portion's padded
    length (its padding is a scratch row).  Same tokens as when those steps are launched kernel by kernel, and
    the plain implementation's."""
    dtype, rnd = DTYPES[dtype_name]
    folder = model_folders["tiny_d"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(11)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (41, 7, 75, 33, 58, 19, 66, 90)]
    from mini_inference_engine_b200 import SamplingParams
    outs = {}
    for keep in (16, 0):
        eng = engine_for(folder, dtype, max_num_batched_tokens=24, max_num_seqs=4, graph_prompt_portions=keep)
        res = eng.generate(prompts, SamplingParams(max_tokens=20, ignore_eos=True))
        outs[keep] = [o.output_ids for o in res]
        if keep:
            assert eng.num_portion_graph_steps >= 8, eng.num_portion_graph_steps
            # what is left for kernel-by-kernel launches: the first occurrence of a shape, and steps with two portions
            assert eng.num_steps - eng.num_graph_steps - eng.num_portion_graph_steps < eng.num_portion_graph_steps
        else:
            assert eng.num_portion_graph_steps == 0
        eng.cache.check()
        assert eng.cache.num_free() == eng.cache.pools[0].num_usable
    if dtype_name == "float32":
        assert outs[16] == outs[0]
    for p, ids in zip(prompts, outs[16]):
        assert_tokens_follow_plain(cfg, W, rnd, p, ids, dtype)


def test_decode_graphs_by_context_bound(model_folders):
    """Decode graphs are captured per bucket AND per context bound; a step replays the one of the smallest
    bound that covers its longest request.  Requests that grow across a bound change graphs on the way,
    and the tokens are those of an engine with one graph per bucket."""
    from mini_inference_engine_b200 import SamplingParams
    folder = model_folders["tiny_a"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(4)
    prompts = [[rng.randrange(256) for _ in range(n)] for n in (20, 41, 58)]
    eng = engine_for(folder, torch.bfloat16, max_model_len=128, graph_context_bounds=(48, 64))
    assert eng.graph_bounds == [48, 64, 128]
    assert eng.decode_graph(3, 10) is eng.graphs[4, 48] and eng.decode_graph(3, 49) is eng.graphs[4, 64]
    assert eng.decode_graph(1, 128) is eng.graphs[1, 128] and eng.graphs[4, 48].buffer is eng.graphs[4, 128].buffer
    outs = eng.generate(prompts, SamplingParams(max_tokens=40, ignore_eos=True))
    one = engine_for(folder, torch.bfloat16, max_model_len=128, graph_context_bounds=())
    assert one.graph_bounds == [128]
    same = one.generate(prompts, SamplingParams(max_tokens=40, ignore_eos=True))
    assert [o.output_ids for o in outs] == [o.output_ids for o in same]
    for p, o in zip(prompts, outs):
        assert_tokens_follow_plain(cfg, W, pl.round_bf16, p, o.output_ids, torch.bfloat16)
    assert eng.num_graph_steps > 30


def test_long_contexts_cut_into_parts_under_graphs(tmp_path):
    """48 requests x 4 kv heads with a context bound of 1,600 keys: the decode graphs' attention launches are
    laid out for three parts merged through scratch memory (a cluster would take two), and every row is cut by its
    own length -- one request grows across 1,024 keys (one part, then two) while the others stay whole.  Tokens
    against the plain implementation, and the scratch that the graphs hold stays in place while eager steps ask for
    more."""
    from mini_inference_engine_b200 import SamplingParams
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.kernels import ops
    from mini_inference_engine_b200.weights import write_model_folder
    folder = str(tmp_path / "long")
    write_model_folder(folder, load_config(dict(
        vocab_size=300, hidden_size=256, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=4, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=1600,
        tie_word_embeddings=True, architectures=["LlamaForCausalLM"])), seed=21)
    cfg, W = pl.read_config(folder), plain_weights(folder)
    assert ops.decode_plan(48, 4, 1600, True, 64) == (3, "scratch", ops.LONG_PART_TILES)
    rng = random.Random(8)
    lengths = [1015, 955] + [rng.randrange(700, 1000) for _ in range(46)]
    prompts = [[rng.randrange(300) for _ in range(n)] for n in lengths]
    eng = engine_for(folder, torch.bfloat16, max_num_seqs=48, max_model_len=1600, cuda_graph_batch_sizes=(48,),
                     max_num_batched_tokens=4096)
    outs = eng.generate(prompts, SamplingParams(max_tokens=24, ignore_eos=True))
    assert eng.num_graph_steps >= 20 and all(len(o.output_ids) == 24 for o in outs)
    for i in (0, 1, 7):
        assert_tokens_follow_plain(cfg, W, pl.round_bf16, prompts[i], outs[i].output_ids, torch.bfloat16)
    ops.check_range_errors()
    ops.check_tc_errors()


@pytest.mark.parametrize("name,graphs", [("tiny_b", False), ("tiny_d", True)])
def test_decode_steps_of_many_requests_rotate_inside_attention(name, graphs, model_folders, monkeypatch):
    """Steps of decoding rows only whose q|k|v product is the library's (more than 32 rows) leave rotation and the
    cache write to the decode attention kernel; steps with a prompt portion among the rows do not.  40 requests of
    ragged lengths: both kinds of step take turns while prompts are still coming in, then decoding alone; every
    request's tokens against the plain implementation, which they could not follow with one key unrotated,
    unwritten or written twice.  Once launched one by one (head_dim 32), once under captured graphs (head_dim 64)."""
    from mini_inference_engine_b200 import SamplingParams
    from mini_inference_engine_b200.kernels import ops
    seen = {"inside": 0, "apart": 0}
    real = ops.decode_attention

    def counted(*a, **k):
        seen["inside" if k.get("rope") is not None else "apart"] += 1
        return real(*a, **k)
    monkeypatch.setattr(ops, "decode_attention", counted)
    folder = model_folders[name]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(31)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(rng.randrange(3, 50))] for _ in range(40)]
    eng = engine_for(folder, torch.bfloat16, max_num_seqs=48, max_num_batched_tokens=256, max_model_len=96,
                     use_cuda_graphs=graphs, cuda_graph_batch_sizes=(8, 48))
    captured = dict(seen)
    outs = eng.generate(prompts, SamplingParams(max_tokens=20, ignore_eos=True))
    if graphs:
        assert captured["inside"] > 0 and captured["apart"] > 0 and eng.num_graph_steps >= 10, (captured, eng.num_graph_steps)
    else:
        assert seen["inside"] >= 10 * cfg["layers"] and seen["apart"] > 0, seen
    for p, o in zip(prompts, outs):
        assert len(o.output_ids) == 20
        assert_tokens_follow_plain(cfg, W, pl.round_bf16, p, o.output_ids, torch.bfloat16)
    ops.check_range_errors()
    ops.check_tc_errors()


def test_warm_up_step_at_construction_leaves_no_trace(model_folders):
    """The engine runs one prompt step of the whole token budget on scratch rows when it is built (kernels loaded, the
    library's choices made before the first request).  It holds no page afterwards, counts no step, and the tokens of
    the requests that follow are those of an engine built without it."""
    from mini_inference_engine_b200 import SamplingParams
    folder = model_folders["tiny_d"]
    rng = random.Random(23)
    prompts = [[rng.randrange(1031) for _ in range(n)] for n in (40, 7, 150)]
    outs = {}
    for warm in (True, False):
        eng = engine_for(folder, torch.bfloat16, warm_up_prompt_step=warm, max_num_batched_tokens=64, max_model_len=192)
        assert eng.num_steps == 0 and eng.cache.num_free() == eng.cache.pools[0].num_usable
        outs[warm] = [o.output_ids for o in eng.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]
        assert eng.cache.num_free() == eng.cache.pools[0].num_usable
    assert outs[True] == outs[False]


def test_prompt_portions_through_the_paired_product(model_folders, monkeypatch):
    """The gate/up product of prompt-sized batches runs on pairs of SMs where its tiles fill the GPU; a tiny
    model never gets there, so the thresholds are lowered here: prompts of 150 - 250 tokens of `tiny_b` (width 96,
    feed-forward 256) in portions of 96 must give the plain implementation's tokens with that kernel on the path."""
    from mini_inference_engine_b200 import SamplingParams
    from mini_inference_engine_b200.kernels import gemm_tc, linear
    monkeypatch.setattr(linear, "PAIR_MIN_TOKENS", 64)
    monkeypatch.setattr(linear, "PAIR_MIN_FILL", 0.0)
    calls = []
    real = gemm_tc.gemm_pair
    monkeypatch.setattr(gemm_tc, "gemm_pair", lambda *a, **k: (calls.append(a[0].shape[0]), real(*a, **k))[1])
    folder = model_folders["tiny_b"]
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(12)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (150, 250, 97)]
    eng = engine_for(folder, torch.bfloat16, max_num_batched_tokens=96, max_model_len=256)
    outs = eng.generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True))
    assert calls and max(calls) >= 64 and min(calls) >= 64, calls
    for p, o in zip(prompts, outs):
        assert_tokens_follow_plain(cfg, W, pl.round_bf16, p, o.output_ids, torch.bfloat16)
    gemm_tc.check_error()


def test_command_line_in_process(model_folders, tmp_path, capsys):
    """The command line's sub-commands on a tiny model: a written model folder loads, generation by
    ids follows the plain implementation, and the latency and profile-decode loops report a step."""
    import json

    from mini_inference_engine_b200.__main__ import main
    out = str(tmp_path / "made")
    small = ["--overrides", '{"num_blocks": 64}']        # not the default cache of most of the device's memory
    main(["make-model", "--preset", "tiny-llama-a", "--seed", "3", "--out", out])
    capsys.readouterr()
    main(["generate", "--model", out, "--prompt-ids", "1,5,17,3", "--prompt-ids", "9,8", "--max-tokens", "6", "--ignore-eos",
          "--dtype", "float32"] + small)
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert [l["prompt_len"] for l in lines] == [4, 2] and all(len(l["output_ids"]) == 6 for l in lines)
    cfg, W = pl.read_config(out), plain_weights(out)
    assert_tokens_follow_plain(cfg, W, pl.identity, [1, 5, 17, 3], lines[0]["output_ids"], torch.float32)
    main(["latency", "--model", out, "--batches", "1", "3", "--prompt", "20", "--steps", "4"] + small)
    got = capsys.readouterr().out
    assert "bs=  1" in got and "bs=  3" in got and "ms/token-step" in got
    for graphs in ("1", "0"):
        main(["profile-decode", "--model", out, "--graphs", graphs, "--batch", "3", "--prompt", "20", "--steps", "5"] + small)
        res = json.loads(next(l for l in capsys.readouterr().out.splitlines() if l.startswith("RESULT "))[7:])
        assert res["graphs"] == (graphs == "1") and res["graph_steps"] == (5 if graphs == "1" else 0)
        assert res["kernels_per_step"] > 10 and res["device_ms_per_step"] > 0
        assert res["launch_calls_per_step"] == (1 if graphs == "1" else res["kernels_per_step"])
