"""The layer sizes of TinyLlama-1.1B (hidden 2048, 32 query / 4 kv heads of 64, feed-forward 5632,
vocabulary 32000) with two layers, and those of Llama-3-8B (hidden 4096, 32 query / 8 kv heads of 128,
feed-forward 14336; one layer and a cut vocabulary, to keep the folder small), so that the kernels run
at the sizes they are tuned for -- the
tcgen05 products and prefill attention, the fused rotation epilogue, the cluster-merged decode
attention -- and are still compared with the plain implementation, in float32 and in bfloat16:
a prompt whole, the same prompt in portions, and its tail decoded token by token beside another
request's portions; and, at TinyLlama's sizes, a prompt of 2,048 tokens (the length the prefill
figure is quoted at) whole, in portions of the token budget, with its last 32 tokens decoded one by
one, and through the engine with its graphs of prompt portions."""
import dataclasses
import random
import shutil

import pytest
import torch

import plain_llama as pl
from conftest import plain_weights
from helpers import close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=[("tinyllama-1.1b", dict(num_hidden_layers=2)),
                                        ("llama-3-8b", dict(num_hidden_layers=1, vocab_size=4096))],
                ids=["tinyllama-1.1b", "llama-3-8b"])
def folder(request, tmp_path_factory):
    from mini_inference_engine_b200.config import load_preset
    from mini_inference_engine_b200.weights import write_model_folder
    preset, changes = request.param
    cfg = dataclasses.replace(load_preset(preset), **changes)
    made = write_model_folder(str(tmp_path_factory.mktemp("real")), cfg, seed=21)
    yield made
    shutil.rmtree(made, ignore_errors=True)        # half a gigabyte: not left for pytest's own clean-up three runs later


@pytest.fixture(scope="module")
def oracle(folder):
    cfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(3)
    a = [rng.randrange(cfg["vocab"]) for _ in range(300)]
    b = [rng.randrange(cfg["vocab"]) for _ in range(150)]
    out = {}
    for name, rnd in (("float32", pl.identity), ("bfloat16", pl.round_bf16)):
        out[name] = (pl.forward(cfg, W, a, rnd), pl.forward(cfg, W, b, rnd))
    return a, b, out


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_real_layer_sizes_whole_portions_and_decode(dtype_name, folder, oracle):
    from mini_inference_engine_b200.cache import RequestCache
    from mini_inference_engine_b200.engine.runner import ModelRunner
    from mini_inference_engine_b200.kernels import gemm_tc, ops
    from mini_inference_engine_b200.models import load_model
    dtype = torch.float32 if dtype_name == "float32" else torch.bfloat16
    a, b, want = oracle
    want_a, want_b = want[dtype_name]
    _, model = load_model(folder, dtype)
    runner = ModelRunner(model, 64, 16, 4)

    rc = RequestCache()
    whole = runner.run([(rc, a, range(len(a)))])
    close(whole, want_a, dtype, "whole prompt")
    runner.cache.free(rc)

    # a in portions (130 + 2 + 129 tokens), then its last 39 tokens one by one beside portions of b
    ra, rb = RequestCache(), RequestCache()
    got_a = [runner.run([(ra, a[:130], range(130))]), runner.run([(ra, a[130:132], range(2))]),
             runner.run([(ra, a[132:261], range(129))])]
    got_b, pb = [], 0
    for p in range(261, 300):
        entries = [(ra, a[p:p + 1], [0])]
        nb = min(7, len(b) - pb)
        if nb:
            entries.append((rb, b[pb:pb + nb], range(nb)))
        out = runner.run(entries)
        got_a.append(out[:1])
        if nb:
            got_b.append(out[1:])
            pb += nb
    while pb < len(b):                                   # the rest of b, single tokens: pure decode steps
        got_b.append(runner.run([(rb, b[pb:pb + 1], [0])]))
        pb += 1
    torch.cuda.synchronize()
    ops.check_tc_errors()
    gemm_tc.check_error()
    close(torch.cat(got_a), want_a, dtype, "portions + decode")
    close(torch.cat(got_b), want_b, dtype, "second request in portions beside decodes")


# --------------------------------------------------------------------------- 2,048 tokens, TinyLlama's layer sizes

LONG = 2048
PLACES = sorted({0, 1, 15, 16, 127, 128, 129, 511, 512, 1023, 1024, 2015, 2016, 2047} | set(range(7, LONG, 97)))


@pytest.fixture(scope="module")
def long_case(tmp_path_factory):
    from mini_inference_engine_b200.config import load_preset
    from mini_inference_engine_b200.weights import write_model_folder
    cfg = dataclasses.replace(load_preset("tinyllama-1.1b"), num_hidden_layers=2)
    folder = write_model_folder(str(tmp_path_factory.mktemp("long")), cfg, seed=33)
    pcfg, W = pl.read_config(folder), plain_weights(folder)
    rng = random.Random(5)
    ids = [rng.randrange(pcfg["vocab"]) for _ in range(LONG)]
    head = W["lm_head.weight"]
    want = {}
    for name, rnd in (("float32", pl.identity), ("bfloat16", pl.round_bf16)):
        # the oracle's logits at every position would be 262 MB a type: the head runs on the places compared
        hidden = pl.forward(pcfg, dict(W, **{"lm_head.weight": torch.eye(pcfg["hidden"])}), ids, rnd)
        want[name] = pl.linear(hidden[PLACES], head)
    yield folder, pcfg, W, ids, want
    shutil.rmtree(folder, ignore_errors=True)


def _wanted(lo, hi):
    """Places of PLACES inside [lo, hi) as offsets into that span, and their indices into PLACES."""
    idx = [i for i, p in enumerate(PLACES) if lo <= p < hi]
    return [PLACES[i] - lo for i in idx], idx


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_2048_tokens_in_every_cutting(dtype_name, long_case):
    from mini_inference_engine_b200.cache import RequestCache
    from mini_inference_engine_b200.engine.runner import ModelRunner
    from mini_inference_engine_b200.kernels import gemm_tc, ops
    from mini_inference_engine_b200.models import load_model
    folder, _, _, ids, want = long_case
    dtype = torch.float32 if dtype_name == "float32" else torch.bfloat16
    _, model = load_model(folder, dtype)
    runner = ModelRunner(model, 2 * (LONG // 16) + 8, 16, 4)

    def cut(spans):
        rc, got = RequestCache(), torch.empty(len(PLACES), want[dtype_name].shape[1])
        for lo, hi in spans:
            offs, idx = _wanted(lo, hi)
            out = runner.run([(rc, ids[lo:hi], offs)])
            if idx:
                got[idx] = out.float().cpu()
        runner.cache.free(rc)
        return got

    cuttings = {
        "whole": [(0, LONG)],
        "portions of 512": [(i, i + 512) for i in range(0, LONG, 512)],
        "portions of changing size": [(0, 700), (700, 702), (702, 1300), (1300, 1429), (1429, 2040), (2040, 2043), (2043, 2048)],
        "all but 32 in one step, the last 32 one by one": [(0, LONG - 32)] + [(p, p + 1) for p in range(LONG - 32, LONG)],
    }
    for what, spans in cuttings.items():
        got = cut(spans)
        torch.cuda.synchronize()
        ops.check_range_errors()
        ops.check_tc_errors()
        gemm_tc.check_error()
        close(got, want[dtype_name], dtype, what)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_long_prompt_through_the_engine_with_graphs_of_its_portions(dtype_name, long_case):
    """Greedy generation from a prompt that goes in portions of the budget; the second request's
    portions all replay graphs captured during the first."""
    from mini_inference_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    folder, pcfg, W, ids, _ = long_case
    dtype = torch.float32 if dtype_name == "float32" else torch.bfloat16
    rnd, tol = (pl.identity, 1e-4) if dtype_name == "float32" else (pl.round_bf16, 2e-2)
    eng = LLMEngine(folder, EngineConfig(max_num_seqs=2, max_num_batched_tokens=512, num_blocks=LONG // 16 + 8),
                    dtype=dtype, load_tokenizer=False, verbose=False)
    prompt = ids[:LONG - 3]
    outs = [eng.generate([prompt], SamplingParams(max_tokens=3, ignore_eos=True))[0].output_ids for _ in range(2)]
    assert eng.num_portion_graph_steps >= 5 and outs[0] == outs[1]
    # the oracle for the first generated token (one forward of 2,045 tokens on the CPU); the two after
    # it are pinned by the agreement of the two runs above and by the decode tests at these sizes
    hidden = pl.forward(pcfg, dict(W, **{"lm_head.weight": torch.eye(pcfg["hidden"])}), prompt, rnd)[-1:]
    logits = pl.linear(hidden, W["lm_head.weight"])[0]
    assert logits[outs[0][0]] >= logits.max() - tol * logits.abs().max()
