"""The layer sizes of TinyLlama-1.1B (hidden 2048, 32 query / 4 kv heads of 64, feed-forward 5632,
vocabulary 32000) with two layers, and those of Llama-3-8B (hidden 4096, 32 query / 8 kv heads of 128,
feed-forward 14336; one layer and a cut vocabulary, to keep the folder small), so that the kernels run
at the sizes they are tuned for -- the
tcgen05 products and prefill attention, the fused rotation epilogue, the cluster-merged decode
attention -- and are still compared with the plain implementation, in float32 and in bfloat16:
a prompt whole, the same prompt in portions, and its tail decoded token by token beside another
request's portions."""
import dataclasses
import random

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
    return write_model_folder(str(tmp_path_factory.mktemp("real")), cfg, seed=21)


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
