"""A toy model whose layers attend to a window of keys (layer 0: the last 20, layer 1: all, layer 2:
the last 37), driven through the model runner so that the cache manager releases the pages the windows
have passed and hands them to the other request, while portions of one request run beside decoded
tokens of the other.  Page 0 (where released block-table entries point) and every page that comes
back are filled with large finite values first, so that a key read from a released page, or a mask
that is off by one at a window's edge, shows in the logits.  No architecture of the reference has a
window; this proves the cache groups and the kernels' window handling together."""
import dataclasses

import pytest
import torch

import plain_llama as pl
from conftest import plain_weights
from helpers import close

pytestmark = pytest.mark.gpu

WINDOWS = {0: 20, 2: 37}
JUNK = 40.0


def register_toy():
    from mini_inference_engine_b200.config import LlamaConfig, register_architecture

    class ToyWindowConfig(LlamaConfig):
        def model_spec(self):
            spec = super().model_spec()
            layers = list(spec.layers)
            for i, w in WINDOWS.items():
                m = layers[i].mixer
                layers[i] = layers[i].with_part("mixer", dataclasses.replace(m, params=dict(m.params, window=w)))
            return dataclasses.replace(spec, layers=tuple(layers))

    register_architecture("ToyWindowForCausalLM", ToyWindowConfig)


def toy(head_dim, heads, kv_heads):
    return dict(vocab_size=200, hidden_size=heads * head_dim, intermediate_size=96, num_hidden_layers=3,
                num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, rms_norm_eps=1e-5,
                rope_theta=10000.0, max_position_embeddings=256, architectures=["ToyWindowForCausalLM"])


def plain_toy(cfg, W, ids, rnd):
    ids = torch.as_tensor(ids)
    pos = torch.arange(len(ids))
    res = pl.embedding(W["model.embed_tokens.weight"], ids)
    for i in range(cfg["layers"]):
        p = f"model.layers.{i}."
        x = rnd(pl.rmsnorm(res, W[p + "input_layernorm.weight"], cfg["eps"]))
        res = res + pl.attention_layer(x, W, p + "self_attn.", cfg, pos, rnd, WINDOWS.get(i))
        x = rnd(pl.rmsnorm(res, W[p + "post_attention_layernorm.weight"], cfg["eps"]))
        res = res + pl.feed_forward(x, W, p + "mlp.", rnd)
    return pl.linear(rnd(pl.rmsnorm(res, W["model.norm.weight"], cfg["eps"])), W["lm_head.weight"])


# head size 64 takes the tensor-core kernels in bfloat16 (and the TMA page copies), 16 the others
@pytest.mark.parametrize("dt,head_dim,heads,kv_heads", [(torch.float32, 16, 3, 3), (torch.bfloat16, 16, 4, 2),
                                                        (torch.bfloat16, 64, 2, 1)])
def test_windowed_layers_with_released_pages_used_again(dt, head_dim, heads, kv_heads, tmp_path):
    register_toy()
    from mini_inference_engine_b200.cache import RequestCache
    from mini_inference_engine_b200.cache.manager import RELEASED
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.engine.runner import ModelRunner
    from mini_inference_engine_b200.kernels import gemm_tc, ops
    from mini_inference_engine_b200.models import load_model
    from mini_inference_engine_b200.weights import write_model_folder
    folder = write_model_folder(str(tmp_path / "m"), load_config(toy(head_dim, heads, kv_heads)), seed=17, dtype=torch.float32)
    _, model = load_model(folder, dt)
    groups = model.cache_layout.groups
    assert sorted(g.window or 0 for g in groups) == [0, 20, 37]
    W, pcfg = plain_weights(folder), pl.read_config(folder)
    rnd = pl.round_bf16 if dt == torch.bfloat16 else pl.identity
    a, b = list(range(3, 183)), list(range(190, 60, -1))
    want_a, want_b = plain_toy(pcfg, W, a, rnd), plain_toy(pcfg, W, b, rnd)
    # the full group needs 12 + 9 pages for both requests; the window groups get by with far fewer,
    # so theirs go round between the two requests
    pages = [{None: 24, 20: 10, 37: 12}[g.window] for g in groups]
    runner = ModelRunner(model, pages, 16, 2)
    for t in runner.storage.kv.values():
        t.fill_(JUNK)                          # page 0 and every page not yet written hold junk, finite

    def junk_released(released):               # what the window has passed is junk from now on
        for g, ids in enumerate(released):
            for layer, (gl, _) in model.cache_layout.kv.items():
                if gl == g and ids:
                    runner.storage.kv[layer][:, ids] = JUNK

    def run(entries):                          # runner.run, with released pages junked before the next step reads
        rows = []
        for rc, tokens, want in entries:
            assert runner.cache.reserve(rc, len(tokens))
            rows.append(runner.make_row(rc, tokens, want))
        out = runner.step(rows)
        for rc, tokens, _ in entries:
            junk_released(runner.cache.advance(rc, len(tokens)))
        return out

    ra, rb = RequestCache(), RequestCache()
    got_a = [run([(ra, a[:50], range(50))])]
    pa, pb, got_b, sizes, k = 50, 0, [], [7, 2, 33, 16, 5, 19], 0
    while pa < len(a) or pb < len(b):          # single tokens of a beside portions of b, then the reverse
        entries, na, nb = [], 0, 0
        if pa < len(a):
            na = 1 if pb < len(b) else min(sizes[k % len(sizes)], len(a) - pa)
            entries.append((ra, a[pa:pa + na], range(na)))
        if pb < len(b):
            nb = min(sizes[k % len(sizes)], len(b) - pb) if pa < 120 else 1
            entries.append((rb, b[pb:pb + nb], range(nb)))
        k += 1
        out = run(entries)
        if na:
            got_a.append(out[:na])
        if nb:
            got_b.append(out[na:])
        pa, pb = pa + na, pb + nb
    torch.cuda.synchronize()
    ops.check_range_errors()
    ops.check_tc_errors()
    gemm_tc.check_error()
    close(torch.cat(got_a), want_a, dt, "windowed toy model, request a")
    close(torch.cat(got_b), want_b, dt, "windowed toy model, request b")
    for g, spec in enumerate(groups):          # the windows did release pages, and the tables show it
        if spec.window is not None:
            assert ra.tables[g][0] == RELEASED and ra.first_live[g] >= (len(a) - spec.window) // 16
            assert sum(p != RELEASED for p in ra.tables[g]) <= -(-spec.window // 16) + 1
    runner.cache.free(ra)
    runner.cache.free(rb)
    runner.cache.check()
