"""Another arrangement of parts in a layer, defined here, is registered as a block, named by a
configuration class defined here, and stepped by the model runner and the engine without a change
to the framework's files.  The toy block has ONE norm and runs its mixer and its feed-forward side by
side on the same normed input:
    x = norm(res) ; res += mixer(x) + feed_forward(x)
Layers 0 and 2 of the toy model are such blocks, layer 1 is Llama's own."""
import dataclasses

import pytest
import torch

import plain_llama as pl
from conftest import plain_weights
from helpers import close

pytestmark = pytest.mark.gpu

SIDE_BY_SIDE = (0, 2)


def register_toy():
    from mini_inference_engine_b200.config import LayerSpec, LlamaConfig, register_architecture
    from mini_inference_engine_b200.parts import register_part
    from mini_inference_engine_b200.parts.block import Block

    class SideBySide(Block):
        roles = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

        def forward(self, delta, res, ctx, cache):
            x = self.norm(delta, res)                      # res += delta (the block before left it pending)
            a = self.mixer.forward(x, ctx, cache)
            f = self.feed_forward.forward(x, ctx)
            return (a.float() + f.float()).to(a.dtype)     # the sum is the next pending delta

    class ToyBlockConfig(LlamaConfig):
        def model_spec(self):
            spec = super().model_spec()
            layers = list(spec.layers)
            for i in SIDE_BY_SIDE:
                p = layers[i].parts
                layers[i] = LayerSpec("toy_side_by_side", dict(norm=p["mixer_norm"], mixer=p["mixer"],
                                                               feed_forward=p["feed_forward"]))
            return dataclasses.replace(spec, layers=tuple(layers))

    register_part("block", "toy_side_by_side", SideBySide)
    register_architecture("ToyBlockForCausalLM", ToyBlockConfig)


TOY = dict(vocab_size=150, hidden_size=80, intermediate_size=112, num_hidden_layers=3, num_attention_heads=5,
           num_key_value_heads=1, head_dim=16, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=96,
           architectures=["ToyBlockForCausalLM"])


def plain_toy(cfg, W, ids, rnd=pl.identity):
    ids = torch.as_tensor(ids)
    pos = torch.arange(len(ids))
    res = pl.embedding(W["model.embed_tokens.weight"], ids)
    for i in range(cfg["layers"]):
        p = f"model.layers.{i}."
        x = rnd(pl.rmsnorm(res, W[p + "input_layernorm.weight"], cfg["eps"]))
        if i in SIDE_BY_SIDE:
            both = pl.attention_layer(x, W, p + "self_attn.", cfg, pos, rnd) + pl.feed_forward(x, W, p + "mlp.", rnd)
            res = res + rnd(both)
        else:
            res = res + pl.attention_layer(x, W, p + "self_attn.", cfg, pos, rnd)
            x = rnd(pl.rmsnorm(res, W[p + "post_attention_layernorm.weight"], cfg["eps"]))
            res = res + pl.feed_forward(x, W, p + "mlp.", rnd)
    return pl.linear(rnd(pl.rmsnorm(res, W["model.norm.weight"], cfg["eps"])), W["lm_head.weight"])


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    register_toy()
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.models.decoder import expected_tensors
    from mini_inference_engine_b200.weights import write_model_folder
    cfg = load_config(dict(TOY))
    names = expected_tensors(cfg.model_spec())
    assert "model.layers.0.post_attention_layernorm.weight" not in names       # a side-by-side layer has one norm
    assert "model.layers.1.post_attention_layernorm.weight" in names
    d = str(tmp_path_factory.mktemp("toyblock"))
    write_model_folder(d, cfg, seed=9, dtype=torch.float32)
    return d


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_toy_block_is_built_and_stepped(toy_folder, dt):
    from mini_inference_engine_b200.cache import RequestCache
    from mini_inference_engine_b200.engine.runner import ModelRunner
    from mini_inference_engine_b200.models import load_model
    cfg, model = load_model(toy_folder, dt)
    assert type(model.blocks[0]).__name__ == "SideBySide" and type(model.blocks[1]).__name__ == "PreNormResidual"
    W, pcfg = plain_weights(toy_folder), pl.read_config(toy_folder)
    rnd = pl.round_bf16 if dt == torch.bfloat16 else pl.identity
    a, b = list(range(3, 60)), list(range(70, 101))
    want_a, want_b = plain_toy(pcfg, W, a, rnd), plain_toy(pcfg, W, b, rnd)
    runner = ModelRunner(model, 12, 16, 3)
    ra, rb = RequestCache(), RequestCache()
    got_a = [runner.run([(ra, a[:30], range(30))])]
    pa, pb, got_b = 30, 0, []
    while pa < len(a) or pb < len(b):                 # single tokens of a beside portions of b
        entries, na, nb = [], 0, 0
        if pa < len(a):
            na = 1
            entries.append((ra, a[pa:pa + 1], [0]))
        if pb < len(b):
            nb = min(7, len(b) - pb)
            entries.append((rb, b[pb:pb + nb], range(nb)))
        out = runner.run(entries)
        if na:
            got_a.append(out[:1])
        if nb:
            got_b.append(out[na:])
        pa, pb = pa + na, pb + nb
    close(torch.cat(got_a), want_a, dt, "toy block model, request a")
    close(torch.cat(got_b), want_b, dt, "toy block model, request b")


def test_toy_block_model_generates_through_the_engine(toy_folder):
    from mini_inference_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    W, pcfg = plain_weights(toy_folder), pl.read_config(toy_folder)
    eng = LLMEngine(toy_folder, EngineConfig(max_num_batched_tokens=11, num_blocks=10, max_num_seqs=3),
                    dtype=torch.float32, load_tokenizer=False, verbose=False)
    prompts = [list(range(1, 20)), list(range(30, 42)), [5, 6]]
    outs = eng.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert eng.num_graph_steps > 0
    for p, o in zip(prompts, outs):
        ids = list(p)
        for tok in o.output_ids:
            logits = plain_toy(pcfg, W, ids)[-1]
            assert logits[tok] >= logits.max() - 1e-4 * logits.abs().max()
            ids.append(tok)
