"""A mixer with state of its own, defined here, is registered, built into a model through a
configuration class defined here, and stepped -- by the model runner and by the engine -- without a
change to the framework's files.  The toy is an exponential moving average:
    s_t = decay * s_{t-1} + x_t W_in^T ;  y_t = s_t W_out^T
with one state vector per request, kept in the cache manager's state slots between steps."""
import dataclasses

import pytest
import torch

import plain_llama as pl
from conftest import plain_weights
from helpers import close

pytestmark = pytest.mark.gpu


def register_toy():
    from mini_inference_engine_b200.config import LlamaConfig, register_architecture
    from mini_inference_engine_b200.config.model_config import PartSpec
    from mini_inference_engine_b200.parts import Mixer, StateNeed, register_part
    from mini_inference_engine_b200.weights import TensorSpec

    class ToyEMA(Mixer):
        def __init__(self, hidden_size, state_size, decay):
            self.hidden_size, self.state_size, self.decay = hidden_size, state_size, decay

        def tensor_specs(self):
            return {"in_proj.weight": TensorSpec((self.state_size, self.hidden_size)),
                    "out_proj.weight": TensorSpec((self.hidden_size, self.state_size))}

        def bind(self, tensors, rt):
            self.rt = rt
            self.w_in, self.w_out = rt.place(tensors["in_proj.weight"]), rt.place(tensors["out_proj.weight"])

        def cache_need(self):
            return StateNeed((self.state_size,), torch.float32)

        def forward(self, x, ctx, cache):
            u = self.rt.linear(x, self.w_in, None, out_dtype=torch.float32)          # [T, state]
            s_all = torch.empty_like(u)
            for start, n, slot in zip(ctx.host["q_start"], ctx.host["q_len"], ctx.host["state_slots"]):
                s = cache.state[slot]
                for t in range(start, start + n):
                    s = self.decay * s + u[t]
                    s_all[t] = s
                cache.state[slot] = s
            return self.rt.linear(s_all.to(self.rt.dtype), self.w_out)

    class ToyConfig(LlamaConfig):
        """Llama's layers, but every odd layer mixes with the toy instead of attention."""

        def model_spec(self):
            spec = super().model_spec()
            layers = list(spec.layers)
            for i in range(1, len(layers), 2):
                layers[i] = layers[i].with_part("mixer", PartSpec(
                    "toy_ema", dict(hidden_size=self.hidden_size, state_size=24, decay=0.9), f"model.layers.{i}.ema."))
            return dataclasses.replace(spec, layers=tuple(layers))

    register_part("mixer", "toy_ema", ToyEMA)
    register_architecture("ToyForCausalLM", ToyConfig)


TOY = dict(vocab_size=120, hidden_size=48, intermediate_size=64, num_hidden_layers=3, num_attention_heads=3,
           num_key_value_heads=3, head_dim=16, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=96,
           architectures=["ToyForCausalLM"])


def plain_toy(cfg, W, ids):
    ids = torch.as_tensor(ids)
    pos = torch.arange(len(ids))
    res = pl.embedding(W["model.embed_tokens.weight"], ids)
    for i in range(cfg["layers"]):
        p = f"model.layers.{i}."
        x = pl.rmsnorm(res, W[p + "input_layernorm.weight"], cfg["eps"])
        if i % 2:
            u = pl.linear(x, W[p + "ema.in_proj.weight"])
            s, out = torch.zeros(24), []
            for t in range(len(ids)):
                s = 0.9 * s + u[t]
                out.append(s)
            res = res + pl.linear(torch.stack(out), W[p + "ema.out_proj.weight"])
        else:
            res = res + pl.attention_layer(x, W, p + "self_attn.", cfg, pos)
        x = pl.rmsnorm(res, W[p + "post_attention_layernorm.weight"], cfg["eps"])
        res = res + pl.feed_forward(x, W, p + "mlp.")
    return pl.linear(pl.rmsnorm(res, W["model.norm.weight"], cfg["eps"]), W["lm_head.weight"])


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    register_toy()
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.weights import write_model_folder
    d = str(tmp_path_factory.mktemp("toy"))
    write_model_folder(d, load_config(dict(TOY)), seed=4, dtype=torch.float32)
    return d


def test_toy_mixer_is_built_and_stepped(toy_folder):
    from mini_inference_engine_b200.cache import RequestCache
    from mini_inference_engine_b200.engine.runner import ModelRunner
    from mini_inference_engine_b200.models import load_model
    cfg, model = load_model(toy_folder, torch.float32)
    assert type(cfg).__name__ == "ToyConfig"
    assert sorted(model.cache_layout.state) == [1] and sorted(model.cache_layout.kv) == [0, 2]
    W = plain_weights(toy_folder)
    pcfg = pl.read_config(toy_folder)
    a, b = list(range(3, 60)), list(range(70, 101))
    want_a, want_b = plain_toy(pcfg, W, a), plain_toy(pcfg, W, b)
    runner = ModelRunner(model, 12, 16, 3)
    ra, rb = RequestCache(), RequestCache()
    # a portion of a, then a portion of b beside single tokens of a, ...: the state must follow each request
    got_a = [runner.run([(ra, a[:30], range(30))])]
    pa, pb, got_b = 30, 0, []
    while pa < len(a) or pb < len(b):
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
    close(torch.cat(got_a), want_a, torch.float32, "toy model, request a")
    close(torch.cat(got_b), want_b, torch.float32, "toy model, request b")
    assert ra.state_slot != rb.state_slot and 0 not in (ra.state_slot, rb.state_slot)
    runner.cache.free(ra)
    # a new request takes a's slot and must start from zero state
    rc = RequestCache()
    got_c = runner.run([(rc, b, range(len(b)))])
    assert rc.state_slot == 3 or rc.state_slot != rb.state_slot
    close(got_c, want_b, torch.float32, "toy model, a slot used again")


def test_toy_model_generates_through_the_engine(toy_folder):
    from mini_inference_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    W, pcfg = plain_weights(toy_folder), pl.read_config(toy_folder)
    eng = LLMEngine(toy_folder, EngineConfig(use_cuda_graphs=False, max_num_batched_tokens=11, num_blocks=8, max_num_seqs=3),
                    dtype=torch.float32, load_tokenizer=False, verbose=False)
    prompts = [list(range(1, 20)), list(range(30, 42)), [5, 6], list(range(50, 80))]
    outs = eng.generate(prompts, [SamplingParams(max_tokens=m, ignore_eos=True) for m in (16, 16, 3, 16)])
    for p, o in zip(prompts, outs):
        ids = list(p)
        for tok in o.output_ids:
            logits = plain_toy(pcfg, W, ids)[-1]
            assert logits[tok] >= logits.max() - 1e-4 * logits.abs().max()
            ids.append(tok)
    assert eng.scheduler.num_preemptions > 0        # 7 usable pages: a preempted request restarts from zero state
