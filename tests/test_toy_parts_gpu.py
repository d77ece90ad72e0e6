"""Two more toy parts, defined here and registered without a change to the framework's files: a
feed-forward with routing (every token goes to its best expert of three, weighted by the router's
probability) and a position encoding that is no rotation and has a tensor of its own (a learned shift
of queries and keys by position).  A configuration class defined here puts them into some layers of a
model and leaves Llama's parts in the others; the model is stepped by the runner in portions and
decoded through the engine, and compared with a plain implementation written here.  The toys compute
with torch operations: they show the interfaces, not kernels."""
import dataclasses
import math

import pytest
import torch

import plain_llama as pl
from conftest import plain_weights
from helpers import close

pytestmark = pytest.mark.gpu

EXPERTS, EXPERT_SIZE, GAIN = 3, 64, 0.5


def register_toys():
    from mini_inference_engine_b200.config import LlamaConfig, register_architecture
    from mini_inference_engine_b200.config.model_config import PartSpec
    from mini_inference_engine_b200.kernels import ops
    from mini_inference_engine_b200.parts import register_part
    from mini_inference_engine_b200.parts.base import FeedForward, Part
    from mini_inference_engine_b200.weights import TensorSpec

    class RoutedReLU(FeedForward):
        """y = p_e(x) * W2_e relu(W1_e x) for the expert e with the largest router logit; the router's
        logits and probabilities in float32."""

        built = []                                     # the instances, in the order the model built them

        def __init__(self, hidden_size, expert_size, num_experts):
            self.hidden_size, self.expert_size, self.num_experts = hidden_size, expert_size, num_experts
            self.chosen = []                           # per call: the expert of every token (for the tests)
            RoutedReLU.built.append(self)

        def tensor_specs(self):
            specs = {"router.weight": TensorSpec((self.num_experts, self.hidden_size))}
            for e in range(self.num_experts):
                specs[f"experts.{e}.w1.weight"] = TensorSpec((self.expert_size, self.hidden_size))
                specs[f"experts.{e}.w2.weight"] = TensorSpec((self.hidden_size, self.expert_size))
            return specs

        def bind(self, tensors, rt):
            self.rt = rt
            self.router = rt.place(tensors["router.weight"].float())      # kept in 32 bits in either mode
            self.w1 = [rt.place(tensors[f"experts.{e}.w1.weight"]) for e in range(self.num_experts)]
            self.w2 = [rt.place(tensors[f"experts.{e}.w2.weight"]) for e in range(self.num_experts)]

        def forward(self, x, ctx):
            logits = self.rt.linear(x.float(), self.router, None, out_dtype=torch.float32)
            prob, expert = torch.softmax(logits, -1).max(-1)
            self.chosen.append(expert.cpu())
            y = torch.zeros(x.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
            for e in range(self.num_experts):
                rows = (expert == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu(self.rt.linear(x[rows].contiguous(), self.w1[e]))
                    y[rows] = self.rt.linear(h, self.w2[e], None, out_dtype=torch.float32) * prob[rows, None]
            return y.to(self.rt.dtype)

    class LearnedShift(Part):
        """q and k of every head get ``gain * table[position]`` added; nothing rotates.  Keys and values
        go to the cache through the package's own store kernel (a rotation over zero dimensions)."""

        built = []

        def __init__(self, head_dim, max_position, gain):
            self.head_dim, self.max_position, self.gain = head_dim, max_position, gain
            self.inputs = set()                        # the types of x that came in (for the tests)
            LearnedShift.built.append(self)

        def tensor_specs(self):
            return {"position_shift.weight": TensorSpec((self.max_position, self.head_dim))}

        def kernel_sources(self):
            return {"rope_cache"}

        def bind(self, tensors, rt):
            self.rt = rt
            self.table = rt.place(tensors["position_shift.weight"].float())
            self.none = torch.zeros(self.max_position, 0, dtype=torch.float32, device=rt.device)

        def rotate_and_store(self, qkv, ctx, cache, num_heads, num_kv_heads):
            D, n = self.head_dim, num_heads + num_kv_heads
            qk = qkv[:, :n * D].view(qkv.shape[0], n, D)
            shift = self.gain * self.table[ctx.positions.long()]
            qk.copy_((qk.float() + shift[:, None, :]).to(qkv.dtype))
            ops.rope_cache_write(qkv, ctx.positions, ctx.slots[cache.group], self.none, self.none, cache.k, cache.v,
                                 num_heads, num_kv_heads, D, 0, cache.page_size, write_cache=cache.writes)

        def project_rotate_and_store(self, x, w_qkv, b_qkv, ctx, cache, num_heads, num_kv_heads):
            self.inputs.add(type(x).__name__)          # a tensor, or a norm left to this product (rt.linear takes both)
            qkv = self.rt.linear(x, w_qkv, b_qkv)
            self.rotate_and_store(qkv, ctx, cache, num_heads, num_kv_heads)
            return qkv

    class ToyPartsConfig(LlamaConfig):
        """Llama's layers, but layers 0 and 2 route their feed-forward and layers 1 and 2 shift by
        position instead of rotating."""

        def model_spec(self):
            spec = super().model_spec()
            layers = list(spec.layers)
            for i in (0, 2):
                layers[i] = layers[i].with_part("feed_forward", PartSpec(
                    "toy_routed_relu", dict(hidden_size=self.hidden_size, expert_size=EXPERT_SIZE, num_experts=EXPERTS),
                    f"model.layers.{i}.moe."))
            for i in (1, 2):
                params = dict(layers[i].mixer.params)
                params["position"] = PartSpec("toy_learned_shift", dict(
                    head_dim=self.head_dim, max_position=self.max_position_embeddings, gain=GAIN))
                layers[i] = layers[i].with_part("mixer", dataclasses.replace(layers[i].mixer, params=params))
            return dataclasses.replace(spec, layers=tuple(layers))

    global routed_parts, shift_parts
    routed_parts, shift_parts = RoutedReLU.built, LearnedShift.built
    register_part("feed_forward", "toy_routed_relu", RoutedReLU)
    register_part("position", "toy_learned_shift", LearnedShift)
    register_architecture("ToyPartsForCausalLM", ToyPartsConfig)


# widths of four and eight 64-wide K tiles, so that in bfloat16 Llama's parts around the toys split K
# on single-token steps and fold their norms
TOY = dict(vocab_size=150, hidden_size=256, intermediate_size=512, num_hidden_layers=4, num_attention_heads=4,
           num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5, rope_theta=5000.0, max_position_embeddings=80,
           architectures=["ToyPartsForCausalLM"])


routed_parts = shift_parts = None


def plain_toy(cfg, W, ids, forced=None, probe=None):
    """``forced``: {layer: expert of every position}, in place of the router's own choice (its
    probability for that expert still weighs the output)."""
    ids = torch.as_tensor(ids)
    T, pos = len(ids), torch.arange(len(ids))
    H, Hkv, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    res = pl.embedding(W["model.embed_tokens.weight"], ids)
    for i in range(cfg["layers"]):
        p = f"model.layers.{i}."
        x = pl.rmsnorm(res, W[p + "input_layernorm.weight"], cfg["eps"])
        if i in (1, 2):
            a = p + "self_attn."
            shift = GAIN * W[a + "position_shift.weight"][pos][:, None, :]
            q = pl.linear(x, W[a + "q_proj.weight"]).view(T, H, D) + shift
            k = pl.linear(x, W[a + "k_proj.weight"]).view(T, Hkv, D) + shift
            v = pl.linear(x, W[a + "v_proj.weight"]).view(T, Hkv, D)
            o = pl.causal_attention(q, k, v, 1.0 / math.sqrt(D))
            res = res + pl.linear(o.reshape(T, H * D), W[a + "o_proj.weight"])
        else:
            res = res + pl.attention_layer(x, W, p + "self_attn.", cfg, pos)
        x = pl.rmsnorm(res, W[p + "post_attention_layernorm.weight"], cfg["eps"])
        if i in (0, 2):
            m = p + "moe."
            probs = torch.softmax(pl.linear(x, W[m + "router.weight"]), -1)
            if probe is not None:
                probe[i] = probs.argmax(-1)
            expert = probs.argmax(-1) if forced is None else forced[i]
            y = torch.zeros_like(res)
            for t in range(T):
                e = int(expert[t])
                h = torch.relu(pl.linear(x[t:t + 1], W[m + f"experts.{e}.w1.weight"]))
                y[t] = pl.linear(h, W[m + f"experts.{e}.w2.weight"])[0] * probs[t, e]
            res = res + y
        else:
            res = res + pl.feed_forward(x, W, p + "mlp.")
    return pl.linear(pl.rmsnorm(res, W["model.norm.weight"], cfg["eps"]), W["lm_head.weight"])


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    register_toys()
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.weights import write_model_folder
    d = str(tmp_path_factory.mktemp("toy_parts"))
    write_model_folder(d, load_config(dict(TOY)), seed=9, dtype=torch.float32)
    return d


@pytest.fixture(scope="module")
def toy_folder_bf16(toy_folder, tmp_path_factory):
    """The same model stored in bfloat16 (a tensor stored in 32 bits would stay so and run on CUDA cores)."""
    from mini_inference_engine_b200.config import load_config
    from mini_inference_engine_b200.weights import write_model_folder
    d = str(tmp_path_factory.mktemp("toy_parts_bf16"))
    write_model_folder(d, load_config(dict(TOY)), seed=9, dtype=torch.bfloat16)
    return d


def test_the_folder_holds_the_toys_tensors(toy_folder):
    W = plain_weights(toy_folder)
    assert "model.layers.0.moe.router.weight" in W and "model.layers.2.moe.experts.2.w2.weight" in W
    assert "model.layers.1.self_attn.position_shift.weight" in W
    assert "model.layers.0.mlp.gate_proj.weight" not in W and "model.layers.1.mlp.gate_proj.weight" in W
    assert "model.layers.0.self_attn.position_shift.weight" not in W


def test_toy_parts_are_built_and_stepped(toy_folder):
    from mini_inference_engine_b200.cache import RequestCache
    from mini_inference_engine_b200.engine.runner import ModelRunner
    from mini_inference_engine_b200.models import load_model
    cfg, model = load_model(toy_folder, torch.float32)
    assert type(cfg).__name__ == "ToyPartsConfig"
    W, pcfg = plain_weights(toy_folder), pl.read_config(toy_folder)
    a, b = list(range(3, 70)), list(range(90, 131))
    want_a, want_b = plain_toy(pcfg, W, a), plain_toy(pcfg, W, b)
    used = torch.softmax(pl.linear(pl.rmsnorm(pl.embedding(W["model.embed_tokens.weight"], torch.as_tensor(a)),
                                              W["model.layers.0.post_attention_layernorm.weight"], pcfg["eps"]),
                                   W["model.layers.0.moe.router.weight"]), -1).argmax(-1)
    assert len(set(used.tolist())) > 1                     # more than one expert is in play
    runner = ModelRunner(model, 14, 16, 3)
    ra, rb = RequestCache(), RequestCache()
    got_a, got_b, pa, pb = [], [], 0, 0
    sizes = [5, 2, 9, 1, 1, 13, 3, 1, 7, 2, 1, 1, 11, 4, 6, 1, 8, 2]
    step = 0
    while pa < len(a) or pb < len(b):
        na = min(sizes[step % len(sizes)], len(a) - pa)
        nb = min(sizes[(step + 5) % len(sizes)], len(b) - pb)
        entries = []
        if na:
            entries.append((ra, a[pa:pa + na], range(na)))
        if nb:
            entries.append((rb, b[pb:pb + nb], range(nb)))
        out = runner.run(entries)
        if na:
            got_a.append(out[:na])
        if nb:
            got_b.append(out[na:])
        pa, pb, step = pa + na, pb + nb, step + 1
    close(torch.cat(got_a), want_a, torch.float32, "toy parts, request a")
    close(torch.cat(got_b), want_b, torch.float32, "toy parts, request b")


def test_toy_parts_in_bfloat16_beside_the_folded_norms(toy_folder_bf16):
    """In bfloat16 Llama's parts fold their norms into their products where the part behind the norm
    can take it; a toy part cannot, so the blocks around it must fall back to the separate norm."""
    from mini_inference_engine_b200.cache import RequestCache
    from mini_inference_engine_b200.engine.runner import ModelRunner
    from mini_inference_engine_b200.models import load_model
    del routed_parts[:], shift_parts[:]
    cfg, model = load_model(toy_folder_bf16, torch.bfloat16)
    W, pcfg = plain_weights(toy_folder_bf16), pl.read_config(toy_folder_bf16)
    a = list(range(20, 75))
    runner = ModelRunner(model, 8, 16, 2)
    r = RequestCache()
    got = [runner.run([(r, a[:40], range(40))])]
    for t in range(40, len(a)):
        got.append(runner.run([(r, a[t:t + 1], [0])]))
    # two near-equal router logits may fall the other way in bfloat16, and the expert is a discrete
    # choice: the plain run takes the experts that the engine chose (the toy records them) and must
    # then agree within the usual tolerance; the choices themselves must agree nearly everywhere
    assert len(routed_parts) == 2
    forced = {layer: torch.cat(part.chosen) for layer, part in zip((0, 2), routed_parts)}
    own = plain_toy(pcfg, W, a)
    want = plain_toy(pcfg, W, a, forced)
    close(torch.cat(got), want, torch.bfloat16, "toy parts in bfloat16")
    flipped = sum(int((plain_choice(pcfg, W, a, layer, forced) != forced[layer]).sum()) for layer in (0, 2))
    assert flipped <= 3 and torch.isfinite(own).all()
    # layer 1's SwiGLU (Llama's) folded the norm in front of layer 2's attention into its last product
    # on the single-token steps, so layer 2's toy position part was handed that norm with its input;
    # layer 1's own attention stands behind a toy feed-forward, which folds nothing
    assert shift_parts[1].inputs == {"Tensor", "DeferredNorm"} and shift_parts[0].inputs == {"Tensor"}


def plain_choice(cfg, W, ids, layer, forced):
    """The plain router's own choice at ``layer``, given the forced choices in the layers before it."""
    probe = {}
    plain_toy(cfg, W, ids, forced, probe)
    return probe[layer]


def test_toy_parts_generate_through_the_engine(toy_folder):
    from mini_inference_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    W, pcfg = plain_weights(toy_folder), pl.read_config(toy_folder)
    eng = LLMEngine(toy_folder, EngineConfig(use_cuda_graphs=False, max_num_batched_tokens=12, num_blocks=12, max_num_seqs=3),
                    dtype=torch.float32, load_tokenizer=False, verbose=False)
    prompts = [list(range(1, 24)), list(range(40, 49)), [7, 8, 9], list(range(100, 131))]
    outs = eng.generate(prompts, [SamplingParams(max_tokens=m, ignore_eos=True) for m in (12, 12, 4, 12)])
    for p, o in zip(prompts, outs):
        ids = list(p)
        for tok in o.output_ids:
            logits = plain_toy(pcfg, W, ids)[-1]
            assert logits[tok] >= logits.max() - 1e-4 * logits.abs().max()
            ids.append(tok)
