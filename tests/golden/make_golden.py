"""Makes tests/golden/*.json: logits of brave30/mini-inference-engine's own ``LlamaModel`` run on the
CPU on two tiny random models: in float32, for the plain implementation (tests/plain_llama.py) to be
checked against, and in bfloat16 (the reference's serving type, with its roundings: residual, normed
value, rotation products and logits in bfloat16), for the bfloat16 engine to be anchored on.

    python tests/golden/make_golden.py /path/to/mini-inference-engine

The reference model is driven the way its engine drives it (inference_engine/engine.py:133-179):
the whole prompt as one fresh portion, then the same prompt as a fresh portion + a continued
portion + single decoded tokens through its eager paged-attention twin.  Weights come from
``golden_weights`` below -- a hash of (seed, tensor name, index) turned into N(0, 0.02) by
Box-Muller in numpy, so that any machine rebuilds the same tensors without a stored file.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CONFIGS = {
    "tiny_a": dict(vocab_size=256, hidden_size=64, intermediate_size=176, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5,
                   rope_theta=10000.0, max_position_embeddings=128, tie_word_embeddings=False),
    "tiny_b": dict(vocab_size=384, hidden_size=96, intermediate_size=256, num_hidden_layers=3,
                   num_attention_heads=3, num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-6,
                   rope_theta=500000.0, max_position_embeddings=256, tie_word_embeddings=True),
}
PROMPT_LEN = {"tiny_a": 21, "tiny_b": 37}


def _mix(x):
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def hashed_normal(seed: int, name: str, n: int, std: float) -> np.ndarray:
    key = np.uint64(int.from_bytes(__import__("hashlib").sha256(f"{seed}:{name}".encode()).digest()[:8], "little"))
    with np.errstate(over="ignore"):
        i = np.arange(n, dtype=np.uint64)
        a = _mix(key + np.uint64(2) * i)
        b = _mix(key + np.uint64(2) * i + np.uint64(1))
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 0.5) / 2.0 ** 53
    u2 = ((b >> np.uint64(11)).astype(np.float64) + 0.5) / 2.0 ** 53
    return (std * np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def tensor_shapes(c: dict) -> dict:
    h, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    H, Hkv, D = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    s = {"model.embed_tokens.weight": (V, h), "model.norm.weight": (h,)}
    if not c["tie_word_embeddings"]:
        s["lm_head.weight"] = (V, h)
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        s.update({p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
                  p + "self_attn.q_proj.weight": (H * D, h), p + "self_attn.k_proj.weight": (Hkv * D, h),
                  p + "self_attn.v_proj.weight": (Hkv * D, h), p + "self_attn.o_proj.weight": (h, H * D),
                  p + "mlp.gate_proj.weight": (I, h), p + "mlp.up_proj.weight": (I, h),
                  p + "mlp.down_proj.weight": (h, I)})
    return s


def golden_weights(c: dict, seed: int) -> dict:
    """float32 tensors by HF name.  Norm weights are 1 + N(0, 0.1) rather than 1, so that a norm
    that forgot its weight is caught."""
    out = {}
    for name, shape in tensor_shapes(c).items():
        n = int(np.prod(shape))
        if name.endswith("norm.weight"):
            v = 1.0 + hashed_normal(seed, name, n, 0.1)
        else:
            v = hashed_normal(seed, name, n, 0.05)
        out[name] = torch.from_numpy(v.reshape(shape).copy())
    return out


def golden_prompt(c: dict, seed: int, n: int) -> list:
    with np.errstate(over="ignore"):
        x = _mix(np.uint64(seed) + np.arange(n, dtype=np.uint64))
    return [int(v) for v in (x % np.uint64(c["vocab_size"]))]


def run_reference(ref_root: str, name: str, seed: int) -> dict:
    sys.path.insert(0, ref_root)
    from inference_engine.config import ModelConfig
    from inference_engine.model import AttentionMetadata, KVCache, LlamaModel, PrefillChunk

    c = CONFIGS[name]
    cfg = ModelConfig(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], intermediate_size=c["intermediate_size"],
                      num_layers=c["num_hidden_layers"], num_heads=c["num_attention_heads"],
                      num_kv_heads=c["num_key_value_heads"], head_dim=c["head_dim"], rms_norm_eps=c["rms_norm_eps"],
                      rope_theta=c["rope_theta"], max_position_embeddings=c["max_position_embeddings"],
                      tie_word_embeddings=c["tie_word_embeddings"], attention_bias=False, eos_token_id=2)
    W = golden_weights(c, seed)
    model = LlamaModel(cfg, {k: v.clone() for k, v in W.items()}, device="cpu", dtype=torch.float32,
                       use_triton_rmsnorm=False, use_triton_decode_attn=False)
    bs, nb = 16, 16
    model.kv_cache = KVCache(cfg, nb, bs, torch.float32, "cpu")
    n = PROMPT_LEN[name]
    ids = golden_prompt(c, seed, n)
    table = [5, 2, 9, 7][: -(-n // bs)]

    def slots(a, b):
        return torch.tensor([table[p // bs] * bs + p % bs for p in range(a, b)])

    # whole prompt, one fresh portion
    meta = AttentionMetadata(slot_mapping=slots(0, n), prefills=[PrefillChunk(0, n, n, None, None)])
    whole = model.forward(torch.tensor(ids), torch.arange(n), meta)

    # fresh portion + continued portion + two decoded tokens, other pages
    model.kv_cache = KVCache(cfg, nb, bs, torch.float32, "cpu")
    table = [11, 3, 14, 6][: -(-n // bs)]
    a, b = n // 2, n - 2
    out = []
    meta = AttentionMetadata(slot_mapping=slots(0, a), prefills=[PrefillChunk(0, a, a, None, None)])
    out.append(model.forward(torch.tensor(ids[:a]), torch.arange(a), meta))
    pos = torch.arange(b)
    ctx_slots = slots(0, b)
    mask = pos[None, :] <= (a + torch.arange(b - a))[:, None]
    meta = AttentionMetadata(slot_mapping=slots(a, b), prefills=[PrefillChunk(0, b - a, b, ctx_slots, mask)])
    out.append(model.forward(torch.tensor(ids[a:b]), torch.arange(a, b), meta))
    for p in range(b, n):
        meta = AttentionMetadata(slot_mapping=slots(p, p + 1), num_decode=1,
                                 block_tables=torch.tensor([table], dtype=torch.int32),
                                 context_lens=torch.tensor([p + 1], dtype=torch.int32), max_decode_context=p + 1)
        out.append(model.forward(torch.tensor(ids[p:p + 1]), torch.tensor([p]), meta))
    cut = torch.cat(out, 0)
    keep = [0, 1, n // 2, n - 2, n - 1]

    # the same model as the reference serves it: bfloat16 weights, activations, tables and logits
    # (inference_engine/engine.py:36, inference_engine/model.py:84-115), whole prompt
    model16 = LlamaModel(cfg, {k: v.clone() for k, v in W.items()}, device="cpu", dtype=torch.bfloat16,
                         use_triton_rmsnorm=False, use_triton_decode_attn=False)
    model16.kv_cache = KVCache(cfg, nb, bs, torch.bfloat16, "cpu")
    table = [5, 2, 9, 7][: -(-n // bs)]
    meta = AttentionMetadata(slot_mapping=slots(0, n), prefills=[PrefillChunk(0, n, n, None, None)])
    whole16 = model16.forward(torch.tensor(ids), torch.arange(n), meta).float()
    return dict(config=c, seed=seed, prompt=ids, positions=keep,
                logits=[[float(x) for x in whole[p]] for p in keep],
                logits_bf16=[[float(x) for x in whole16[p]] for p in keep],
                reference_bf16_vs_float32_max_abs=float((whole16 - whole).abs().max()),
                reference_cut_vs_whole_max_abs=float((cut - whole).abs().max()))


def reference_root() -> str:
    if len(sys.argv) != 2 or not os.path.isdir(os.path.join(sys.argv[1], "inference_engine")):
        sys.exit(__doc__)
    return sys.argv[1]


if __name__ == "__main__":
    ref = reference_root()
    for name, seed in (("tiny_a", 11), ("tiny_b", 12)):
        g = run_reference(ref, name, seed)
        with open(os.path.join(HERE, name + ".json"), "w") as f:
            json.dump(g, f)
        print(name, "written; reference cut-vs-whole max abs", g["reference_cut_vs_whole_max_abs"])


# --------------------------------------------------------------------------- scheduler decisions

SCHED_CASES = {
    "roomy": dict(prompts=[5, 17, 33, 40, 3], max_tokens=[8, 8, 8, 4, 12], budget=48, num_blocks=64, max_num_seqs=4),
    "tight_pages": dict(prompts=[30, 30, 30, 30], max_tokens=[40, 40, 40, 40], budget=64, num_blocks=9, max_num_seqs=4),
    "tiny_budget": dict(prompts=[20, 9, 1, 50], max_tokens=[5, 5, 5, 5], budget=7, num_blocks=32, max_num_seqs=3),
}


def run_reference_scheduler(ref_root: str, case: dict) -> dict:
    """Drives the reference's Scheduler + BlockAllocator with the bookkeeping of its engine step
    (inference_engine/engine.py:212-229), a token being appended whenever a portion reaches the end."""
    sys.path.insert(0, ref_root)
    from inference_engine.block_manager import BlockAllocator
    from inference_engine.config import EngineConfig
    from inference_engine.sampling import SamplingParams
    from inference_engine.scheduler import Scheduler
    from inference_engine.sequence import Sequence

    cfg = EngineConfig(max_num_seqs=case["max_num_seqs"], max_num_batched_tokens=case["budget"])
    alloc = BlockAllocator(case["num_blocks"], 16)
    sched = Scheduler(cfg, alloc)
    seqs = [Sequence([1] * p, SamplingParams(max_tokens=m, ignore_eos=True))
            for p, m in zip(case["prompts"], case["max_tokens"])]
    for s in seqs:
        sched.add(s)
    steps = []
    while sched.has_work() and len(steps) < 2000:
        batch = sched.schedule()
        steps.append([[seqs.index(s), n] for s, n in batch])
        for s, n in batch:
            last = s.num_computed + n == s.num_tokens
            s.num_computed += n
            if last:
                s.token_ids.append(7)
                if s.num_output_tokens >= s.params.max_tokens:
                    sched.finish(s)
    return dict(case=case, steps=steps, preemptions=sched.num_preemptions, free_at_end=alloc.num_free)


if __name__ == "__main__":
    ref = reference_root()
    out = {name: run_reference_scheduler(ref, case) for name, case in SCHED_CASES.items()}
    with open(os.path.join(HERE, "scheduler.json"), "w") as f:
        json.dump(out, f)
    print("scheduler:", {k: (len(v["steps"]), v["preemptions"]) for k, v in out.items()})
