"""Plain, slow Llama: the oracle every engine test compares with.

Whole sequences, no cache, no batching, one function per part, float32 on the CPU.
It shares no code with the package: it reads a model folder's ``config.json`` with
``json`` and takes weights as a plain ``{HF tensor name: tensor}`` dict.

Every function is written from the formulas of brave30/mini-inference-engine and names
the lines it restates (paths inside that project).  The file was compared once with
that project's own ``LlamaModel`` run on the CPU; ``tests/golden/make_golden.py`` is
the script that did it and ``tests/golden/*.json`` are its small outputs, which
``tests/test_plain.py`` checks on every run.

``rnd`` is a rounding hook: identity for the 32-bit oracle, a bfloat16 round trip to
imitate where a bfloat16 engine stores activations.  The hook is applied where the
engine under test writes an activation to memory (after the norm, after each
projection, after the rotation, after the attention and after the activation), while
the residual stream, the softmax, the norm statistics and the rotation angles stay in
32-bit, as they do in the engine.
"""
from __future__ import annotations

import json
import math
import os

import torch


def identity(x: torch.Tensor) -> torch.Tensor:
    return x


def round_bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


# --------------------------------------------------------------------------- config

def read_config(folder: str) -> dict:
    """Keys and defaults of inference_engine/config.py:22-42."""
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    eos = c.get("eos_token_id", 2)
    return dict(
        vocab=c["vocab_size"],
        hidden=c["hidden_size"],
        inter=c["intermediate_size"],
        layers=c["num_hidden_layers"],
        heads=heads,
        kv_heads=c.get("num_key_value_heads", heads),
        head_dim=c.get("head_dim") or c["hidden_size"] // heads,
        eps=c["rms_norm_eps"],
        theta=c.get("rope_theta", 10000.0),
        max_pos=c["max_position_embeddings"],
        tied=c.get("tie_word_embeddings", False),
        bias=c.get("attention_bias", False),
        eos=eos[0] if isinstance(eos, list) else eos,
    )


# --------------------------------------------------------------------------- parts

def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """h = E[ids]  (inference_engine/model.py:168)."""
    return table.float()[ids.long()]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w, statistics in float32
    (inference_engine/kernels/rmsnorm.py:56-65)."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return xf * torch.rsqrt(var + eps) * weight.float()


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """ang[p, j] = p * theta^(-2j/D), j < D/2, float32 (inference_engine/model.py:56-61)."""
    j = torch.arange(0, head_dim, 2, dtype=torch.int64).float()
    inv_freq = 1.0 / (theta ** (j / head_dim))
    return torch.outer(positions.float(), inv_freq)


def apply_rope(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """Rotate-half convention over the full head: x*cos + cat(-x2, x1)*sin with cos/sin
    repeated over both halves (inference_engine/model.py:64-69).  x is [T, heads, D]."""
    cos = torch.cat((ang, ang), -1).cos()[:, None, :]
    sin = torch.cat((ang, ang), -1).sin()[:, None, :]
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), -1)
    return x * cos + rot * sin


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int | None = None) -> torch.Tensor:
    """softmax(q k^T * scale + causal mask) v per head; query head h reads key/value head
    h // (H / H_kv)  (inference_engine/model.py:122-126,147-152;
    inference_engine/kernels/decode_attention.py:45).  q [T,H,D]; k, v [T,H_kv,D].
    ``window`` keeps, for query i, the keys j with i - window < j <= i (the reference has
    no window; the parameter is for the engine's attention part, which has one)."""
    T, H, D = q.shape
    G = H // k.shape[1]
    kk = k.repeat_interleave(G, dim=1)
    vv = v.repeat_interleave(G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q.float(), kk.float()) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    keep = j <= i
    if window is not None:
        keep = keep & (j > i - window)
    s = s.masked_fill(~keep[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, vv.float())


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up, silu(z) = z * sigmoid(z)  (inference_engine/model.py:181)."""
    g = gate.float()
    return g * torch.sigmoid(g) * up.float()


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """y = x W^T (+ b), W stored [out, in]  (inference_engine/model.py:172,178,180,181,185)."""
    y = x.float() @ w.float().t()
    return y if b is None else y + b.float()


# --------------------------------------------------------------------------- layers

def attention_layer(x, W, prefix, cfg, positions, rnd=identity, window=None):
    """QKV projection, rotation of q and k, causal attention, output projection
    (inference_engine/model.py:172-178)."""
    T = x.shape[0]
    H, Hkv, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    bias = (lambda n: W[prefix + n + ".bias"]) if cfg["bias"] else (lambda n: None)
    q = rnd(linear(x, W[prefix + "q_proj.weight"], bias("q_proj"))).view(T, H, D)
    k = rnd(linear(x, W[prefix + "k_proj.weight"], bias("k_proj"))).view(T, Hkv, D)
    v = rnd(linear(x, W[prefix + "v_proj.weight"], bias("v_proj"))).view(T, Hkv, D)
    ang = rope_angles(positions, D, cfg["theta"])
    q = rnd(apply_rope(q, ang))
    k = rnd(apply_rope(k, ang))
    a = rnd(causal_attention(q, k, v, 1.0 / math.sqrt(D), window))
    return rnd(linear(a.reshape(T, H * D), W[prefix + "o_proj.weight"]))


def feed_forward(x, W, prefix, rnd=identity):
    """down(silu(gate(x)) * up(x))  (inference_engine/model.py:180-181)."""
    a = rnd(swiglu(linear(x, W[prefix + "gate_proj.weight"]), linear(x, W[prefix + "up_proj.weight"])))
    return rnd(linear(a, W[prefix + "down_proj.weight"]))


def forward(cfg: dict, W: dict, ids, rnd=identity, window=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (inference_engine/model.py:161-185).
    The residual stream is summed in float32: res += mixer(norm(res)); res += ffn(norm(res))."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    pos = torch.arange(ids.numel())
    res = embedding(W["model.embed_tokens.weight"], ids)
    for i in range(cfg["layers"]):
        p = f"model.layers.{i}."
        x = rnd(rmsnorm(res, W[p + "input_layernorm.weight"], cfg["eps"]))
        res = res + attention_layer(x, W, p + "self_attn.", cfg, pos, rnd, window)
        x = rnd(rmsnorm(res, W[p + "post_attention_layernorm.weight"], cfg["eps"]))
        res = res + feed_forward(x, W, p + "mlp.", rnd)
    x = rnd(rmsnorm(res, W["model.norm.weight"], cfg["eps"]))
    head = W["model.embed_tokens.weight"] if cfg["tied"] else W["lm_head.weight"]
    return linear(x, head)


# --------------------------------------------------------------------------- sampling

def greedy(logits: torch.Tensor) -> torch.Tensor:
    """argmax over the vocabulary (inference_engine/sampling.py:15); the lowest index wins a tie."""
    return logits.float().argmax(-1)


_MASK64 = (1 << 64) - 1


def mix64(x: int) -> int:
    """A 64-bit finalizer (splitmix64's); the engine's sampling kernel uses the same integers."""
    x &= _MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK64
    return x ^ (x >> 31)


def uniform(seed: int, request: int, position: int, token: int) -> float:
    """u in (0,1) for one (sampling seed, request, output position, vocabulary entry)."""
    h = mix64(seed * 0x9E3779B97F4A7C15 + request)
    h = mix64(h ^ (position * 0xD1B54A32D192ED03 & _MASK64))
    h = mix64(h + token)
    return ((h >> 41) + 0.5) * (1.0 / (1 << 23))   # 23 bits + 0.5: exact in float32, never 0 or 1


def sample_scores(logits: torch.Tensor, temperature: float, seed: int, request: int,
                  position: int) -> torch.Tensor:
    """logit/t + Gumbel noise.  argmax of it is a draw from softmax(logit/t): the same law as
    the exponential race argmax(p / E), E ~ Exp(1), of inference_engine/sampling.py:18-22,
    because log(p/E) = logit/t - logsumexp - log E and -log E is Gumbel for E = -log u."""
    V = logits.numel()
    u = torch.tensor([uniform(seed, request, position, t) for t in range(V)], dtype=torch.float32)
    g = -torch.log(-torch.log(u))
    return logits.float() / temperature + g


def sample(logits, temperature, seed, request, position) -> int:
    if temperature <= 0:
        return int(greedy(logits))
    return int(sample_scores(logits, temperature, seed, request, position).argmax())


def generate(cfg, W, prompt, max_tokens, temperature=0.0, seed=0, request=0, rnd=identity,
             ignore_eos=True):
    """Recomputes the whole sequence for every new token; stop rules of
    inference_engine/engine.py:219-228 (the EOS token is kept)."""
    ids = list(prompt)
    out = []
    for n in range(max_tokens):
        logits = forward(cfg, W, ids, rnd)[-1]
        tok = sample(logits, temperature, seed, request, n)
        ids.append(tok)
        out.append(tok)
        if tok == cfg["eos"] and not ignore_eos:
            break
    return out
