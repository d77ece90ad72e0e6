"""Typed model configuration read from a model folder's ``config.json``.

Keys and defaults are those of inference_engine/config.py:6-42 (``ModelConfig``).  Unlike
that class, a missing key or an impossible combination is reported as one
``ConfigError`` that names the key, and the architecture name is checked against the
registry (the reference builds its Llama unconditionally, inference_engine/engine.py:44).

A configuration describes itself to the rest of the framework as *data*: ``model_spec()``
returns a ``ModelSpec`` (which parts each layer is made of, with their sizes, and in which
order layers run).  Nothing outside this file reads Llama's key names.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields


class ConfigError(ValueError):
    """A config.json that cannot describe a model this framework can build."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered ``kind`` and the constructor parameters."""
    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""          # tensor-name prefix of this part's weights in the checkpoint


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the registered arrangement ``block`` and the parts it is made of, by role name.
    Which roles there are, and which category of part fills each (mixer, feed_forward, norm, ...), is
    the block class's business (its ``roles``); Llama's ``prenorm_residual`` has ``mixer``,
    ``feed_forward``, ``mixer_norm`` and ``feed_forward_norm``.  A role reads as an attribute too:
    ``layer.mixer`` is ``layer.parts["mixer"]``."""
    block: str
    parts: dict

    def __getattr__(self, role):
        parts = object.__getattribute__(self, "parts")
        if role in parts:
            return parts[role]
        raise AttributeError(f"layer of block {object.__getattribute__(self, 'block')!r} has no part {role!r} "
                             f"(it has {', '.join(sorted(parts))})")

    def with_part(self, role: str, spec: PartSpec) -> "LayerSpec":
        """A copy of this layer with one part exchanged (or added)."""
        return LayerSpec(self.block, {**self.parts, role: spec})


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order: run ``layer`` (an index into ``layers``; the same layer may be
    named by several entries, which then share its weights) on cache ``cache`` (an id of the
    entry's choosing: entries with the same id work on the same keys and values or state).
    ``writes_cache`` is False when this run only reads what an earlier entry wrote there."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: tuple
    run_order: tuple
    final_norm: PartSpec
    head: PartSpec
    max_position: int
    eos_token_id: int
    # checkpoint tensors that the model does not read and that are no error when present (fnmatch patterns)
    ignore: tuple = ()


_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "rms_norm_eps", "max_position_embeddings")


@dataclass(frozen=True)
class LlamaConfig:
    """The Llama dense decoder (inference_engine/model.py): RMSNorm, rotate-half rotary
    position encoding over the whole head, grouped-query attention, SwiGLU feed-forward,
    tied or untied output head."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    eos_token_id: int = 2
    architecture: str = "LlamaForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, c: dict) -> "LlamaConfig":
        missing = [k for k in _REQUIRED if k not in c]
        if missing:
            raise ConfigError(f"config.json lacks required key(s): {', '.join(missing)}")
        # Keys that change the arithmetic and that this model does not honour are refused; the reference
        # does not read them (inference_engine/config.py:27-42) and would compute something else silently.
        if c.get("rope_scaling") is not None:
            raise ConfigError(f"rope_scaling {c['rope_scaling']!r} is not supported: the rotation uses "
                              "theta^(-2j/d) unscaled (remove the key only if the checkpoint was trained without it)")
        if c.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {c['hidden_act']!r} is not supported: the feed-forward is SwiGLU (silu)")
        if c.get("mlp_bias"):
            raise ConfigError("mlp_bias true is not supported: the feed-forward has no biases")
        heads = c["num_attention_heads"]
        eos = c.get("eos_token_id", 2)           # inference_engine/config.py:26,41
        if isinstance(eos, list):
            eos = eos[0]
        arch = c.get("architectures") or ["LlamaForCausalLM"]
        cfg = cls(
            vocab_size=int(c["vocab_size"]),
            hidden_size=int(c["hidden_size"]),
            intermediate_size=int(c["intermediate_size"]),
            num_hidden_layers=int(c["num_hidden_layers"]),
            num_attention_heads=int(heads),
            num_key_value_heads=int(c.get("num_key_value_heads") or heads),
            head_dim=int(c.get("head_dim") or c["hidden_size"] // heads),
            rms_norm_eps=float(c["rms_norm_eps"]),
            rope_theta=float(c.get("rope_theta", 10000.0)),
            max_position_embeddings=int(c["max_position_embeddings"]),
            tie_word_embeddings=bool(c.get("tie_word_embeddings", False)),
            attention_bias=bool(c.get("attention_bias", False)),
            eos_token_id=int(eos) if eos is not None else -1,
            architecture=str(arch[0]),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_pretrained(cls, path: str) -> "LlamaConfig":
        return cls.from_dict(read_config_json(path))

    def validate(self) -> None:
        for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim",
                  "max_position_embeddings"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"{f} must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for the rotation")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")

    def to_dict(self) -> dict:
        """The config.json that ``from_dict`` reads back to an equal configuration."""
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "architecture"}
        d["architectures"] = [self.architecture]
        d["model_type"] = "llama"
        d["hidden_act"] = "silu"
        return d

    # ------------------------------------------------------------------ description as data
    def model_spec(self) -> ModelSpec:
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            norm = dict(size=self.hidden_size, eps=self.rms_norm_eps)
            layers.append(LayerSpec("prenorm_residual", dict(
                mixer=PartSpec("attention", dict(
                    hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                    num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                    bias=self.attention_bias, window=None,
                    position=PartSpec("rope", dict(head_dim=self.head_dim, rotary_dim=self.head_dim,
                                                   theta=self.rope_theta,
                                                   max_position=self.max_position_embeddings)),
                ), p + "self_attn."),
                feed_forward=PartSpec("swiglu", dict(hidden_size=self.hidden_size,
                                                     intermediate_size=self.intermediate_size),
                                      p + "mlp."),
                mixer_norm=PartSpec("rmsnorm", norm, p + "input_layernorm."),
                feed_forward_norm=PartSpec("rmsnorm", norm, p + "post_attention_layernorm."),
            )))
        head_prefix = "model.embed_tokens." if self.tie_word_embeddings else "lm_head."
        return ModelSpec(
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            embedding=PartSpec("embedding", dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size),
                               "model.embed_tokens."),
            layers=tuple(layers),
            run_order=tuple(RunEntry(i, i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", dict(size=self.hidden_size, eps=self.rms_norm_eps), "model.norm."),
            head=PartSpec("linear_head", dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                                              tied=self.tie_word_embeddings), head_prefix),
            max_position=self.max_position_embeddings,
            eos_token_id=self.eos_token_id,
            # older checkpoints store the rotation's frequencies; a tied model may still carry a head
            ignore=("*rotary_emb.inv_freq",) + (("lm_head.weight",) if self.tie_word_embeddings else ()),
        )


def read_config_json(path: str) -> dict:
    f = os.path.join(path, "config.json")
    if not os.path.isfile(f):
        raise ConfigError(f"no config.json in {path!r}")
    with open(f) as fh:
        try:
            c = json.load(fh)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{f}: not valid JSON ({e})") from None
    if not isinstance(c, dict):
        raise ConfigError(f"{f}: expected a JSON object")
    return c
