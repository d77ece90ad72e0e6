"""One registry from the architecture's name (``config.json["architectures"][0]``) to its
configuration class.  The configuration class is the only architecture-specific code: it
turns config.json into a ``ModelSpec`` that the generic model builds from registered parts.
The reference has no registry (inference_engine/engine.py:44 builds Llama for anything)."""
from __future__ import annotations

from .model_config import ConfigError, LlamaConfig, read_config_json

_ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_cls: type) -> None:
    """``config_cls`` needs ``from_dict(dict)``, ``to_dict()`` and ``model_spec()``."""
    _ARCHITECTURES[name] = config_cls


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; registered: {', '.join(architectures())}") from None


def load_config(path_or_dict):
    """Reads config.json (or takes its dict) and returns the typed configuration of the
    architecture it names."""
    c = path_or_dict if isinstance(path_or_dict, dict) else read_config_json(path_or_dict)
    arch = c.get("architectures")
    if not arch or not isinstance(arch, list):
        raise ConfigError("config.json lacks 'architectures' (a list with the architecture's name)")
    return config_class_for(str(arch[0])).from_dict(c)


register_architecture("LlamaForCausalLM", LlamaConfig)


def preset_names() -> list[str]:
    import os
    d = os.path.join(os.path.dirname(__file__), "presets")
    return sorted(f[:-5] for f in os.listdir(d) if f.endswith(".json"))


def load_preset(name: str):
    """A named config.json shipped with the package (the shapes the benchmarks quote), for the
    random-weights mode.  These are data files, read like any config.json."""
    import json
    import os
    path = os.path.join(os.path.dirname(__file__), "presets", name + ".json")
    if not os.path.isfile(path):
        raise ConfigError(f"no preset {name!r}; available: {', '.join(preset_names())}")
    with open(path) as f:
        return load_config(json.load(f))
