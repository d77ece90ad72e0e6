"""Random-weights mode: a model folder (config.json + model.safetensors) from a
configuration and a seed.  The reference always loads a real checkpoint; the distributions
here are the usual initialisation of this architecture: matrices and embeddings N(0, 0.02),
norm weights 1, biases 0.  Each tensor has its own generator keyed by (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or in which order they are made."""
from __future__ import annotations

import hashlib
import json
import os

import torch

from .loader import TensorSpec
from .safetensors_io import write_file

INIT_STD = 0.02


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensor(seed: int, name: str, spec: TensorSpec, dtype: torch.dtype) -> torch.Tensor:
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=dtype)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype)
    if spec.init != "normal":
        raise ValueError(f"unknown init {spec.init!r} for {name}")
    t = torch.empty(spec.shape, dtype=torch.float32)
    t.normal_(0.0, INIT_STD, generator=_generator(seed, name))
    return t.to(dtype)


def random_state(expected: dict[str, TensorSpec], seed: int, dtype: torch.dtype = torch.bfloat16):
    return {name: random_tensor(seed, name, spec, dtype) for name, spec in expected.items()}


def write_model_folder(path: str, config, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` (any registered
    configuration object) and returns the folder."""
    from ..models.decoder import expected_tensors     # parts are needed only to list the tensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    state = random_state(expected_tensors(config.model_spec()), seed, dtype)
    write_file(os.path.join(path, "model.safetensors"), state, {"format": "pt", "seed": seed})
    return path
