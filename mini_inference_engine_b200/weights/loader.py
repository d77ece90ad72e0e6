"""Weights by tensor name.

``read_model_folder`` merges every ``*.safetensors`` of a folder in sorted order
(inference_engine/weights.py:15-21).  ``check_and_bind`` compares what the files hold with
what the model's parts declare and raises ONE ``WeightError`` that lists every missing
tensor, every unexpected tensor and every wrong shape (the reference fails on the first
missing name with a bare KeyError and ignores the rest, inference_engine/model.py:93-94).

Storage rule: floating-point tensors are kept in bfloat16 when the file holds them in 16 bits,
a tensor that the file holds in 32 bits stays in 32 bits, and integer tables become int32.
The float32 mode of the engine widens everything to float32 afterwards (exact).
"""
from __future__ import annotations

import fnmatch
import glob
import os
from dataclasses import dataclass

import torch

from .safetensors_io import read_file


class WeightError(ValueError):
    """The checkpoint does not match the model: carries the three lists."""

    def __init__(self, where: str, missing, unexpected, wrong_shape):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights in {where} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: file {tuple(g)} != model {tuple(w)}" for n, g, w in self.wrong_shape))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects of one checkpoint tensor."""
    shape: tuple
    init: str = "normal"      # random-weights mode: "normal" (N(0, 0.02)), "ones" or "zeros"


def read_model_folder(path: str) -> dict[str, torch.Tensor]:
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {path!r}")
    state: dict[str, torch.Tensor] = {}
    for f in files:
        state.update(read_file(f))
    return state


def storage_dtype(t: torch.Tensor) -> torch.dtype:
    if t.dtype in (torch.float32, torch.float64):
        return torch.float32
    if t.dtype.is_floating_point:
        return torch.bfloat16
    return torch.int32


def check_and_bind(state: dict[str, torch.Tensor], expected: dict[str, TensorSpec], *,
                   ignore: tuple = (), where: str = "checkpoint") -> dict[str, torch.Tensor]:
    """Returns ``{name: tensor}`` for exactly the expected names, each in its storage dtype."""
    missing = [n for n in expected if n not in state]
    unexpected = [n for n in state if n not in expected
                  and not any(fnmatch.fnmatchcase(n, pat) for pat in ignore)]
    wrong = [(n, tuple(state[n].shape), tuple(s.shape)) for n, s in expected.items()
             if n in state and tuple(state[n].shape) != tuple(s.shape)]
    if missing or unexpected or wrong:
        raise WeightError(where, sorted(missing), sorted(unexpected), sorted(wrong))
    return {n: state[n].to(storage_dtype(state[n])) for n in expected}
