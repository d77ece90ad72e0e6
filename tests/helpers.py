"""Shared by the GPU tests: tolerances, scattered page tables, and a StepContext built by hand."""
import math
import random

import torch

# Tolerances, as a fraction of the largest reference magnitude.  float32: only the order of sums
# differs.  bfloat16: the bound of the reference's own kernel tests (atol = rtol = 2e-2,
# tests/test_kernels.py:28,59 of the reference).
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def close(got: torch.Tensor, want: torch.Tensor, dtype, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    scale = max(want.abs().max().item(), 1e-6)
    err = (got - want).abs().max().item()
    assert err <= TOL[dtype] * scale, f"{what}: max abs error {err:.3e} > {TOL[dtype]:g} x {scale:.3e}"
    return err / scale


def first_bad_row(got, want, dtype):
    """Index of the first row beyond tolerance (to ask what is special about its place)."""
    got, want = got.float().cpu(), want.float().cpu()
    scale = max(want.abs().max().item(), 1e-6)
    bad = ((got - want).abs().amax(-1) > TOL[dtype] * scale).nonzero()
    return int(bad[0]) if bad.numel() else None


def scattered_tables(ctx_lens, page, num_pages, seed=0):
    """Block tables with randomly permuted physical pages; page 0 (scratch) is never used."""
    rng = random.Random(seed)
    ids = list(range(1, num_pages))
    rng.shuffle(ids)
    tables, i = [], 0
    for c in ctx_lens:
        n = math.ceil(c / page)
        assert i + n <= len(ids), "not enough pages for the test"
        tables.append(ids[i:i + n])
        i += n
    return tables
