"""Shared test helpers: golden fixtures + seeded cases."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = ROOT / "tests" / "golden"
sys.path.insert(0, str(GOLDEN))

from oracle import cases as C          # noqa: E402
from oracle import d2d_oracle as O     # noqa: E402
import make_golden as MG               # noqa: E402

# Tolerances (max|a-b| / max|b| over the tensor), as the target states them.
TOL = {"fp32": 1e-5, "bf16": 2e-2}
# Near-threshold window for mask comparison: relative to the row max.
WINDOW = {"fp32": 1e-6, "bf16": 2.0 ** -7}


def all_cases():
    return MG.all_cases()


def case_ids():
    return [c.name for c in all_cases()]


def load_golden(c):
    g = dict(np.load(GOLDEN / f"{c.name}.npz"))
    t = C.make_tensors(c)
    assert C.digest(t["x"]) == str(g["dg_x"]), "seeded generator drifted (x)"
    assert C.digest(t["w1"]) == str(g["dg_w1"]), "seeded generator drifted (w1)"
    assert C.digest(t["wa"]) == str(g["dg_wa"]), "seeded generator drifted (wa)"
    return g, t


def golden_scores(g, c):
    return torch.from_numpy(g["scores"]).to(c.torch_dtype)


def golden_mask(g, c):
    return O.unpack_mask(g["mask_bits"], c.E)
