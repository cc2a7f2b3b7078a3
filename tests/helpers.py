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


# -- topk / dynk rules --------------------------------------------------------------
def gate_fixture_items():
    """(case, rule, parameter, upstream mask [N,E] bool, upstream scores in the case dtype)
    for every mask of tests/golden/gates.npz."""
    gz = np.load(GOLDEN / "gates.npz")
    by_name = {c.name: c for c in all_cases()}
    out = []
    for key in gz.files:
        name, rule, par = key.split("/")
        c = by_name[name]
        out.append((c, rule, float(par) if rule == "dynk" else int(par), gz[key]))
    return out


def gate_fixture_ids():
    return [k for k in np.load(GOLDEN / "gates.npz").files]


def rule_tie_tokens(scores, rule, par, window, ref_mask):
    """Tokens whose decision sits inside the tie window.  top-k: the k-th and (k+1)-th largest
    scores closer than window*max.  dynk: a cumulative share within `window` of tau, or the
    boundary of the upstream selection falling inside a group of (nearly) equal shares —
    which member of such a group is taken depends on the order an unstable sort leaves."""
    E = scores.shape[-1]
    if rule == "topk":
        if par >= E:
            return torch.zeros(scores.shape[0], dtype=torch.bool)
        srt = torch.sort(scores.double(), dim=-1, descending=True).values
        return (srt[:, par - 1] - srt[:, par]).abs() <= window * srt[:, 0].abs()
    sh = (scores / scores.sum(-1, keepdim=True)).double()       # shares in the tensor dtype
    srt = torch.sort(sh, dim=-1, descending=True).values
    # bf16 shares add up exactly in fp32, so only fp32 tensors have a summation-order window
    near = ((torch.cumsum(srt, dim=-1) - par).abs() <= window).any(-1)
    if scores.dtype == torch.bfloat16:
        near = torch.zeros_like(near)
    n = ref_mask.sum(-1).clamp(max=E - 1)                        # first rank left out upstream
    idx = torch.arange(scores.shape[0])
    group = (srt[idx, n - 1] - srt[idx, n]).abs() <= window * srt[:, 0]
    return near | (group & (ref_mask.sum(-1) < E))
