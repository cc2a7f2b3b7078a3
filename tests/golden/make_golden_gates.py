"""Generate tests/golden/gates.npz by running the UPSTREAM gate on CPU.

Usage:  python tests/golden/make_golden_gates.py      (needs an upstream checkout;
        see oracle/ref_shim.py for where it is looked up)

For a few cases of the parity grid this feeds the router scores stored in the case's
fixture (what the upstream router returned, in the case's dtype) back into the upstream
MoeficationMoE through a fixed-score router and records the routing tensor that
MoeficationMoE.gate returns in 'topk' mode (k = 1, 3, E) and in 'dynk' mode
(tau = 0.3, 0.6, 0.9, 1.5), bit-packed.  Keys: "<case>/topk/<k>", "<case>/dynk/<tau>".
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

from oracle import d2d_oracle as O                 # noqa: E402
from oracle.ref_shim import load_reference         # noqa: E402
import make_golden as MG                           # noqa: E402

CASES = ["config0_vit_layer_fp32", "n197_vit_bf16", "e96_h32_bert", "n257_e128", "n33_e33",
         "lognormal_gpt"]
TAUS = [0.3, 0.6, 0.9, 1.5]


def ks(E):
    return sorted({1, min(3, E), E})


@torch.no_grad()
def main():
    ref = load_reference()
    if ref is None:
        raise SystemExit("no upstream checkout found (set D2DMOE_REFERENCE_ROOT)")
    here = Path(__file__).resolve().parent
    by_name = {c.name: c for c in MG.all_cases()}
    rec = {}
    for name in CASES:
        c = by_name[name]
        g = np.load(here / f"{name}.npz")
        s = torch.from_numpy(g["scores"]).to(c.torch_dtype).reshape(c.B, c.S, c.E)
        moe = ref.MoeficationMoE(c.name, c.d, c.E, True, c.H, torch.nn.ReLU,
                                 experts_class="custom_kernel")
        moe.router = MG._FixedScores(s)
        x = torch.zeros(c.B, c.S, c.d, dtype=c.torch_dtype)
        for k in ks(c.E):
            moe.forward_mode, moe.k = "topk", k
            rt = moe.gate(x)
            assert rt.dtype == s.dtype
            rec[f"{name}/topk/{k}"] = O.pack_mask(rt.reshape(c.N, c.E) > 0)
        for tau in TAUS:
            moe.forward_mode, moe.tau = "dynk", tau
            rt = moe.gate(x)
            rec[f"{name}/dynk/{tau}"] = O.pack_mask(rt.reshape(c.N, c.E) > 0)
            print(name, "dynk", tau, "mean k", float((rt > 0).sum()) / c.N)
    np.savez_compressed(here / "gates.npz", **rec)
    print("wrote", len(rec), "masks")


if __name__ == "__main__":
    main()
