"""Generate tests/golden/blocks.npz: the FFN half of an upstream transformer block on CPU.

Usage:  python tests/golden/make_golden_blocks.py     (needs an upstream checkout;
        see oracle/ref_shim.py for where it is looked up)

For each case this runs what the upstream block forwards run after attention
(architectures/moe/moe_models.py:69-76 / :91-100 / :148-156):

    y = norm(x);  y, gating = mlp(y);  out = x + y

with ``norm`` = torch's nn.LayerNorm or transformers' GemmaRMSNorm carrying seeded affine
parameters and ``mlp`` = the upstream MoeficationMoE with its router, and stores the
normalised rows, the router scores, the routing tensor (bit-packed) and ``out`` for a strided
subset of rows.  Keys: "<case>/<field>".
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

from oracle import cases as C                      # noqa: E402
from oracle import d2d_oracle as O                 # noqa: E402
from oracle.ref_shim import load_reference         # noqa: E402
import make_golden as MG                           # noqa: E402


def block_cases():
    """(layer case, norm kind, eps).  x of these cases is NOT normalised (norm='none'): the
    block input is scaled and shifted so that the normalisation has something to do."""
    return [
        (C.LayerCase("block_vit_bf16", 2, 197, 768, 128, 24, tau=0.1, dtype="bf16", norm="none",
                     zero_last_bias=False, seed=21), "layer", 1e-6),
        (C.LayerCase("block_small_fp32", 3, 17, 64, 32, 8, tau=0.3, act="gelu", norm="none",
                     zero_last_bias=False, seed=22), "layer", 1e-5),
        (C.LayerCase("block_gemma_rms_bf16", 2, 65, 128, 64, 16, tau=0.4, dtype="bf16",
                     act="gelu", glu=True, norm="none", seed=23), "rms", 1e-6),
    ]


def block_tensors(c: C.LayerCase, kind: str):
    """Layer tensors plus the block input and the norm's affine parameters (seeded)."""
    t = C.make_tensors(c)
    g = torch.Generator().manual_seed(1000 + c.seed)
    dt = c.torch_dtype
    t["x"] = (t["x"].float() * 1.5 + 0.3).to(dt)
    if kind == "layer":
        t["gamma"] = (1.0 + 0.1 * torch.randn(c.d, generator=g)).to(dt)
        t["beta"] = (0.1 * torch.randn(c.d, generator=g)).to(dt)
    else:
        t["gamma"] = (0.1 * torch.randn(c.d, generator=g)).to(dt)      # applied as 1 + gamma
        t["beta"] = None
    return t


@torch.no_grad()
def main():
    ref = load_reference()
    if ref is None:
        raise SystemExit("no upstream checkout found (set D2DMOE_REFERENCE_ROOT)")
    from transformers.models.gemma.modeling_gemma import GemmaRMSNorm
    rec = {}
    for c, kind, eps in block_cases():
        t = block_tensors(c, kind)
        if kind == "layer":
            norm = torch.nn.LayerNorm(c.d, eps=eps).to(c.torch_dtype)
            norm.weight.copy_(t["gamma"])
            norm.bias.copy_(t["beta"])
        else:
            norm = GemmaRMSNorm(c.d, eps=eps).to(c.torch_dtype)
            norm.weight.copy_(t["gamma"])
        moe = MG.build_reference_module(ref, c, t)
        if not c.glu:
            moe.experts.forward_mode = "naive"
        x = t["x"]
        y = norm(x)
        out, gd = moe(y)
        out = x + out
        rows = np.arange(0, c.N, max(1, c.N // 48), dtype=np.int64)
        rec[f"{c.name}/rows"] = rows
        rec[f"{c.name}/xn"] = y.float().reshape(c.N, c.d)[rows].numpy()
        rec[f"{c.name}/scores"] = moe.router(y).float().reshape(c.N, c.E).numpy()
        rec[f"{c.name}/mask_bits"] = O.pack_mask(gd[c.name][0].reshape(c.N, c.E) > 0)
        rec[f"{c.name}/out"] = out.float().reshape(c.N, c.d)[rows].numpy()
        rec[f"{c.name}/dg_x"] = C.digest(x)
        k = O.unpack_mask(rec[f"{c.name}/mask_bits"], c.E).sum().item() / c.N
        print(f"{c.name:24s} N={c.N} d={c.d} E={c.E} {c.dtype} {kind} mean_k={k:.2f}")
    np.savez_compressed(Path(__file__).resolve().parent / "blocks.npz", **rec)


if __name__ == "__main__":
    main()
