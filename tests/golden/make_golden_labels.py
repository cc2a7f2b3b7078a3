"""Generate tests/golden/labels.npz: router-training labels captured from the upstream layer.

Usage:  python tests/golden/make_golden_labels.py     (needs an upstream checkout;
        see oracle/ref_shim.py for where it is looked up)

Each case runs the upstream MoeficationMoE in forward mode 'all' on CPU with the upstream
norm-capturing forward hooks (utils.py:353-369 add_save_output_norm_hook) on the modules router
training names (methods/dynamic_sparsification/train_routers.py:49-71): for CustomKernelExperts
its two extraction stubs, for ExecuteAllExperts layers[0] / layers[1].  Stored per case: the
[E, N] norms for layer in {intermediate, output} and ord in {1, 2}, and the layer output rows.
Keys: "<case>/<field>".
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

from oracle import cases as C                      # noqa: E402
from oracle.ref_shim import load_reference         # noqa: E402
import make_golden as MG                           # noqa: E402

ORDS = (1, 2)


def label_cases():
    return [
        C.LayerCase("labels_bf16", 2, 77, 256, 64, 8, tau=0.5, dtype="bf16", seed=31),
        C.LayerCase("labels_fp32", 3, 17, 64, 32, 8, tau=0.5, act="gelu", seed=32),
        C.LayerCase("labels_glu_bf16", 2, 65, 128, 64, 16, tau=0.5, dtype="bf16", act="gelu",
                    glu=True, seed=33),
        C.LayerCase("labels_odd_fp32", 1, 45, 40, 24, 5, tau=0.5, act="tanh", seed=34),
    ]


@torch.no_grad()
def main():
    ref = load_reference()
    if ref is None:
        raise SystemExit("no upstream checkout found (set D2DMOE_REFERENCE_ROOT)")
    up_utils = importlib.import_module("utils")
    rec = {}
    for c in label_cases():
        t = C.make_tensors(c)
        moe = MG.build_reference_module(ref, c, t)
        moe.forward_mode = "all"
        if c.glu:
            names = {"intermediate": "experts.layers.0", "output": "experts.layers.1"}
        else:
            moe.experts.forward_mode = "masked"
            names = {"intermediate": "experts.intermediate_activation_extraction_stub",
                     "output": "experts.output_activation_extraction_stub"}
        for ordv in ORDS:
            saved, handles = up_utils.add_save_output_norm_hook(moe, list(names.values()),
                                                                ord=ordv, dim=-1)
            out, gd = moe(t["x"])
            up_utils.remove_hooks(handles)
            assert bool((gd[c.name][0] == 1).all())
            for layer, nm in names.items():
                v = saved[nm]
                assert v.shape == (c.E, c.N), v.shape
                rec[f"{c.name}/{layer}_ord{ordv}"] = v.float().numpy()
        rec[f"{c.name}/out"] = out.float().reshape(c.N, c.d).numpy()
        rec[f"{c.name}/dg_x"] = C.digest(t["x"])
        print(f"{c.name:18s} N={c.N} d={c.d} H={c.H} E={c.E} {c.dtype}")
    np.savez_compressed(Path(__file__).resolve().parent / "labels.npz", **rec)


if __name__ == "__main__":
    main()
