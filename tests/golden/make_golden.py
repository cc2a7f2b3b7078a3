"""Generate tests/golden/*.npz by running the UPSTREAM modules on CPU.

Usage:  python tests/golden/make_golden.py            (needs an upstream checkout;
        see oracle/ref_shim.py for where it is looked up)

For every case of oracle/cases.py (parity grid, config 0, small GeGLU cases, the Gemma-size layer shape)
this builds the upstream MoeficationMoE + MoeficationRouter, loads the seeded
tensors into it, runs forward in 'dynk_max' mode with the experts in 'masked'
(dense) and 'naive' (sparse loop) modes, and stores what the upstream code
returned: router scores, the 0/1 routing tensor (bit-packed) and the output
(all rows for small cases, an evenly strided row subset for large ones),
together with digests of the seeded inputs so that a drifting random generator
is detected instead of being reported as a parity failure.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import cases as C                      # noqa: E402
from oracle import d2d_oracle as O                 # noqa: E402
from oracle.ref_shim import load_reference         # noqa: E402

ACT = {"relu": torch.nn.ReLU, "gelu": torch.nn.GELU, "tanh": torch.nn.Tanh,
       "leaky_relu": torch.nn.LeakyReLU}
MAX_OUT_ELEMS = 32768


class _FixedScores(torch.nn.Module):
    """Router stand-in returning a given score tensor (the mechanism upstream's own
    override hook uses, architectures/moe/moefication.py:331-339)."""

    def __init__(self, s):
        super().__init__()
        self.s = s

    def forward(self, x):
        return self.s


def glu_case() -> C.LayerCase:
    return C.LayerCase("glu_small", 2, 17, 64, 32, 8, tau=0.4, act="gelu", glu=True,
                       norm="rms")


def glu_case_bf16() -> C.LayerCase:
    return C.LayerCase("glu_small_bf16", 2, 65, 128, 64, 16, tau=0.4, act="gelu", glu=True,
                       norm="rms", dtype="bf16")


def gemma_shape_cases() -> list[C.LayerCase]:
    """The Gemma-2B-size layer's own shape (d 2048, 128 experts x 128, router 2048->256->128,
    GeGLU with erf GELU, RMS-normed input, bf16) at a ragged token count: the two-half router,
    16 output chunks per tile, E = 128 with H = 128.  The second case keeps more experts per
    token, so that some experts own more than one 128-row tile."""
    return [
        C.LayerCase("gemma_shape", 3, 701, 2048, 128, 128, R=256, tau=0.1, dtype="bf16",
                    act="gelu", glu=True, norm="rms", seed=4),
        C.LayerCase("gemma_shape_k", 3, 701, 2048, 128, 128, R=256, tau=0.3, dtype="bf16",
                    act="gelu", glu=True, norm="rms", seed=5),
    ]


# cases whose saved output rows are capped at this many (others: MAX_OUT_ELEMS elements)
ROWS_SAVED = {"gemma_shape": 96, "gemma_shape_k": 96}
# upstream's dense gated experts materialise [E, N, d]: such cases run in token chunks
TOKEN_CHUNK = {"gemma_shape": 192, "gemma_shape_k": 192}


def attention_projection_case() -> C.LayerCase:
    """A MoE-fied attention projection of ViT-B/16 (architectures/moe/dsti.py:88-138 with
    flops_factor 1: attention_dim = round((d*d + d) / (2d + 1)) = 384, split into 12 experts of
    32; architectures/moe/moe_models.py:13-52 calls it like any MoE layer): GELU, last bias,
    residual connection, bf16."""
    return C.LayerCase("attn_proj_residual", 2, 197, 768, 32, 12, tau=0.2, dtype="bf16",
                       act="gelu", zero_last_bias=False, residual=True, seed=7)


def all_cases():
    return C.parity_grid() + [C.config0(), glu_case(), glu_case_bf16()] + gemma_shape_cases() + \
        [attention_projection_case()]


def build_reference_module(ref, c: C.LayerCase, t: dict):
    dt = c.torch_dtype
    if c.glu:
        moe = ref.MoeficationMoE(c.name, c.d, c.E, False, c.H, ACT[c.act],
                                 experts_class="execute_all", add_intermediate_gating=True)
        sd = {"experts.layers.0.w": t["w1"], "experts.layers.1.w": t["w2"],
              "experts.layers.2.w": t["w_up"]}
    else:
        moe = ref.MoeficationMoE(c.name, c.d, c.E, True, c.H, ACT[c.act],
                                 experts_class="custom_kernel",
                                 add_residual_connection=c.residual)
        sd = {"experts.w1": t["w1"], "experts.b1": t["b1"], "experts.w2": t["w2"],
              "last_bias": t["last_bias"]}
    moe.router = ref.MoeficationRouter(c.d, c.E, width=c.R, depth=2, bias=False,
                                       activation="relu", output_activation="abs")
    sd["router.layers.0.weight"] = t["wa"]
    sd["router.layers.2.weight"] = t["wb"]
    moe = moe.to(dt)
    moe.load_state_dict(sd, strict=True)
    if c.score_override:
        moe.router = _FixedScores(t["scores"])
    moe.forward_mode = "dynk_max"
    moe.tau = c.tau
    moe.eval()
    return moe


@torch.no_grad()
def run_case(ref, c: C.LayerCase) -> dict:
    t = C.make_tensors(c)
    moe = build_reference_module(ref, c, t)
    scores = moe.router(t["x"])
    rec = {"dtype": c.dtype, "N": c.N, "d": c.d, "E": c.E,
           "dg_x": C.digest(t["x"]), "dg_w1": C.digest(t["w1"]), "dg_wa": C.digest(t["wa"]),
           "scores": scores.float().reshape(c.N, c.E).numpy()}
    outs = {}
    modes = ["execute_all"] if c.glu else ["masked", "naive"]
    chunk = TOKEN_CHUNK.get(c.name)
    for mode in modes:
        if not c.glu:
            moe.experts.forward_mode = mode
        if chunk is None:
            out, gd = moe(t["x"])
            rt = gd[c.name][0]
        else:
            # tokens are independent: the module run on slices of the token axis gives the
            # rows of a run on the whole batch
            # (the scores are those of the whole-batch router run above, fed back through the
            # fixed-score router, so that no slice depends on how a CPU GEMM blocks its rows)
            xs = t["x"].reshape(1, c.N, c.d)
            ss = scores.reshape(1, c.N, c.E)
            router = moe.router
            o_parts, r_parts = [], []
            for lo in range(0, c.N, chunk):
                moe.router = _FixedScores(ss[:, lo:lo + chunk])
                o, gd = moe(xs[:, lo:lo + chunk])
                o_parts.append(o)
                r_parts.append(gd[c.name][0])
            moe.router = router
            out = torch.cat(o_parts, 1).reshape(c.B, c.S, c.d)
            rt = torch.cat(r_parts, 1).reshape(c.B, c.S, c.E)
        assert rt.dtype == scores.dtype and rt.shape == (c.B, c.S, c.E)
        outs[mode] = out.float().reshape(c.N, c.d)
        rec["mask_bits"] = O.pack_mask(rt.reshape(c.N, c.E) > 0)
    if c.glu:
        # the sparse CPU form of the same layer: experts_class='module' (one GLUExpert of
        # three nn.Linear per expert), fed the same parameters
        sp = ref.MoeficationMoE(c.name, c.d, c.E, False, c.H, ACT[c.act], experts_class="module",
                                add_intermediate_gating=True).to(c.torch_dtype)
        for e in range(c.E):
            sp.experts.e[e].gate.weight.copy_(t["w1"][e].t())
            sp.experts.e[e].up_scale.weight.copy_(t["w_up"][e].t())
            sp.experts.e[e].down_scale.weight.copy_(t["w2"][e].t())
        sp.router = _FixedScores(scores)
        sp.forward_mode, sp.tau = "dynk_max", c.tau
        sp.eval()
        out, gd = sp(t["x"])
        assert torch.equal(gd[c.name][0].reshape(c.N, c.E) > 0,
                           O.unpack_mask(rec["mask_bits"], c.E))
        outs["module"] = out.float().reshape(c.N, c.d)
    if c.name in ROWS_SAVED:
        stride = max(1, c.N // ROWS_SAVED[c.name])
    else:
        stride = max(1, -(-c.N * c.d // MAX_OUT_ELEMS))
    rows = np.arange(0, c.N, stride, dtype=np.int64)
    rec["rows"] = rows
    for mode, o in outs.items():
        rec[f"out_{mode}"] = o[rows].numpy()
        rec[f"sum_{mode}"] = np.float64(o.double().sum().item())
    return rec


def main():
    ref = load_reference()
    if ref is None:
        raise SystemExit("no upstream checkout found (set D2DMOE_REFERENCE_ROOT)")
    torch.set_num_threads(8)
    outdir = Path(__file__).resolve().parent
    only = set(sys.argv[1:])          # optional: names of the cases to (re)generate
    for c in all_cases():
        if only and c.name not in only:
            continue
        rec = run_case(ref, c)
        np.savez_compressed(outdir / f"{c.name}.npz", **rec)
        k = O.unpack_mask(rec["mask_bits"], c.E).sum().item() / c.N
        print(f"{c.name:24s} N={c.N:5d} d={c.d:4d} E={c.E:3d} {c.dtype} mean_k={k:.2f} "
              f"rows_saved={len(rec['rows'])}")


if __name__ == "__main__":
    main()
