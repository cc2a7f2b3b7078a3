"""Layer micro-benchmark over the other model configurations of the layer path.

    python -m d2dmoe_b200.config_sweep [--layers L] [--reps K]

bench.py at the repository root measures the ViT-B/16 configuration only (it is the
contract line).  This script times the same fused layer call (``ops.moe_forward``) on
the remaining shapes with seeded synthetic tensors and prints one JSON line per
(configuration, tau): per-layer time, tokens/s, measured mean k and the fraction of the
roofline  max(selected-expert FLOPs / bf16 peak, algorithmic bytes / HBM bandwidth).

  vit_fp32  single layer, 8x197 tokens, d=768, 24 experts x 128, fp32 (general-shape kernels)
  gpt2      32x1024 tokens, d=768, 24 x 128, bf16, router scores overridden by a seeded
            log-normal(0, 1.5) tensor (rule from scores, no router GEMM)
  bert      512x128 tokens, d=768, 96 experts x 32, bf16
  gemma     64x2048 tokens, d=2048, 128 GeGLU experts x 128, router 2048->256->128, bf16
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import ops

ROOT = Path(__file__).resolve().parents[1]

CONFIGS = {
    "vit_fp32": dict(B=8, S=197, d=768, H=128, E=24, R=128, dtype=torch.float32, act="relu",
                     glu=False, scores=False, norm="layer", taus=[0.9], layers=1),
    "gpt2": dict(B=32, S=1024, d=768, H=128, E=24, R=128, dtype=torch.bfloat16, act="relu",
                 glu=False, scores=True, norm="layer", taus=[0.8, 0.9, 0.95], layers=12),
    "bert": dict(B=512, S=128, d=768, H=32, E=96, R=128, dtype=torch.bfloat16, act="relu",
                 glu=False, scores=False, norm="layer", taus=[0.9], layers=12),
    "gemma": dict(B=64, S=2048, d=2048, H=128, E=128, R=256, dtype=torch.bfloat16, act="gelu",
                  glu=True, scores=False, norm="rms", taus=[0.9], layers=18),
}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops_sustained"], "measured"
    return 6650.0, 1400.0, "fallback"


class Layer:
    def __init__(self, c, seed, dev):
        g = torch.Generator(device=dev).manual_seed(2000 + seed)
        rn = lambda *s: torch.randn(*s, generator=g, device=dev)          # noqa: E731
        d, H, E, R, dt = c["d"], c["H"], c["E"], c["R"], c["dtype"]
        x = rn(c["B"] * c["S"], d)
        if c["norm"] == "layer":
            x = torch.nn.functional.layer_norm(x, (d,))
        else:
            x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
        self.x = x.to(dt).contiguous()
        self.n = self.x.shape[0]
        cast = lambda t: (t * 0.02).to(dt).contiguous()                    # noqa: E731
        self.w1, self.w2 = cast(rn(E, d, H)), cast(rn(E, H, d))
        self.b1 = None if c["glu"] else cast(rn(E, H))
        self.w_up = cast(rn(E, d, H)) if c["glu"] else None
        self.wa, self.wb = cast(rn(R, d)), cast(rn(E, R))
        self.lb = None if c["glu"] else torch.zeros(d, dtype=dt, device=dev)
        self.scores = torch.exp(1.5 * rn(self.n, E)).to(dt).contiguous() if c["scores"] else None
        self.out = torch.empty_like(self.x)
        self.wsp = ops.Workspace.allocate(self.n, E, dev)
        self.rp = None if c["scores"] else ops.prepack_router(self.wa, self.wb)
        self.ep = ops.prepack_experts(self.w1, self.b1, self.w2, self.w_up)
        self.act = c["act"]

    def forward(self, tau):
        if self.scores is not None:
            ops.moe_forward(self.x, None, None, tau, self.w1, self.b1, self.w2, self.act, self.out,
                            self.wsp, w_up=self.w_up, scores=self.scores, last_bias=self.lb,
                            experts_packed=self.ep)
        else:
            ops.moe_forward(self.x, self.wa, self.wb, tau, self.w1, self.b1, self.w2, self.act,
                            self.out, self.wsp, w_up=self.w_up, last_bias=self.lb,
                            router_packed=self.rp, experts_packed=self.ep)


def run(name, c, max_layers, reps, dev):
    hbm, tf, src = peaks()
    nl = min(c["layers"], max_layers)
    layers = [Layer(c, i, dev) for i in range(nl)]
    s = 4 if c["dtype"] == torch.float32 else 2
    G = 2 if c["glu"] else 1
    d, H, E, R = c["d"], c["H"], c["E"], c["R"]
    for tau_cfg in c["taus"]:
        tau = 1.0 - tau_cfg
        for _ in range(3):
            for L in layers:
                L.forward(tau)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for L in layers:
                L.forward(tau)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * nl)
        for L in layers:
            L.wsp.check_status()
        n = layers[0].n
        sum_c = sum(int(L.wsp.offsets[E].item()) for L in layers) / nl
        flops = 2 * d * H * (G + 1) * sum_c
        w = s * ((G + 1) * E * d * H + (0 if c["glu"] else E * H + d) + d * R + R * E)
        byts = 2 * n * d * s + w
        t_hbm = byts / (hbm * 1e9)
        t_tc = flops / (tf * 1e12) if c["dtype"] != torch.float32 else 0.0
        t_roof = max(t_hbm, t_tc)
        print(json.dumps({
            "config": name, "tau_cfg": tau_cfg, "dtype": str(c["dtype"]).split(".")[-1],
            "tokens_per_layer": n, "layers_timed": nl, "us_per_layer": round(us, 2),
            "tokens_per_s": round(n / (us * 1e-6)), "mean_k": round(sum_c / n, 3),
            "roofline_us": round(t_roof * 1e6, 2), "bound": "tensor" if t_tc > t_hbm else "hbm",
            "roofline_frac": round(t_roof * 1e6 / us, 4), "peaks": src}), flush=True)
    del layers
    torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4, help="at most this many distinct layers")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    for name, c in CONFIGS.items():
        if a.only and name != a.only:
            continue
        run(name, c, a.layers, a.reps, dev)


if __name__ == "__main__":
    main()
