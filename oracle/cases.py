"""Seeded synthetic layer inputs shared by the golden generator, tests and bench.

TEST / MEASUREMENT INFRASTRUCTURE.  Every tensor is drawn on the CPU in fp32
from ``torch.Generator().manual_seed(seed)`` in the fixed order
x, W1, b1, W2, (W_up for GLU), router Wa, router Wb and only then cast, so the
oracle, the upstream modules and the CUDA path all see identical bits.

Parameter layouts follow the upstream modules:
  w1 [E, d, H], b1 [E, H], w2 [E, H, d]   (architectures/moe/moe_layers.py:157-159)
  last_bias [1, d]                         (architectures/moe/moefication.py:46-47)
  router.layers.0.weight [R, d], router.layers.2.weight [E, R]
                                           (architectures/moe/moefication.py:313-323)
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

import torch


@dataclass
class LayerCase:
    name: str
    B: int
    S: int
    d: int
    H: int
    E: int
    R: int = 128
    dtype: str = "fp32"           # "fp32" | "bf16"
    act: str = "relu"             # relu | gelu | tanh | leaky_relu
    tau: float = 0.1              # module attribute: keep iff s >= max*(1.0 - tau)
    seed: int = 0
    std: float = 0.02
    norm: str = "layer"           # "layer" | "rms" | "none": how x is normalised
    glu: bool = False
    zero_last_bias: bool = True
    residual: bool = False
    score_override: str | None = None   # "lognormal": scores = exp(1.5*randn)
    tensors: dict = field(default_factory=dict, repr=False)

    @property
    def N(self) -> int:
        return self.B * self.S

    @property
    def torch_dtype(self):
        return torch.float32 if self.dtype == "fp32" else torch.bfloat16


def make_tensors(c: LayerCase) -> dict:
    """Draw the layer's tensors (fp32 draw, then cast to the case dtype)."""
    g = torch.Generator().manual_seed(c.seed)
    x = torch.randn(c.B, c.S, c.d, generator=g)
    if c.norm == "layer":
        x = torch.nn.functional.layer_norm(x, (c.d,))
    elif c.norm == "rms":
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    t = {"x": x}
    t["w1"] = torch.randn(c.E, c.d, c.H, generator=g) * c.std
    t["b1"] = torch.randn(c.E, c.H, generator=g) * c.std
    t["w2"] = torch.randn(c.E, c.H, c.d, generator=g) * c.std
    if c.glu:
        t["w_up"] = torch.randn(c.E, c.d, c.H, generator=g) * c.std
    t["wa"] = torch.randn(c.R, c.d, generator=g) * c.std
    t["wb"] = torch.randn(c.E, c.R, generator=g) * c.std
    if c.zero_last_bias:
        t["last_bias"] = torch.zeros(1, c.d)
    else:
        t["last_bias"] = torch.randn(1, c.d, generator=g) * c.std
    if c.score_override == "lognormal":
        t["scores"] = torch.exp(1.5 * torch.randn(c.B, c.S, c.E, generator=g))
    dt = c.torch_dtype
    t = {k: v.to(dt).contiguous() for k, v in t.items()}
    c.tensors = t
    return t


def digest(t: torch.Tensor) -> str:
    """sha256 of the tensor's bytes: pins the seeded generator across machines."""
    v = t.contiguous().view(torch.uint8) if t.dtype != torch.bool else t.to(torch.uint8)
    return hashlib.sha256(v.numpy().tobytes()).hexdigest()[:16]


# The shape grid the upstream self-consistency test lists, its live values and
# the commented alternatives (scripts/test_moe_implementations.py:37-55), plus
# ragged token counts around warp/tile boundaries.
def parity_grid() -> list[LayerCase]:
    g = [
        LayerCase("ref_test_live", 5, 2, 64, 32, 4, tau=0.5),
        LayerCase("ref_test_live_bf16", 5, 2, 64, 32, 4, tau=0.5, dtype="bf16"),
        LayerCase("d1_h1", 5, 2, 1, 1, 4, tau=0.5, norm="none"),
        LayerCase("one_token", 1, 1, 64, 32, 4, tau=0.5),
        LayerCase("n31", 1, 31, 64, 32, 16, tau=0.3),
        LayerCase("n33_e33", 1, 33, 64, 16, 33, tau=0.3),
        LayerCase("n129_e64", 3, 43, 128, 64, 64, tau=0.2, dtype="bf16"),
        LayerCase("n197_vit", 1, 197, 768, 128, 24, tau=0.1),
        LayerCase("n197_vit_bf16", 1, 197, 768, 128, 24, tau=0.1, dtype="bf16"),
        LayerCase("n257_e128", 1, 257, 128, 32, 128, tau=0.1, dtype="bf16"),
        LayerCase("gelu_bias_res", 2, 65, 128, 64, 8, tau=0.4, act="gelu",
                  zero_last_bias=False, residual=True),
        LayerCase("tanh", 2, 17, 64, 32, 4, tau=0.4, act="tanh", zero_last_bias=False),
        LayerCase("leaky", 2, 17, 64, 32, 4, tau=0.4, act="leaky_relu", dtype="bf16"),
        LayerCase("tau1_all", 2, 19, 64, 32, 8, tau=1.0),
        LayerCase("tau0_argmax", 2, 19, 64, 32, 8, tau=0.0),
        LayerCase("e96_h32_bert", 2, 128, 768, 32, 96, tau=0.1, dtype="bf16"),
        LayerCase("lognormal_gpt", 1, 256, 768, 128, 24, tau=0.1, dtype="bf16",
                  score_override="lognormal"),
    ]
    return g


def config0() -> LayerCase:
    """Single ViT-B/16-sized layer in fp32: 8x197 tokens, E=24 x H=128, tau_cfg 0.9."""
    return LayerCase("config0_vit_layer_fp32", 8, 197, 768, 128, 24, tau=1.0 - 0.9, seed=0)


def vit_layer(batch: int, layer: int, tau_cfg: float, dtype: str = "bf16") -> LayerCase:
    """One of the 12 MoE-FFN layers of the ViT-B/16 config (197 tokens per image)."""
    return LayerCase(f"vit_b16_l{layer}", batch, 197, 768, 128, 24, tau=1.0 - tau_cfg,
                     dtype=dtype, seed=layer)


def gpt2_layer(batch: int, layer: int, tau_cfg: float) -> LayerCase:
    return LayerCase(f"gpt2_l{layer}", batch, 1024, 768, 128, 24, tau=1.0 - tau_cfg,
                     dtype="bf16", seed=layer, score_override="lognormal")


def bert_layer(batch: int, layer: int, tau_cfg: float = 0.9) -> LayerCase:
    return LayerCase(f"bert_l{layer}", batch, 128, 768, 32, 96, tau=1.0 - tau_cfg,
                     dtype="bf16", seed=layer)


def gemma_layer(batch: int, layer: int, tau_cfg: float = 0.9, seq: int = 2048) -> LayerCase:
    return LayerCase(f"gemma_l{layer}", batch, seq, 2048, 128, 128, R=256, tau=1.0 - tau_cfg,
                     dtype="bf16", act="gelu", seed=layer, norm="rms", glu=True)
