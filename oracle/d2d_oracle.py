"""CPU restatement of the D2DMoE MoE-FFN inference layer.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA path: only tests, the smoke check and
the benchmark's CPU-baseline leg import it.  Nothing in the product package
imports it, and the product path fails loudly without its CUDA library.

Every function restates, in explicit arithmetic, one piece of the upstream
layer and cites the upstream file:line it follows.  Matrix products are taken
in fp32 (or fp64 for the "exact" variants) over the dtype-rounded operands and
rounded to the tensor dtype at exactly the points where the upstream code
materialises a tensor, so the bf16 behaviour is stated here rather than
inherited from a library kernel.

Parity pinning: the upstream repository holds no golden vectors or
known-answer tests for this path (its only check prints a max-abs error between
two modes of the same module on unseeded inputs,
scripts/test_moe_implementations.py:36-85).  This oracle is therefore pinned
against OUTPUTS OF THE UPSTREAM MODULES THEMSELVES, run on CPU on seeded inputs
by tests/golden/make_golden.py and committed under tests/golden/.
"""
from __future__ import annotations

import math

import numpy as np
import torch

ACTS = ("relu", "gelu", "tanh", "leaky_relu", "gelu_tanh")


def _round(t: torch.Tensor, dtype) -> torch.Tensor:
    """Materialise an fp32 intermediate in the tensor dtype and come back to fp32."""
    return t.to(dtype).to(torch.float32)


def activation(h: torch.Tensor, act: str) -> torch.Tensor:
    """Expert activations (architectures/moe/moe_layers.py:11-16; utils.py:730-756).

    relu = max(x,0); gelu = exact erf form; tanh; leaky_relu slope 0.01.
    """
    if act == "relu":
        return torch.clamp_min(h, 0.0)
    if act == "gelu":
        return h * 0.5 * (1.0 + torch.erf(h * (1.0 / math.sqrt(2.0))))
    if act == "gelu_tanh":
        k = math.sqrt(2.0 / math.pi)
        return 0.5 * h * (1.0 + torch.tanh(k * (h + 0.044715 * h * h * h)))
    if act == "tanh":
        return torch.tanh(h)
    if act == "leaky_relu":
        return torch.where(h >= 0, h, 0.01 * h)
    raise ValueError(act)


# --------------------------------------------------------------------------
# router + gate
# --------------------------------------------------------------------------
def router_scores(x2d: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor) -> torch.Tensor:
    """scores = |relu(x Wa^T) Wb^T|, no biases (architectures/moe/moefication.py:313-330
    with the D2DMoE settings depth 2, relu, abs: scripts/d2dmoe_vit_wallclock.py:317-325).

    Each Linear output is one tensor in the upstream code, hence one rounding
    to the tensor dtype after an fp32 accumulation.  Returns scores in x's dtype.
    """
    dt = x2d.dtype
    h = x2d.float() @ wa.float().t()
    h = _round(h, dt)
    h = torch.clamp_min(h, 0.0)
    s = h @ wb.float().t()
    s = _round(s, dt)
    return s.abs().to(dt)


def threshold_multiplier(tau: float) -> float:
    """(1.0 - tau) in Python double, then narrowed to fp32 by the tensor multiply
    (architectures/moe/moefication.py:83)."""
    return float(np.float32(1.0 - float(tau)))


def dynk_max_mask(scores: torch.Tensor, tau: float) -> torch.Tensor:
    """Dynamic-k rule (architectures/moe/moefication.py:80-85): keep expert e iff
    score_e >= max_e(score) * (1.0 - tau), threshold materialised in the score dtype.

    Consequences restated: the arg-max expert is always kept; an all-zero row keeps
    every expert; NaN scores are never kept.  Returns bool [..., E].
    """
    dt = scores.dtype
    s = scores.float()
    mx = s.max(dim=-1, keepdim=True).values
    thr = (mx * torch.tensor(threshold_multiplier(tau), dtype=torch.float32)).to(dt).float()
    return s >= thr


def near_threshold(scores: torch.Tensor, tau: float, rel_window: float) -> torch.Tensor:
    """Entries whose score lies within rel_window*row_max of the threshold: these
    token-expert pairs are excluded from bit-exact mask comparison and counted."""
    s = scores.float()
    mx = s.max(dim=-1, keepdim=True).values
    thr = mx * threshold_multiplier(tau)
    return (s - thr).abs() <= rel_window * mx


def gate_topk(scores: torch.Tensor, k: int) -> torch.Tensor:
    """'topk' gate (architectures/moe/moefication.py:59-63)."""
    top = torch.topk(scores.float(), k=k, dim=-1)[1]
    m = torch.zeros(scores.shape, dtype=torch.bool)
    m.scatter_(-1, top, True)
    return m


def gate_dynk_cumulative(scores: torch.Tensor, tau: float) -> torch.Tensor:
    """'dynk' gate (architectures/moe/moefication.py:64-79): smallest prefix of the
    experts, sorted by descending share, whose cumulative share reaches tau; at
    least one expert."""
    dt = scores.dtype
    tot = scores.sum(dim=-1, keepdim=True)
    shares = scores / tot
    srt, idx = torch.sort(shares, dim=-1, descending=True)
    cum = torch.cumsum(srt, dim=-1)
    m = cum < tau
    m = m.roll(shifts=1, dims=-1)
    m[..., 0] = True
    del dt
    return m.gather(dim=-1, index=idx.argsort(dim=-1))


def pack_mask(mask: torch.Tensor) -> np.ndarray:
    """bool [N, E] -> uint32 [N, ceil(E/32)], bit (e % 32) of word (e // 32)."""
    m = mask.reshape(-1, mask.shape[-1]).numpy().astype(np.uint32)
    n, e = m.shape
    w = (e + 31) // 32
    out = np.zeros((n, w), dtype=np.uint32)
    for j in range(e):
        out[:, j // 32] |= m[:, j] << np.uint32(j % 32)
    return out


def unpack_mask(bits: np.ndarray, E: int) -> torch.Tensor:
    n = bits.shape[0]
    out = np.zeros((n, E), dtype=bool)
    for j in range(E):
        out[:, j] = (bits[:, j // 32] >> np.uint32(j % 32)) & 1
    return torch.from_numpy(out)


# --------------------------------------------------------------------------
# per-expert token lists
# --------------------------------------------------------------------------
def expert_token_lists(mask: torch.Tensor):
    """Per-expert token lists and offsets.

    Upstream (architectures/moe/moe_layers.py:241-249) takes, for column e of the
    0/1 routing tensor, the first bincount[e] rows of a descending argsort along
    tokens: the SET of tokens with a 1 in column e, in an order the sort does not
    define.  Restated as ascending token index (torch.nonzero order).
    Returns (offsets int32 [E+1], token_idx int32 [sum c_e]).
    """
    m = mask.reshape(-1, mask.shape[-1]).numpy()
    n, e = m.shape
    counts = m.sum(axis=0).astype(np.int64)
    offsets = np.zeros(e + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    idx = np.concatenate([np.nonzero(m[:, j])[0] for j in range(e)]) if e else np.zeros(0)
    return offsets, idx.astype(np.int32)


# --------------------------------------------------------------------------
# experts
# --------------------------------------------------------------------------
def experts_ffn_naive(x2d, mask, w1, b1, w2, act="relu") -> torch.Tensor:
    """Sparse per-expert loop with the upstream rounding points
    (architectures/moe/moe_layers.py:200-211): for e in 0..E-1:
    rows = tokens with mask[:, e]; h = act(round(x W1[e]) + b1[e]) (bias add and
    activation each materialise a tensor); y = round(h W2[e]); out[rows] += y in the
    tensor dtype."""
    dt = x2d.dtype
    out = torch.zeros(x2d.shape, dtype=torch.float32)
    xf = x2d.float()
    for e in range(w1.shape[0]):
        rows = mask[:, e].nonzero().flatten()
        if rows.numel() == 0:
            continue
        h = _round(xf[rows] @ w1[e].float(), dt)
        h = _round(h + b1[e].float(), dt)
        h = _round(activation(h, act), dt)
        y = _round(h @ w2[e].float(), dt)
        out[rows] = _round(out[rows] + y, dt)
    return out.to(dt)


def experts_ffn_exact(x2d, mask, w1, b1, w2, act="relu", w_up=None) -> torch.Tensor:
    """fp64 evaluation of the same sum over the dtype-rounded operands, no
    intermediate rounding: the truth both the upstream bf16 result and the CUDA
    result are measured against.  GLU form when w_up is given
    (architectures/moe/moe_layers.py:91-96: down(act(gate(x)) * up(x)))."""
    out = torch.zeros(x2d.shape, dtype=torch.float64)
    xd = x2d.double()
    for e in range(w1.shape[0]):
        rows = mask[:, e].nonzero().flatten()
        if rows.numel() == 0:
            continue
        h = xd[rows] @ w1[e].double()
        if b1 is not None:
            h = h + b1[e].double()
        h = activation(h, act)
        if w_up is not None:
            h = h * (xd[rows] @ w_up[e].double())
        out[rows] += h @ w2[e].double()
    return out


def experts_ffn_dense(x2d, mask, w1, b1, w2, act="relu") -> torch.Tensor:
    """Dense all-experts form (architectures/moe/moe_layers.py:116-133,193-198):
    y[e] = act(x W1[e] + b1[e]) W2[e] for every expert, then sum_e y[e]*mask[:, e]."""
    dt = x2d.dtype
    xf = x2d.float()
    h = _round(torch.einsum("ni,eio->eno", xf, w1.float()), dt)
    h = _round(h + b1.float().unsqueeze(-2), dt)
    h = _round(activation(h, act), dt)
    y = _round(torch.einsum("eni,eio->eno", h, w2.float()), dt)
    return torch.einsum("end,ne->nd", y, mask.float()).to(dt)


def moe_forward(x, p: dict, tau: float, act="relu", residual=False, scores=None,
                exact=False):
    """Whole layer (architectures/moe/moefication.py:90-101): gate -> flatten ->
    experts -> + last_bias (once per token) -> (+ x) -> reshape.

    p: w1, b1, w2, wa, wb, last_bias (optional), w_up (optional).
    Returns (out [B,S,d], mask bool [B,S,E], scores [B,S,E]).
    """
    dt = x.dtype
    x2d = x.reshape(-1, x.shape[-1])
    if scores is None:
        scores = router_scores(x2d, p["wa"], p["wb"])
    s2d = scores.reshape(x2d.shape[0], -1)
    mask = dynk_max_mask(s2d, tau)
    if exact or p.get("w_up") is not None:
        out = experts_ffn_exact(x2d, mask, p["w1"], p.get("b1"), p["w2"], act, p.get("w_up"))
        if p.get("last_bias") is not None:
            out = out + p["last_bias"].double()
        if residual:
            out = out + x2d.double()
    else:
        out = experts_ffn_naive(x2d, mask, p["w1"], p["b1"], p["w2"], act)
        if p.get("last_bias") is not None:
            out = (out.float() + p["last_bias"].float()).to(dt)
        if residual:
            out = (out.float() + x2d.float()).to(dt)
    E = s2d.shape[-1]
    return out.reshape(x.shape), mask.reshape(*x.shape[:-1], E), s2d.reshape(*x.shape[:-1], E)


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / max|b| over the tensor: the error form the tolerances are stated in."""
    a = a.double()
    b = b.double()
    den = b.abs().max().item()
    return (a - b).abs().max().item() / (den if den > 0 else 1.0)


# --------------------------------------------------------------------------
# timed CPU path (benchmark baseline): the upstream CPU mode, restated
# --------------------------------------------------------------------------
@torch.inference_mode()
def cpu_layer_forward_naive(x, p: dict, tau: float, act="relu", scores=None):
    """The upstream CPU performance path in library calls, as upstream runs it:
    router Linear/ReLU/Linear/abs (moefication.py:328-330), dynk_max gate
    (:80-85), then the 'naive' expert loop (moe_layers.py:200-211) with boolean-mask
    gather, two matmuls and a masked += per expert, then + last_bias
    (moefication.py:96-97).  Uses every host thread torch is configured for."""
    F = torch.nn.functional
    x2d = x.reshape(-1, x.shape[-1])
    if scores is None:
        s = F.linear(torch.relu(F.linear(x2d, p["wa"])), p["wb"]).abs()
    else:
        s = scores.reshape(x2d.shape[0], -1)
    mx = s.max(dim=-1, keepdim=True).values
    thr = mx * (1.0 - tau)
    rt = torch.zeros_like(s)
    rt[s >= thr] = 1.0
    out = torch.zeros_like(x2d)
    fn = {"relu": torch.relu, "gelu": F.gelu, "tanh": torch.tanh,
          "leaky_relu": F.leaky_relu}[act]
    for e in range(p["w1"].shape[0]):
        m = rt[:, e] > 0.0
        xe = x2d[m]
        xe = fn(xe @ p["w1"][e] + p["b1"][e])
        xe = xe @ p["w2"][e]
        out[m] += xe
    if p.get("last_bias") is not None:
        out = out + p["last_bias"]
    return out.view(x.shape), rt


def glu_module_weights(w_gate, w_up, w_down):
    """Per-expert ``nn.Linear`` weights of the upstream 'module' experts, from the stacked
    GLU parameters: gate.weight = layers.0.w[e]^T, up_scale.weight = layers.2.w[e]^T,
    down_scale.weight = layers.1.w[e]^T (nn.Linear stores [out, in];
    architectures/moe/moe_layers.py:104-110).  Made once, like a module's parameters."""
    tr = lambda w: [w[e].t().contiguous() for e in range(w.shape[0])]       # noqa: E731
    return {"gate": tr(w_gate), "up": tr(w_up), "down": tr(w_down)}


@torch.inference_mode()
def experts_glu_module(x2d, rt, lin: dict, act="gelu"):
    """ModuleBatchedExperts.forward with GLUExpert experts, no biases
    (architectures/moe/moe_layers.py:104-113,310-324): for every expert i the rows with a
    non-zero routing entry are gathered, down(act(gate(x)) * up(x)) is evaluated with three
    nn.Linear calls, multiplied by the routing entries and added to the output rows."""
    F = torch.nn.functional
    fn = {"relu": torch.relu, "gelu": F.gelu, "tanh": torch.tanh, "leaky_relu": F.leaky_relu,
          "gelu_tanh": lambda v: F.gelu(v, approximate="tanh")}[act]
    out = torch.zeros_like(x2d)
    for i in range(len(lin["gate"])):
        col = rt[:, i]
        m = col != 0.0
        sc = col[m].unsqueeze(1)
        xe = x2d[m]
        y = F.linear(fn(F.linear(xe, lin["gate"][i])) * F.linear(xe, lin["up"][i]), lin["down"][i])
        out[m] += y * sc
    return out


@torch.inference_mode()
def cpu_layer_forward_module_glu(x, p: dict, tau: float, act="gelu"):
    """The upstream CPU path of a gated (GeGLU) layer: router and dynk_max gate as in
    cpu_layer_forward_naive (moefication.py:328-330, :80-85), experts_class='module' with
    add_intermediate_gating (moefication.py:39-45 -> ModuleBatchedExperts + GLUExpert), no
    last_bias (bias=False).  p: wa, wb and ``lin`` from glu_module_weights."""
    F = torch.nn.functional
    x2d = x.reshape(-1, x.shape[-1])
    s = F.linear(torch.relu(F.linear(x2d, p["wa"])), p["wb"]).abs()
    mx = s.max(dim=-1, keepdim=True).values
    thr = mx * (1.0 - tau)
    rt = torch.zeros_like(s)
    rt[s >= thr] = 1.0
    out = experts_glu_module(x2d, rt, p["lin"], act)
    return out.view(x.shape), rt


# --------------------------------------------------------------------------
# pre-norm in front of the layer (block-level callers)
# --------------------------------------------------------------------------
def prenorm(x: torch.Tensor, gamma: torch.Tensor, beta, eps: float, kind: str,
            gamma_offset: float = 0.0) -> torch.Tensor:
    """The normalisation an upstream block applies before its MoE-FFN layer
    (architectures/moe/moe_models.py:69 ``self.ln_2(x)`` = nn.LayerNorm; :148-151 Gemma's
    RMSNorm, transformers GemmaRMSNorm: ``x.float() * rsqrt(mean(x^2) + eps) * (1 + w)``):
    statistics and affine map in fp32 over the dtype-rounded input, one rounding to the tensor
    dtype.  kind: "layer" | "rms"."""
    dt = x.dtype
    xf = x.float()
    if kind == "layer":
        mean = xf.mean(-1, keepdim=True)
        var = ((xf - mean) ** 2).mean(-1, keepdim=True)
        y = (xf - mean) * torch.rsqrt(var + eps) * gamma.float()
        if beta is not None:
            y = y + beta.float()
    else:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (gamma_offset + gamma.float())
    return y.to(dt)


# --------------------------------------------------------------------------
# router-training labels: per-expert norms of what every expert computes
# --------------------------------------------------------------------------
def expert_activation_norms(x2d: torch.Tensor, w1, b1, w2, act: str, w_up=None, *,
                            layer: str = "output", ord=2) -> torch.Tensor:
    """[E, N] vector norms over the last dimension of every expert's activations on every
    token, as router training captures them with forward hooks while the layer runs in
    mode 'all' (methods/dynamic_sparsification/train_routers.py:49-71,77-82,204-209;
    utils.py:353-369 ``torch.linalg.vector_norm(output, ord=ord, dim=-1)``):
      layer "intermediate": act(x W1[e] + b1[e])      (moe_layers.py:116-124, :41-49 layers[0])
      layer "output":       (that, times x W_up[e] in the gated form) W2[e]
                                                      (moe_layers.py:127-133, :91-96 layers[1])
    Every product and sum is rounded to the tensor dtype like the upstream einsum chain."""
    dt = x2d.dtype
    xe = x2d.unsqueeze(0)
    h = torch.einsum("eni,eio->eno", xe, w1)
    if b1 is not None:
        h = h + b1.unsqueeze(-2)
    h = activation(h, act)
    if layer == "intermediate":
        return torch.linalg.vector_norm(h, ord=ord, dim=-1)
    if w_up is not None:
        h = h * torch.einsum("eni,eio->eno", xe, w_up)
    y = torch.einsum("eni,eio->eno", h, w2).to(dt)
    return torch.linalg.vector_norm(y, ord=ord, dim=-1)
