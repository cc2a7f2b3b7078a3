"""Pre-norm + MoE-FFN + residual (the FFN half of an upstream block) against outputs of the
unmodified upstream modules (tests/golden/blocks.npz, made by make_golden_blocks.py)."""
import numpy as np
import pytest
import torch

from helpers import C, GOLDEN, O, TOL, WINDOW
import make_golden_blocks as MB

CASES = MB.block_cases()
IDS = [c.name for c, _, _ in CASES]


def load(c, kind):
    gz = np.load(GOLDEN / "blocks.npz")
    g = {k.split("/", 1)[1]: gz[k] for k in gz.files if k.startswith(c.name + "/")}
    t = MB.block_tensors(c, kind)
    assert C.digest(t["x"]) == str(g["dg_x"]), "seeded generator drifted (x)"
    return g, t


def exact_block(c, t, xn2d, mask):
    """x + last_bias + sum of the kept experts' outputs on the normalised rows, in float64."""
    e = O.experts_ffn_exact(xn2d, mask, t["w1"], None if c.glu else t["b1"], t["w2"], c.act,
                            t.get("w_up") if c.glu else None)
    if not c.glu and t.get("last_bias") is not None:
        e = e + t["last_bias"].double()
    return e + t["x"].reshape(c.N, c.d).double()


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_oracle_prenorm_and_block_match_upstream(case):
    c, kind, eps = case
    g, t = load(c, kind)
    rows = torch.from_numpy(g["rows"])
    x2d = t["x"].reshape(c.N, c.d)
    xn = O.prenorm(x2d, t["gamma"], t["beta"], eps, kind, 1.0 if kind == "rms" else 0.0)
    # one rounding to the tensor dtype on both sides: at most one ulp apart
    assert O.rel_err(xn.float()[rows], torch.from_numpy(g["xn"])) <= \
        (2e-6 if c.dtype == "fp32" else 2.0 ** -8)
    sg = torch.from_numpy(g["scores"]).to(c.torch_dtype)
    s = O.router_scores(xn, t["wa"], t["wb"])
    assert O.rel_err(s, sg) <= (1e-5 if c.dtype == "fp32" else 2.0 ** -6)
    m_up = O.unpack_mask(g["mask_bits"], c.E)
    assert np.array_equal(O.pack_mask(O.dynk_max_mask(sg, c.tau)), g["mask_bits"])
    out = exact_block(c, t, xn, m_up)
    assert O.rel_err(out[rows], torch.from_numpy(g["out"])) <= TOL[c.dtype]


def _module(c, t):
    import d2dmoe_b200 as D
    act = {"relu": torch.nn.ReLU, "gelu": torch.nn.GELU}[c.act]
    if c.glu:
        moe = D.MoeficationMoE(c.name, c.d, c.E, False, c.H, act, experts_class="execute_all",
                               add_intermediate_gating=True)
        sd = {"experts.layers.0.w": t["w1"], "experts.layers.1.w": t["w2"],
              "experts.layers.2.w": t["w_up"]}
    else:
        moe = D.MoeficationMoE(c.name, c.d, c.E, True, c.H, act, experts_class="custom_kernel")
        sd = {"experts.w1": t["w1"], "experts.b1": t["b1"], "experts.w2": t["w2"],
              "last_bias": t["last_bias"]}
    moe.router = D.MoeficationRouter(c.d, c.E, width=c.R, depth=2, bias=False, activation="relu",
                                     output_activation="abs")
    sd["router.layers.0.weight"], sd["router.layers.2.weight"] = t["wa"], t["wb"]
    moe = moe.to(c.torch_dtype)
    moe.load_state_dict(sd, strict=True)
    moe = moe.cuda().eval()
    moe.forward_mode, moe.tau = "dynk_max", c.tau
    return moe


def _norm(c, t, kind, eps):
    if kind == "layer":
        n = torch.nn.LayerNorm(c.d, eps=eps).to(c.torch_dtype)
        with torch.no_grad():
            n.weight.copy_(t["gamma"])
            n.bias.copy_(t["beta"])
        return n.cuda()

    class GemmaRMSNorm(torch.nn.Module):          # same contract as transformers' module
        def __init__(self):
            super().__init__()
            self.eps = eps
            self.weight = torch.nn.Parameter(t["gamma"].clone())

        def forward(self, x):
            xf = x.float()
            y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
            return (y * (1.0 + self.weight.float())).type_as(x)
    return GemmaRMSNorm().cuda()


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_prenorm_init_kernel(case):
    from d2dmoe_b200 import ops
    c, kind, eps = case
    g, t = load(c, kind)
    rows = torch.from_numpy(g["rows"])
    x2d = t["x"].reshape(c.N, c.d).cuda()
    xn = torch.empty_like(x2d)
    init = torch.empty_like(x2d)
    lb = None if c.glu else t["last_bias"].cuda().view(-1)
    ops.prenorm_init(x2d, t["gamma"].cuda(), None if t["beta"] is None else t["beta"].cuda(), eps,
                     ops.NORM_LAYER if kind == "layer" else ops.NORM_RMS, xn, init,
                     last_bias=lb, gamma_offset=1.0 if kind == "rms" else 0.0)
    tol = 2e-6 if c.dtype == "fp32" else 2.0 ** -8
    assert O.rel_err(xn.cpu().float()[rows], torch.from_numpy(g["xn"])) <= tol
    ref = O.prenorm(t["x"].reshape(c.N, c.d), t["gamma"], t["beta"], eps, kind,
                    1.0 if kind == "rms" else 0.0)
    assert O.rel_err(xn.cpu().float(), ref.float()) <= tol
    want = t["x"].reshape(c.N, c.d).float()
    if lb is not None:
        want = (want + t["last_bias"].float().view(-1)).to(c.torch_dtype).float()
    assert torch.equal(init.cpu().float(), want)
    # the normalised rows alone (no initial value asked for)
    xn2 = torch.zeros_like(x2d)
    ops.prenorm_init(x2d, t["gamma"].cuda(), None if t["beta"] is None else t["beta"].cuda(), eps,
                     ops.NORM_LAYER if kind == "layer" else ops.NORM_RMS, xn2,
                     gamma_offset=1.0 if kind == "rms" else 0.0)
    assert torch.equal(xn2, xn)


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_forward_block_matches_upstream(case):
    c, kind, eps = case
    g, t = load(c, kind)
    moe, norm = _module(c, t), _norm(c, t, kind, eps)
    x = t["x"].cuda()
    moe.forward_block(x, norm)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        out, gd = moe.forward_block(x, norm)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    rt = gd[c.name][0]
    assert out.shape == x.shape and rt.shape == (c.B, c.S, c.E)
    m = rt.reshape(c.N, c.E).cpu() > 0
    sg = torch.from_numpy(g["scores"]).to(c.torch_dtype)
    m_up = O.unpack_mask(g["mask_bits"], c.E)
    near = O.near_threshold(sg, c.tau, WINDOW[c.dtype] * 2)
    assert ((m != m_up) & ~near).sum().item() == 0
    xn = O.prenorm(t["x"].reshape(c.N, c.d), t["gamma"], t["beta"], eps, kind,
                   1.0 if kind == "rms" else 0.0)
    got = out.reshape(c.N, c.d).cpu().float()
    assert O.rel_err(got, exact_block(c, t, xn, m)) <= TOL[c.dtype]
    rows = torch.from_numpy(g["rows"])
    same = (m == m_up).all(-1)[rows]
    assert same.float().mean().item() >= 0.9
    assert O.rel_err(got[rows][same], torch.from_numpy(g["out"])[same]) <= TOL[c.dtype]
    # and the unfused route through the same module gives the same block output
    y, gd2 = moe(norm(x))
    ref = (x + y).reshape(c.N, c.d).cpu().float()
    agree = (gd2[c.name][0].reshape(c.N, c.E).cpu() > 0).eq(m).all(-1)
    assert agree.float().mean().item() >= 0.98
    assert O.rel_err(got[agree], ref[agree]) <= TOL[c.dtype]
    moe.last_workspace(c.N, x.device).check_status()


@pytest.mark.gpu
def test_forward_block_falls_back_when_not_fusable():
    c, kind, eps = CASES[1]
    g, t = load(c, kind)
    moe, norm = _module(c, t), _norm(c, t, kind, eps)
    x = t["x"].cuda()
    fused, _ = moe.forward_block(x, norm)
    ident = torch.nn.Identity()                    # not a norm the fused pass knows
    out, _ = moe.forward_block(x, ident)
    y, _ = moe(x)
    # (the scatter-add's order differs from call to call: equal up to fp32 rounding)
    assert O.rel_err(out.cpu(), (x + y).cpu()) <= 1e-6
    moe.forward_mode, moe.k = "topk", 2            # another gate: three separate steps
    out, _ = moe.forward_block(x, norm)
    y, _ = moe(norm(x))
    assert O.rel_err(out.cpu(), (x + y).cpu()) <= 1e-6
    assert O.rel_err(out.cpu(), fused.cpu()) > 1e-4


@pytest.mark.gpu
def test_fused_vit_block_forward_equals_the_unfused_block():
    import functools
    import d2dmoe_b200 as D
    c, kind, eps = CASES[0]
    g, t = load(c, kind)

    class Block(torch.nn.Module):                  # attribute names of torchvision's EncoderBlock
        def __init__(self):
            super().__init__()
            self.ln_1 = torch.nn.LayerNorm(c.d, eps=eps)
            self.self_attention = torch.nn.MultiheadAttention(c.d, 12, batch_first=True)
            self.dropout = torch.nn.Dropout(0.0)
            self.ln_2 = torch.nn.LayerNorm(c.d, eps=eps)
            self.mlp = None

    torch.manual_seed(5)
    blk = Block().to(c.torch_dtype)
    with torch.no_grad():
        blk.ln_2.weight.copy_(t["gamma"])
        blk.ln_2.bias.copy_(t["beta"])
    blk.mlp = _module(c, t)
    blk = blk.cuda().eval()
    blk.forward = functools.partial(D.fused_vit_block_forward, blk)
    x = t["x"].cuda()
    with torch.no_grad():
        out, gd = blk(x)
        h = blk.ln_1(x)
        h = blk.self_attention(h, h, h, need_weights=False)[0] + x
        y, gd2 = blk.mlp(blk.ln_2(h))
        ref = h + y
    assert c.name in gd
    agree = gd[c.name][0].eq(gd2[c.name][0]).all(-1)
    assert agree.float().mean().item() >= 0.98
    assert O.rel_err(out[agree].float().cpu(), ref[agree].float().cpu()) <= TOL[c.dtype]


@pytest.mark.gpu
def test_prenorm_rejects_rows_it_cannot_hold():
    from d2dmoe_b200 import ops
    x = torch.randn(4, 8200, device="cuda", dtype=torch.bfloat16)      # 16400-byte rows
    g = torch.ones(8200, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ops._capi.D2DError):
        ops.prenorm_init(x, g, None, 1e-6, ops.NORM_RMS, torch.empty_like(x))
    x = torch.randn(4, 100, device="cuda", dtype=torch.bfloat16)       # 200-byte rows
    g = torch.ones(100, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ops._capi.D2DError):
        ops.prenorm_init(x, g, None, 1e-6, ops.NORM_RMS, torch.empty_like(x))


@pytest.mark.gpu
def test_fused_gpt_block_forward_equals_the_unfused_block():
    import functools
    import d2dmoe_b200 as D
    c, kind, eps = CASES[0]
    g, t = load(c, kind)

    class CausalSelfAttention(torch.nn.Module):     # one-argument attention, as in the GPT block
        def __init__(self):
            super().__init__()
            self.c_attn = torch.nn.Linear(c.d, c.d)

        def forward(self, x):
            return torch.tanh(self.c_attn(x))

    class Block(torch.nn.Module):                  # attribute names of the upstream GPT block
        def __init__(self):
            super().__init__()
            self.ln_1 = torch.nn.LayerNorm(c.d, eps=eps)
            self.attn = CausalSelfAttention()
            self.ln_2 = torch.nn.LayerNorm(c.d, eps=eps)
            self.mlp = None

    torch.manual_seed(6)
    blk = Block().to(c.torch_dtype)
    with torch.no_grad():
        blk.ln_2.weight.copy_(t["gamma"])
        blk.ln_2.bias.copy_(t["beta"])
    blk.mlp = _module(c, t)
    blk.mlp.dropout = torch.nn.Dropout(0.1)        # upstream attaches it; inactive in eval mode
    blk = blk.cuda().eval()
    blk.forward = functools.partial(D.fused_gpt_block_forward, blk)
    x = t["x"].cuda()
    with torch.no_grad():
        out, gd = blk(x)
        h = x + blk.attn(blk.ln_1(x))
        y, gd2 = blk.mlp(blk.ln_2(h))
        ref = h + y
    agree = gd[c.name][0].eq(gd2[c.name][0]).all(-1)
    assert agree.float().mean().item() >= 0.98
    assert O.rel_err(out[agree].float().cpu(), ref[agree].float().cpu()) <= TOL[c.dtype]


@pytest.mark.gpu
def test_fused_gemma_decoder_forward_equals_the_unfused_layer():
    import functools
    import d2dmoe_b200 as D
    c, kind, eps = CASES[2]
    g, t = load(c, kind)

    class Attn(torch.nn.Module):                   # keyword interface of the Gemma attention
        def __init__(self):
            super().__init__()
            self.o = torch.nn.Linear(c.d, c.d, bias=False)

        def forward(self, hidden_states, attention_mask, position_ids, cache_position):
            return self.o(hidden_states), None, None

    class Layer(torch.nn.Module):                  # attribute names of GemmaDecoderLayer
        def __init__(self):
            super().__init__()
            self.input_layernorm = _norm(c, t, kind, eps)
            self.self_attn = Attn()
            self.post_attention_layernorm = _norm(c, t, kind, eps)
            self.mlp = None

    torch.manual_seed(7)
    lyr = Layer().to(c.torch_dtype)
    lyr.mlp = _module(c, t)
    lyr = lyr.cuda().eval()
    lyr.forward = functools.partial(D.fused_gemma_decoder_forward, lyr)
    x = t["x"].cuda()
    with torch.no_grad():
        out, gd = lyr(x, None, None, None)
        h = x + lyr.self_attn(lyr.input_layernorm(x), None, None, None)[0]
        y, gd2 = lyr.mlp(lyr.post_attention_layernorm(h))
        ref = h + y
    agree = gd[c.name][0].eq(gd2[c.name][0]).all(-1)
    assert agree.float().mean().item() >= 0.97
    assert O.rel_err(out[agree].float().cpu(), ref[agree].float().cpu()) <= TOL[c.dtype]


@pytest.mark.gpu
def test_forward_block_keeps_the_framework_norm_for_mixed_precision_and_capture():
    c, kind, eps = CASES[0]
    g, t = load(c, kind)
    moe, norm = _module(c, t), _norm(c, t, kind, eps)
    x = t["x"].cuda()
    fused, _ = moe.forward_block(x, norm)
    # parameters of the norm in another dtype than x: three separate steps, same result class
    norm32 = torch.nn.LayerNorm(c.d, eps=eps).cuda()
    with torch.no_grad():
        norm32.weight.copy_(t["gamma"].float())
        norm32.bias.copy_(t["beta"].float())

    class Mixed(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight, self.bias, self.eps = norm32.weight, norm32.bias, eps
            self.normalized_shape = (c.d,)

        def forward(self, v):
            return norm32(v.float()).to(v.dtype)
    mixed = Mixed()
    assert moe._norm_args(mixed) is None           # not an nn.LayerNorm: ordinary route
    out, _ = moe.forward_block(x, mixed)
    assert O.rel_err(out.float().cpu(), fused.float().cpu()) <= TOL[c.dtype]
    # while the experts capture labels the block runs unfused and the capture still happens
    moe.experts.capture_norms("output", 2)
    out3, _ = moe.forward_block(x, norm)
    assert moe.experts.captured_norms is not None
    assert O.rel_err(out3.float().cpu(), fused.float().cpu()) <= TOL[c.dtype]
    moe.experts.capture_norms(None)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("kind", ["layer", "rms"])
def test_prenorm_init_shapes_against_the_oracle(dtype, kind):
    """Row lengths from one vector per row to the longest supported (every register-footprint
    variant of the kernel), ragged row counts, with and without the initial-value output."""
    from d2dmoe_b200 import ops
    es = 4 if dtype == torch.float32 else 2
    g = torch.Generator().manual_seed(40)
    tol = 2e-6 if dtype == torch.float32 else 2.0 ** -8
    for d in (16 // es, 40, 64, 200, 768, 1024, 2048, 8192 // es):
        for n in (1, 33, 257):
            x = (torch.randn(n, d, generator=g) * 1.7 + 0.4).to(dtype)
            gamma = (1.0 + 0.1 * torch.randn(d, generator=g)).to(dtype)
            beta = (0.1 * torch.randn(d, generator=g)).to(dtype) if kind == "layer" else None
            lb = (0.05 * torch.randn(d, generator=g)).to(dtype)
            goff = 1.0 if kind == "rms" else 0.0
            ref = O.prenorm(x, gamma, beta, 1e-6, kind, goff).float()
            xd = x.cuda()
            xn = torch.full_like(xd, float("nan"))
            init = torch.full_like(xd, float("nan"))
            ops.prenorm_init(xd, gamma.cuda(), None if beta is None else beta.cuda(), 1e-6,
                             ops.NORM_LAYER if kind == "layer" else ops.NORM_RMS, xn, init,
                             last_bias=lb.cuda(), gamma_offset=goff)
            assert O.rel_err(xn.cpu().float(), ref) <= tol, (d, n)
            want = (x.float() + lb.float()).to(dtype).float()
            assert torch.equal(init.cpu().float(), want), (d, n)
