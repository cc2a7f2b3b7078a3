"""Size-independent properties at the benchmark's full layer size (ViT-B/16, batch 256:
50432 tokens x 768, 24 experts x 128, bf16), where the CPU oracle is too slow to run
on every row."""
import numpy as np
import pytest
import torch

from helpers import C, O

pytestmark = pytest.mark.gpu

B, S, D, H, E, R = 256, 197, 768, 128, 24, 128
N = B * S


@pytest.fixture(scope="module")
def layer():
    import d2dmoe_b200 as Dm
    g = torch.Generator(device="cuda").manual_seed(11)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")           # noqa: E731
    x = torch.nn.functional.layer_norm(rn(B, S, D), (D,)).bfloat16()
    moe = Dm.MoeficationMoE("moe", D, E, True, H, torch.nn.ReLU, experts_class="custom_kernel")
    moe.router = Dm.MoeficationRouter(D, E, width=R, depth=2, bias=False, activation="relu",
                                      output_activation="abs")
    moe = moe.to(torch.bfloat16).cuda()
    with torch.no_grad():
        for p in moe.parameters():
            p.copy_((rn(*p.shape) * 0.02).to(p.dtype))
    moe.forward_mode, moe.tau = "dynk_max", 0.1
    return moe, x


def _lists(moe):
    w = moe.last_workspace(N, torch.device("cuda", torch.cuda.current_device()))
    off = w.offsets.clone()
    idx = w.token_idx[: int(off[E])].clone()
    bits = w.mask_bits[:N, 0].clone()
    w.check_status()
    return bits, off, idx


def test_lists_are_the_mask(layer):
    moe, x = layer
    out, gd = moe(x)
    rt = gd["moe"][0].reshape(N, E)
    bits, off, idx = _lists(moe)
    # bit mask <-> routing tensor
    e = torch.arange(E, device="cuda")
    assert torch.equal(((bits.unsqueeze(1) >> e) & 1).bool(), rt > 0)
    # offsets are the column sums, lists are torch.nonzero order (ascending, unique)
    counts = (rt > 0).sum(0).to(torch.int32)
    assert torch.equal(off[1:] - off[:-1], counts) and int(off[0]) == 0
    ref = torch.cat([torch.nonzero(rt[:, j] > 0).flatten() for j in range(E)]).to(torch.int32)
    assert torch.equal(idx, ref)
    # the rule itself, evaluated by tensor ops on the kernel-independent scores
    assert (rt.sum(1) >= 1).all()


def test_run_twice_same_bits(layer):
    moe, x = layer
    moe(x)
    a = _lists(moe)
    o1, _ = moe(x)
    b = _lists(moe)
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    o2, _ = moe(x)
    # scatter-add order is not fixed: outputs agree within the bf16 tolerance
    assert O.rel_err(o1.float().cpu(), o2.float().cpu()) <= 2e-2


def test_all_experts_equals_dense_ffn(layer):
    """tau = 1.0 keeps every expert: the layer is then the dense FFN the experts were cut
    from, relu(x W1cat + b1cat) W2cat + last_bias, computed here by fp32 matmuls."""
    moe, x = layer
    moe.tau = 1.0
    try:
        out, gd = moe(x)
    finally:
        moe.tau = 0.1
    assert bool((gd["moe"][0] == 1).all())
    x2 = x.reshape(N, D).float()
    w1 = moe.experts.w1.float().permute(1, 0, 2).reshape(D, E * H)
    b1 = moe.experts.b1.float().reshape(E * H)
    w2 = moe.experts.w2.float().reshape(E * H, D)
    torch.backends.cuda.matmul.allow_tf32 = False
    h = torch.relu((x2 @ w1).bfloat16().float() + b1).bfloat16().float()
    ref = h @ w2 + moe.last_bias.float()
    assert O.rel_err(out.reshape(N, D).float().cpu(), ref.cpu()) <= 2e-2


def test_token_permutation_equivariance(layer):
    moe, x = layer
    perm = torch.randperm(N, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    o1, g1 = moe(x)
    xp = x.reshape(N, D)[perm].reshape(B, S, D).contiguous()
    o2, g2 = moe(xp)
    assert torch.equal(g1["moe"][0].reshape(N, E)[perm], g2["moe"][0].reshape(N, E))   # bit-exact
    assert O.rel_err(o2.reshape(N, D).float().cpu(), o1.reshape(N, D)[perm].float().cpu()) <= 2e-2


def test_rule_on_lognormal_scores_full_size():
    """GPT-2-sized score override: 32768 tokens, log-normal(0, 1.5) scores, rule only."""
    from d2dmoe_b200 import ops
    n = 32 * 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    s = torch.exp(1.5 * torch.randn(n, E, generator=g, device="cuda")).bfloat16()
    wsp = ops.Workspace.allocate(n, E, "cuda")
    for tau_cfg in (0.8, 0.9, 0.95):
        tau = 1.0 - tau_cfg
        ops.mask_from_scores(s, tau, wsp)
        rt = ops.expand_mask(wsp, n, E, torch.bfloat16)
        mx = s.float().max(-1, keepdim=True).values
        thr = (mx * torch.tensor(np.float32(1.0 - tau), device="cuda")).bfloat16().float()
        assert torch.equal(rt > 0, s.float() >= thr)            # bit-exact, zero exclusions
    wsp.check_status()


def test_sampled_rows_against_oracle(layer):
    moe, x = layer
    out, gd = moe(x)
    idx = torch.arange(0, N, N // 64)[:64]
    xs = x.reshape(N, D)[idx.cuda()].cpu()
    p = {k: v.detach().cpu() for k, v in moe.state_dict().items()}
    s = O.router_scores(xs, p["router.layers.0.weight"], p["router.layers.2.weight"])
    m_or = O.dynk_max_mask(s, moe.tau)
    m = gd["moe"][0].reshape(N, E)[idx.cuda()].cpu() > 0
    near = O.near_threshold(s, moe.tau, 2.0 ** -7)
    assert ((m != m_or) & ~near).sum().item() == 0
    ex = O.experts_ffn_exact(xs, m, p["experts.w1"], p["experts.b1"], p["experts.w2"]) \
        + p["last_bias"].double()
    assert O.rel_err(out.reshape(N, D)[idx.cuda()].float().cpu(), ex) <= 2e-2


# ---------------------------------------------------------------------------------------
# The other configurations at their full layer size: sampled rows against the CPU oracle.
# ---------------------------------------------------------------------------------------
FULL = {
    # name: (B, S, d, H, E, R, glu, act, norm, scores given)
    "gpt2_scores_32768": (32, 1024, 768, 128, 24, 128, False, "relu", "layer", True),
    "bert_96x32_65536": (512, 128, 768, 32, 96, 128, False, "relu", "layer", False),
    "gemma_geglu_131072": (64, 2048, 2048, 128, 128, 256, True, "gelu", "rms", False),
}


@pytest.mark.parametrize("name", list(FULL), ids=list(FULL))
def test_full_size_configs_sampled_rows(name):
    """One layer of the GPT-2 (log-normal score override), BERT (96 experts x 32) and
    Gemma-size (GeGLU, d 2048, 128 experts, 256-wide router) configurations at full token
    count through the module: the routing tensor must be the rule on the scores (all tokens
    for given scores; sampled tokens, outside the tie window, for the fused router), the token
    lists must be the routing tensor's columns, and sampled output rows must match the fp64
    evaluation of the experts the layer selected."""
    import d2dmoe_b200 as Dm
    Bn, Sn, d, Hn, En, Rn, glu, act, norm, given = FULL[name]
    n = Bn * Sn
    g = torch.Generator(device="cuda").manual_seed(len(name))
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")           # noqa: E731
    x = rn(Bn, Sn, d)
    if norm == "layer":
        x = torch.nn.functional.layer_norm(x, (d,))
    else:
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    x = x.bfloat16()
    actm = {"relu": torch.nn.ReLU, "gelu": torch.nn.GELU}[act]
    if glu:
        moe = Dm.MoeficationMoE("moe", d, En, False, Hn, actm, experts_class="execute_all",
                                add_intermediate_gating=True)
    else:
        moe = Dm.MoeficationMoE("moe", d, En, True, Hn, actm, experts_class="custom_kernel")
    moe.router = Dm.MoeficationRouter(d, En, width=Rn, depth=2, bias=False, activation="relu",
                                      output_activation="abs")
    moe = moe.to(torch.bfloat16).cuda()
    with torch.no_grad():
        for p in moe.parameters():
            p.copy_((rn(*p.shape) * 0.02).to(p.dtype))
    scores = None
    if given:
        scores = torch.exp(1.5 * rn(Bn, Sn, En)).bfloat16()

        class Fixed(torch.nn.Module):
            def forward(self, x):
                return scores
        moe.router = Fixed()
    moe.forward_mode, moe.tau = "dynk_max", 0.1
    out, gd = moe(x)
    torch.cuda.synchronize()
    rt = gd["moe"][0].reshape(n, En)
    w = moe.last_workspace(n, x.device)
    w.check_status()
    # token lists = columns of the routing tensor, ascending
    off = w.offsets.clone()
    counts = (rt > 0).sum(0).to(torch.int32)
    assert int(off[0]) == 0 and torch.equal(off[1:] - off[:-1], counts)
    for e in (0, En // 3, En - 1):
        seg = w.token_idx[int(off[e]):int(off[e + 1])]
        assert torch.equal(seg, torch.nonzero(rt[:, e] > 0).flatten().to(torch.int32))
    assert (rt.sum(1) >= 1).all()
    idx = torch.arange(0, n, n // 64)[:64]
    xs = x.reshape(n, d)[idx.cuda()].cpu()
    m = rt[idx.cuda()].cpu() > 0
    sd = {k: v.detach().cpu() for k, v in moe.state_dict().items()}
    if given:
        s2 = scores.reshape(n, En)
        mx = s2.float().max(-1, keepdim=True).values
        thr = (mx * torch.tensor(np.float32(1.0 - 0.1), device="cuda")).bfloat16().float()
        assert torch.equal(rt > 0, s2.float() >= thr)               # every token, bit-exact
    else:
        s = O.router_scores(xs, sd["router.layers.0.weight"], sd["router.layers.2.weight"])
        near = O.near_threshold(s, moe.tau, 2.0 ** -7)
        assert ((m != O.dynk_max_mask(s, moe.tau)) & ~near).sum().item() == 0
    if glu:
        ex = O.experts_ffn_exact(xs, m, sd["experts.layers.0.w"], None, sd["experts.layers.1.w"],
                                 act, sd["experts.layers.2.w"])
    else:
        ex = O.experts_ffn_exact(xs, m, sd["experts.w1"], sd["experts.b1"], sd["experts.w2"], act) \
            + sd["last_bias"].double()
    assert O.rel_err(out.reshape(n, d)[idx.cuda()].float().cpu(), ex) <= 2e-2
    # every row was written (no row left at its pre-call contents): all finite and no row of zeros
    assert torch.isfinite(out.float()).all()


def test_fused_block_at_full_size(layer):
    """Pre-norm + residual folded around the layer at 50432 tokens: the fused call against
    torch LayerNorm + layer + add on every row whose routing agrees, and against the fp64
    evaluation (normalised row through the experts the layer chose) on sampled rows."""
    moe, x = layer
    g = torch.Generator(device="cuda").manual_seed(12)
    xin = (x.float() * 1.3 + 0.2).bfloat16()
    ln = torch.nn.LayerNorm(D, eps=1e-6).cuda().bfloat16()
    with torch.no_grad():
        ln.weight.copy_(1.0 + 0.1 * torch.randn(D, generator=g, device="cuda"))
        ln.bias.copy_(0.1 * torch.randn(D, generator=g, device="cuda"))
    out, gd = moe.forward_block(xin, ln)
    y, gd2 = moe(ln(xin))
    ref = xin + y
    m = gd["moe"][0].reshape(N, E) > 0
    agree = m.eq(gd2["moe"][0].reshape(N, E) > 0).all(-1)
    assert agree.float().mean().item() >= 0.99
    o2, r2 = out.reshape(N, D)[agree].float(), ref.reshape(N, D)[agree].float()
    assert ((o2 - r2).abs().max() / r2.abs().max()).item() <= 2e-2
    rows = torch.arange(0, N, 997, device="cuda")
    xs = xin.reshape(N, D)[rows].cpu()
    xn = O.prenorm(xs, ln.weight.detach().cpu(), ln.bias.detach().cpu(), 1e-6, "layer")
    exact = O.experts_ffn_exact(xn, m[rows].cpu(), moe.experts.w1.detach().cpu(),
                                moe.experts.b1.detach().cpu(), moe.experts.w2.detach().cpu(), "relu")
    exact = exact + moe.last_bias.detach().cpu().double() + xs.double()
    assert O.rel_err(out.reshape(N, D)[rows].cpu().float(), exact) <= 2e-2
    moe.last_workspace(N, x.device).check_status()


def test_label_capture_at_full_size(layer):
    """Mode 'all' at 50432 tokens x 24 experts: every pair carries a label, sampled tokens
    agree with the upstream recipe evaluated on the host, and the output is the dense FFN."""
    moe, x = layer
    mode = moe.forward_mode
    moe.forward_mode = "all"
    moe.experts.capture_norms("output", 2)
    try:
        out, gd = moe(x)
        norms = moe.experts.captured_norms
    finally:
        moe.experts.capture_norms(None)
        moe.forward_mode = mode
    assert norms.shape == (E, N) and bool((norms > 0).all())
    rows = torch.arange(0, N, 1009, device="cuda")
    xs = x.reshape(N, D)[rows].cpu()
    w1, b1, w2 = (p.detach().cpu() for p in (moe.experts.w1, moe.experts.b1, moe.experts.w2))
    ref = O.expert_activation_norms(xs, w1, b1, w2, "relu", layer="output", ord=2)
    assert O.rel_err(norms[:, rows].cpu().float(), ref.float()) <= 2e-2
    exact = O.experts_ffn_exact(xs, torch.ones(len(rows), E, dtype=torch.bool), w1, b1, w2, "relu")
    exact = exact + moe.last_bias.detach().cpu().double()
    # 24 bf16 adds per element: the summation-order bound of a dense row
    assert O.rel_err(out.reshape(N, D)[rows].cpu().float(), exact) <= 4e-2
    moe.last_workspace(N, x.device).check_status()
