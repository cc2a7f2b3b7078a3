"""CUDA path vs the committed upstream outputs and the CPU oracle (through the C ABI)."""
import numpy as np
import pytest
import torch

from helpers import (C, O, TOL, WINDOW, all_cases, case_ids, gate_fixture_ids, gate_fixture_items,
                     golden_mask, golden_scores, load_golden, rule_tie_tokens)

pytestmark = pytest.mark.gpu


def dev(t):
    return None if t is None else t.cuda().contiguous()


def bits_of(wsp, N):
    return wsp.mask_bits[:N].cpu().numpy().view(np.uint32)


def lists_of(wsp, E):
    off = wsp.offsets.cpu().numpy()
    idx = wsp.token_idx[: int(off[E])].cpu().numpy()
    return off, idx


def load_mask(wsp, mask):
    b = torch.from_numpy(O.pack_mask(mask).view(np.int32)).cuda()
    wsp.mask_bits[: b.shape[0]].copy_(b)


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_mask_from_upstream_scores_bit_exact(c):
    from d2dmoe_b200 import ops
    g, t = load_golden(c)
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    ops.mask_from_scores(dev(golden_scores(g, c)), c.tau, wsp)
    assert np.array_equal(bits_of(wsp, c.N), g["mask_bits"])      # zero exclusions
    wsp.check_status()


@pytest.mark.parametrize("item", gate_fixture_items(), ids=gate_fixture_ids())
def test_topk_and_dynk_rules(item):
    """The top-k and cumulative-share rules on the upstream scores against the routing tensor
    the upstream gate returned: every token outside the tie window must agree exactly."""
    from d2dmoe_b200 import ops
    c, rule, par, bits = item
    g, _ = load_golden(c)
    s = golden_scores(g, c).reshape(c.N, c.E)
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    if rule == "topk":
        ops.mask_rule_from_scores(dev(s), "topk", wsp, k=par)
    else:
        ops.mask_rule_from_scores(dev(s), "dynk", wsp, tau=par)
    m = O.unpack_mask(bits_of(wsp, c.N), c.E)
    ref = O.unpack_mask(bits, c.E)
    bad = (m != ref).any(-1)
    tie = rule_tie_tokens(s, rule, par, WINDOW[c.dtype], ref)
    assert (bad & ~tie).sum().item() == 0, f"{int(bad.sum())} tokens differ, {int(tie.sum())} in window"
    wsp.check_status()


@pytest.mark.parametrize("E", [24, 96, 130])
def test_rule_kernel_equals_c_oracle_bf16(E):
    """bf16 scores add up exactly in fp32 and both sides order equal values by index, so the
    rule kernel and the C restatement must agree on every bit, ties included."""
    import ctypes as CT
    from d2dmoe_b200 import ops
    from oracle.build_c import build
    lib = CT.CDLL(str(build()))
    N = 20000
    g = torch.Generator().manual_seed(E)
    s = torch.exp(1.5 * torch.randn(N, E, generator=g)).to(torch.bfloat16)
    a = s.view(torch.int16).numpy().view(np.uint16)
    nw = (E + 31) // 32
    wsp = ops.Workspace.allocate(N, E, "cuda")
    for rule, r, k, tau in (("topk", 1, 3, 0.0), ("dynk", 2, 0, 0.7)):
        ref = np.zeros((N, nw), dtype=np.uint32)
        lib.d2d_oracle_rule_bf16(a.ctypes.data_as(CT.c_void_p), r, k, CT.c_float(tau),
                                 ref.ctypes.data_as(CT.c_void_p), CT.c_long(N), E)
        if rule == "topk":
            ops.mask_rule_from_scores(dev(s), "topk", wsp, k=k)
        else:
            ops.mask_rule_from_scores(dev(s), "dynk", wsp, tau=tau)
        assert np.array_equal(bits_of(wsp, N), ref), rule
    wsp.check_status()


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_router_mask(c):
    from d2dmoe_b200 import ops
    g, t = load_golden(c)
    if c.score_override:
        pytest.skip("scores are given, no router")
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    x2d = dev(t["x"].reshape(c.N, c.d))
    scores = torch.empty(c.N, c.E, dtype=c.torch_dtype, device="cuda")
    wa, wb = dev(t["wa"]), dev(t["wb"])
    for packed in (None, ops.prepack_router(wa, wb)):
        ops.router_mask(x2d, wa, wb, c.tau, wsp, scores_out=scores, packed=packed)
        sg = golden_scores(g, c)
        err = O.rel_err(scores.cpu(), sg)
        assert err <= (1e-5 if c.dtype == "fp32" else 2.0 ** -7), err
        m = O.unpack_mask(bits_of(wsp, c.N), c.E)
        # our own scores -> our own mask must be exactly the rule
        assert torch.equal(m, O.dynk_max_mask(scores.cpu(), c.tau))
        near = O.near_threshold(sg, c.tau, WINDOW[c.dtype])
        bad = ((m != golden_mask(g, c)) & ~near).sum().item()
        assert bad == 0, f"{bad} mask bits differ outside the tie window ({near.sum().item()} excluded)"
        wsp.check_status()


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_compaction_bit_exact(c):
    from d2dmoe_b200 import ops
    g, t = load_golden(c)
    mask = golden_mask(g, c)
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    load_mask(wsp, mask)
    ops.compact(wsp, c.N, c.E)
    off, idx = lists_of(wsp, c.E)
    roff, ridx = O.expert_token_lists(mask)
    assert np.array_equal(off, roff) and np.array_equal(idx, ridx)
    ops.compact(wsp, c.N, c.E)          # run twice: same bits
    off2, idx2 = lists_of(wsp, c.E)
    assert np.array_equal(off, off2) and np.array_equal(idx, idx2)
    wsp.check_status()


def _exact(c, t, mask):
    x2d = t["x"].reshape(c.N, c.d)
    b1 = None if c.glu else t["b1"]
    ex = O.experts_ffn_exact(x2d, mask, t["w1"], b1, t["w2"], c.act, t.get("w_up"))
    if not c.glu:
        ex = ex + t["last_bias"].double()
    if c.residual:
        ex = ex + x2d.double()
    return ex


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_experts_ffn(c):
    from d2dmoe_b200 import ops
    g, t = load_golden(c)
    mask = golden_mask(g, c)
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    load_mask(wsp, mask)
    ops.compact(wsp, c.N, c.E)
    x2d = dev(t["x"].reshape(c.N, c.d))
    w1, w2 = dev(t["w1"]), dev(t["w2"])
    b1 = None if c.glu else dev(t["b1"])
    w_up = dev(t.get("w_up"))
    lb = None if c.glu else dev(t["last_bias"].reshape(-1))
    rows = torch.from_numpy(g["rows"])
    ref = torch.from_numpy(g["out_execute_all" if c.glu else "out_naive"])
    exact = _exact(c, t, mask)
    for packed in (None, ops.prepack_experts(w1, b1, w2, w_up)):
        out = torch.full((c.N, c.d), float("nan"), dtype=c.torch_dtype, device="cuda")
        ops.experts_ffn(x2d, wsp, w1, b1, w2, c.act, out, w_up=w_up, packed=packed, last_bias=lb,
                        add_residual=c.residual, accumulate=False)
        o = out.cpu().float()
        assert O.rel_err(o[rows], ref) <= TOL[c.dtype]          # vs upstream output
        assert O.rel_err(o, exact) <= TOL[c.dtype]              # vs fp64 truth, every row
        wsp.check_status()


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_fused_forward_writes_every_row(c):
    """The one-call layer on an output buffer pre-filled with NaN: the router kernel writes every
    row's initial value (last_bias, plus x with a residual connection) and the expert kernel
    adds to it, so a row that neither wrote would still hold NaN."""
    from d2dmoe_b200 import ops
    g, t = load_golden(c)
    x2d = dev(t["x"].reshape(c.N, c.d))
    w1, w2 = dev(t["w1"]), dev(t["w2"])
    b1 = None if c.glu else dev(t["b1"])
    w_up = dev(t.get("w_up"))
    lb = None if c.glu else dev(t["last_bias"].reshape(-1))
    wa, wb = dev(t["wa"]), dev(t["wb"])
    scores = dev(t["scores"].reshape(c.N, c.E)) if c.score_override else None
    rp = None if c.score_override else ops.prepack_router(wa, wb)
    ep = ops.prepack_experts(w1, b1, w2, w_up)
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    for packed in ((None, None), (rp, ep)):
        out = torch.full((c.N, c.d), float("nan"), dtype=c.torch_dtype, device="cuda")
        ops.moe_forward(x2d, wa, wb, c.tau, w1, b1, w2, c.act, out, wsp, w_up=w_up, scores=scores,
                        last_bias=lb, add_residual=c.residual, router_packed=packed[0],
                        experts_packed=packed[1])
        wsp.check_status()
        m = O.unpack_mask(bits_of(wsp, c.N), c.E)
        near = O.near_threshold(golden_scores(g, c), c.tau, WINDOW[c.dtype])
        assert ((m != golden_mask(g, c)) & ~near).sum().item() == 0
        o = out.cpu().float()
        assert torch.isfinite(o).all()
        assert O.rel_err(o, _exact(c, t, m)) <= TOL[c.dtype]
        # the token lists the call leaves behind are the compaction of that mask
        off_ref, idx_ref = O.expert_token_lists(m)
        off, idx = lists_of(wsp, c.E)
        assert np.array_equal(off, np.asarray(off_ref)) and np.array_equal(idx, np.asarray(idx_ref))


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_module_forward(c):
    import d2dmoe_b200 as D
    g, t = load_golden(c)
    act = {"relu": torch.nn.ReLU, "gelu": torch.nn.GELU, "tanh": torch.nn.Tanh,
           "leaky_relu": torch.nn.LeakyReLU}[c.act]
    if c.glu:
        moe = D.MoeficationMoE(c.name, c.d, c.E, False, c.H, act, experts_class="execute_all",
                               add_intermediate_gating=True)
        sd = {"experts.layers.0.w": t["w1"], "experts.layers.1.w": t["w2"],
              "experts.layers.2.w": t["w_up"]}
    else:
        moe = D.MoeficationMoE(c.name, c.d, c.E, True, c.H, act, experts_class="custom_kernel",
                               add_residual_connection=c.residual)
        sd = {"experts.w1": t["w1"], "experts.b1": t["b1"], "experts.w2": t["w2"],
              "last_bias": t["last_bias"]}
    moe.router = D.MoeficationRouter(c.d, c.E, width=c.R, depth=2, bias=False, activation="relu",
                                     output_activation="abs")
    sd["router.layers.0.weight"], sd["router.layers.2.weight"] = t["wa"], t["wb"]
    moe = moe.to(c.torch_dtype)
    moe.load_state_dict(sd, strict=True)
    if c.score_override:
        dev_scores = t["scores"].cuda()

        class Fixed(torch.nn.Module):
            def forward(self, x):
                return dev_scores
        moe.router = Fixed()
    moe = moe.cuda().eval()
    moe.forward_mode, moe.tau = "dynk_max", c.tau
    x = t["x"].cuda()
    moe(x)                                   # warm-up: caches, packed weights
    torch.cuda.synchronize()
    # the layer must not synchronise with the host
    # (upstream enforces this for its GPU mode: scripts/test_moe_implementations.py:78-83)
    torch.cuda.set_sync_debug_mode("error")
    try:
        out, gd = moe(x)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    rt = gd[c.name][0]
    assert out.shape == x.shape and rt.shape == (c.B, c.S, c.E) and rt.dtype == x.dtype
    m = rt.reshape(c.N, c.E).cpu() > 0
    assert set(rt.unique().tolist()) <= {0.0, 1.0}
    near = O.near_threshold(golden_scores(g, c), c.tau, WINDOW[c.dtype])
    assert ((m != golden_mask(g, c)) & ~near).sum().item() == 0
    exact = _exact(c, t, m)                  # truth for the mask the layer itself chose
    assert O.rel_err(out.reshape(c.N, c.d).cpu().float(), exact) <= TOL[c.dtype]
    if torch.equal(m, golden_mask(g, c)):
        rows = torch.from_numpy(g["rows"])
        ref = torch.from_numpy(g["out_execute_all" if c.glu else "out_naive"])
        assert O.rel_err(out.reshape(c.N, c.d).cpu().float()[rows], ref) <= TOL[c.dtype]
    moe.last_workspace(c.N, x.device).check_status()


def test_other_forward_modes_match_oracle():
    import d2dmoe_b200 as D
    c = C.LayerCase("modes", 2, 37, 64, 32, 8, tau=0.6)
    t = C.make_tensors(c)
    moe = D.MoeficationMoE(c.name, c.d, c.E, True, c.H, torch.nn.ReLU)
    moe.router = D.MoeficationRouter(c.d, c.E, width=c.R, depth=2, bias=False, activation="relu",
                                     output_activation="abs")
    moe.load_state_dict({"experts.w1": t["w1"], "experts.b1": t["b1"], "experts.w2": t["w2"],
                         "last_bias": t["last_bias"], "router.layers.0.weight": t["wa"],
                         "router.layers.2.weight": t["wb"]})
    moe = moe.cuda()
    x2d = t["x"].reshape(c.N, c.d)
    s = O.router_scores(x2d, t["wa"], t["wb"])
    for mode, mask in (("all", torch.ones(c.N, c.E, dtype=torch.bool)),
                       ("topk", O.gate_topk(s, 3)),
                       ("dynk", O.gate_dynk_cumulative(s, 0.6))):
        moe.forward_mode, moe.k, moe.tau = mode, 3, 0.6
        out, gd = moe(t["x"].cuda())
        m = gd[c.name][0].reshape(c.N, c.E).cpu() > 0
        assert (m != mask).sum().item() <= 2          # fp32 router ties only
        ex = O.experts_ffn_exact(x2d, m, t["w1"], t["b1"], t["w2"]) + t["last_bias"].double()
        assert O.rel_err(out.reshape(c.N, c.d).cpu(), ex) <= TOL["fp32"]


def test_fused_forward_in_a_cuda_graph():
    """The one-call layer issues no host synchronisation and allocates nothing, so it can be
    captured in a CUDA graph; a replay on new input contents must give the new result."""
    from d2dmoe_b200 import ops
    c = C.LayerCase("graph", 4, 197, 256, 64, 16, tau=0.2, dtype="bf16")
    t = C.make_tensors(c)
    x = dev(t["x"].reshape(c.N, c.d))
    w1, b1, w2 = dev(t["w1"]), dev(t["b1"]), dev(t["w2"])
    wa, wb, lb = dev(t["wa"]), dev(t["wb"]), dev(t["last_bias"].reshape(-1))
    rp, ep = ops.prepack_router(wa, wb), ops.prepack_experts(w1, b1, w2)
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    out = torch.empty_like(x)

    def call():
        ops.moe_forward(x, wa, wb, c.tau, w1, b1, w2, c.act, out, wsp, last_bias=lb,
                        router_packed=rp, experts_packed=ep)
    call()
    torch.cuda.synchronize()
    ref1 = out.clone()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        call()                                         # warm-up on the capture stream
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            call()
    x2 = torch.roll(x, 7, 0).contiguous()
    x.copy_(x2)
    out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    got2 = out.clone()
    call()                                             # same input, eager
    torch.cuda.synchronize()
    wsp.check_status()
    assert torch.isfinite(got2.float()).all()
    assert O.rel_err(got2.float().cpu(), out.float().cpu()) <= TOL["bf16"]
    assert O.rel_err(torch.roll(ref1, 7, 0).float().cpu(), got2.float().cpu()) <= TOL["bf16"]


@pytest.mark.parametrize("n", [4700, 4800])
def test_general_shape_router_mid_sizes(n):
    """fp32 router + rule of the general-shape kernel at a few thousand tokens with a narrow
    router (d=96, R=64): scores against the oracle, mask exactly the rule on those scores."""
    from d2dmoe_b200 import ops
    c = C.LayerCase("tiles", 1, n, 96, 32, 24, R=64, tau=0.2)
    t = C.make_tensors(c)
    x2d = dev(t["x"].reshape(c.N, c.d))
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    scores = torch.empty(c.N, c.E, dtype=torch.float32, device="cuda")
    ops.router_mask(x2d, dev(t["wa"]), dev(t["wb"]), c.tau, wsp, scores_out=scores)
    s_ref = O.router_scores(t["x"].reshape(c.N, c.d), t["wa"], t["wb"])
    assert O.rel_err(scores.cpu(), s_ref) <= 1e-5
    m = O.unpack_mask(bits_of(wsp, c.N), c.E)
    assert torch.equal(m, O.dynk_max_mask(scores.cpu(), c.tau))
    wsp.check_status()


def test_fused_forward_on_two_streams():
    """Two layers issued alternately on two streams (each with its own workspace and output)
    give what they give one after the other: kernels wait only for their own stream's
    predecessor."""
    from d2dmoe_b200 import ops
    c = C.LayerCase("streams", 8, 197, 256, 64, 16, tau=0.3, dtype="bf16")
    t = C.make_tensors(c)
    w1, b1, w2 = dev(t["w1"]), dev(t["b1"]), dev(t["w2"])
    wa, wb, lb = dev(t["wa"]), dev(t["wb"]), dev(t["last_bias"].reshape(-1))
    rp, ep = ops.prepack_router(wa, wb), ops.prepack_experts(w1, b1, w2)
    xs = [dev(t["x"].reshape(c.N, c.d)), dev(torch.roll(t["x"].reshape(c.N, c.d), 5, 0))]
    wsp = [ops.Workspace.allocate(c.N, c.E, "cuda") for _ in range(2)]
    outs = [torch.empty_like(xs[0]) for _ in range(2)]
    ref = []
    for i in range(2):
        ops.moe_forward(xs[i], wa, wb, c.tau, w1, b1, w2, c.act, outs[i], wsp[i], last_bias=lb,
                        router_packed=rp, experts_packed=ep)
        torch.cuda.synchronize()
        ref.append(outs[i].clone())
        outs[i].fill_(float("nan"))
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for rep in range(6):
        for i in range(2):
            with torch.cuda.stream(streams[i]):
                ops.moe_forward(xs[i], wa, wb, c.tau, w1, b1, w2, c.act, outs[i], wsp[i],
                                last_bias=lb, router_packed=rp, experts_packed=ep)
    torch.cuda.synchronize()
    for i in range(2):
        wsp[i].check_status()
        assert O.rel_err(outs[i].float().cpu(), ref[i].float().cpu()) <= TOL["bf16"]


def test_empty_and_error_paths():
    from d2dmoe_b200 import ops, _capi
    import d2dmoe_b200 as D
    moe = D.MoeficationMoE("e", 64, 4, True, 32, torch.nn.ReLU).cuda()
    moe.router = D.MoeficationRouter(64, 4, activation="relu", output_activation="abs").cuda()
    moe.forward_mode, moe.tau = "dynk_max", 0.5
    out, gd = moe(torch.empty(0, 3, 64, device="cuda"))
    assert out.shape == (0, 3, 64) and gd["e"][0].shape == (0, 3, 4)
    wsp = ops.Workspace.allocate(8, 4, "cuda")
    small = ops.Workspace.allocate(8, 4, "cuda")
    small.ws = small.ws[:0]
    with pytest.raises(_capi.D2DError, match="WORKSPACE|BAD_ARG"):
        ops.compact(small, 5000, 4)
    # out-of-range token index: reported through the device status word, no fault
    wsp.offsets.copy_(torch.tensor([0, 1, 1, 1, 1], dtype=torch.int32))
    wsp.token_idx[:1] = 12345
    x = torch.randn(8, 64, device="cuda")
    w1 = torch.randn(4, 64, 32, device="cuda")
    b1 = torch.randn(4, 32, device="cuda")
    w2 = torch.randn(4, 32, 64, device="cuda")
    out = torch.empty(8, 64, device="cuda")
    ops.experts_ffn(x, wsp, w1, b1, w2, "relu", out)
    with pytest.raises(_capi.D2DError, match="INDEX_RANGE"):
        wsp.check_status()
    assert torch.equal(out, torch.zeros_like(out))      # nothing was added


def test_forward_host_matches_forward():
    """Host-buffer entry point: pipelined slices give the rule's bits and outputs of forward()."""
    import d2dmoe_b200 as D
    c = C.LayerCase("host", 16, 33, 128, 64, 8, tau=0.3, dtype="bf16")
    t = C.make_tensors(c)
    moe = D.MoeficationMoE(c.name, c.d, c.E, True, c.H, torch.nn.ReLU)
    moe.router = D.MoeficationRouter(c.d, c.E, width=c.R, depth=2, bias=False, activation="relu",
                                     output_activation="abs")
    moe = moe.to(torch.bfloat16)
    moe.load_state_dict({"experts.w1": t["w1"], "experts.b1": t["b1"], "experts.w2": t["w2"],
                         "last_bias": t["last_bias"], "router.layers.0.weight": t["wa"],
                         "router.layers.2.weight": t["wb"]})
    moe = moe.cuda()
    moe.forward_mode, moe.tau = "dynk_max", c.tau
    ref, _ = moe(t["x"].cuda())
    xh = t["x"].pin_memory()
    o1 = moe.forward_host(xh, chunks=3)
    o2 = torch.empty_like(xh).pin_memory()
    o3 = torch.empty_like(xh).pin_memory()
    moe.forward_host(xh, o2, chunks=5, sync=False)
    moe.forward_host(xh, o3, chunks=2, sync=False)
    D.MoeficationMoE.host_synchronize()
    for o in (o1, o2, o3):
        assert O.rel_err(o.float(), ref.float().cpu()) <= TOL["bf16"]


DIRECT = ["n197_vit_bf16", "n129_e64", "gelu_bias_res", "e96_h32_bert", "glu_small_bf16",
          "gemma_shape"]


@pytest.mark.parametrize("name", DIRECT)
def test_experts_module_called_directly(name):
    """``experts(x2d, routing_tensor)``, the ExpertsLayer interface
    (architectures/moe/moe_layers.py:174-191), fed the upstream routing tensor: output against
    the upstream experts output (out_naive has last_bias and the residual added, so they are
    added here too) and against the fp64 evaluation."""
    import d2dmoe_b200 as D
    c = {k.name: k for k in all_cases()}[name]
    g, t = load_golden(c)
    act = {"relu": torch.nn.ReLU, "gelu": torch.nn.GELU}[c.act]
    if c.glu:
        ex = D.B200GluExperts(c.d, c.E, depth=2, expert_dim=c.H, bias=False, activation=act)
        sd = {"layers.0.w": t["w1"], "layers.1.w": t["w2"], "layers.2.w": t["w_up"]}
    else:
        ex = D.B200KernelExperts(c.d, c.E, depth=2, expert_dim=c.H, bias="without_last",
                                 activation=act)
        sd = {"w1": t["w1"], "b1": t["b1"], "w2": t["w2"]}
    ex = ex.to(c.torch_dtype)
    ex.load_state_dict(sd, strict=True)
    ex = ex.cuda()
    mask = golden_mask(g, c)
    rt = mask.to(c.torch_dtype).cuda()
    x2d = t["x"].reshape(c.N, c.d).cuda()
    out = ex(x2d, rt)
    out2 = ex(x2d, rt)                                  # cached workspace and packed weights
    o = out.float().cpu()
    if not c.glu:
        o = (o.to(c.torch_dtype) + t["last_bias"]).float()     # what MoeficationMoE.forward adds
    if c.residual:
        o = (o.to(c.torch_dtype) + x2d.cpu()).float()
    rows = torch.from_numpy(g["rows"])
    ref = torch.from_numpy(g["out_execute_all" if c.glu else "out_naive"])
    assert O.rel_err(o[rows], ref) <= TOL[c.dtype]
    assert O.rel_err(o, _exact(c, t, mask)) <= TOL[c.dtype]
    assert O.rel_err(out2.float().cpu(), out.float().cpu()) <= TOL[c.dtype]
    with pytest.raises(NotImplementedError):
        ex.forward_mode = "naive"
        ex(x2d, rt)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_gelu_tanh_activation(dtype):
    """The tanh form of GELU (what Gemma's own act_fn uses) on both kernel families, against
    the fp64 evaluation of the same formula."""
    from d2dmoe_b200 import ops
    c = C.LayerCase("gelu_tanh", 3, 67, 128, 64, 8, tau=0.4, dtype=dtype, act="gelu_tanh",
                    glu=(dtype == "bf16"), norm="rms")
    t = C.make_tensors(c)
    x2d = t["x"].reshape(c.N, c.d)
    s = O.router_scores(x2d, t["wa"], t["wb"])
    mask = O.dynk_max_mask(s, c.tau)
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    load_mask(wsp, mask)
    ops.compact(wsp, c.N, c.E)
    b1 = None if c.glu else t["b1"]
    exact = O.experts_ffn_exact(x2d, mask, t["w1"], b1, t["w2"], "gelu_tanh", t.get("w_up"))
    w1, w2, w_up = dev(t["w1"]), dev(t["w2"]), dev(t.get("w_up"))
    for packed in (None, ops.prepack_experts(w1, dev(b1), w2, w_up)):
        out = torch.full((c.N, c.d), float("nan"), dtype=c.torch_dtype, device="cuda")
        ops.experts_ffn(dev(x2d), wsp, w1, dev(b1), w2, "gelu_tanh", out, w_up=w_up, packed=packed)
        assert O.rel_err(out.float().cpu(), exact) <= TOL[dtype]
    wsp.check_status()


def test_residual_summation_order_bound():
    """bf16 layer with a residual connection and inputs of magnitude ~1 against small expert
    outputs.  Upstream adds the expert sum, then last_bias, then x (one rounding at the
    magnitude of x); here the output starts as bf16(last_bias + x) and every expert
    contribution is added to it in bf16, i.e. k+1 roundings at the magnitude of the output.
    Every element must stay inside that bound around the fp64 value."""
    from d2dmoe_b200 import ops
    c = C.LayerCase("res_order", 4, 97, 128, 64, 8, tau=0.6, dtype="bf16", norm="none",
                    zero_last_bias=False, residual=True, seed=9)
    t = C.make_tensors(c)
    x2d = t["x"].reshape(c.N, c.d)
    wa, wb = dev(t["wa"]), dev(t["wb"])
    w1, b1, w2 = dev(t["w1"]), dev(t["b1"]), dev(t["w2"])
    lb = dev(t["last_bias"].reshape(-1))
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    out = torch.empty(c.N, c.d, dtype=torch.bfloat16, device="cuda")
    ops.moe_forward(dev(x2d), wa, wb, c.tau, w1, b1, w2, "relu", out, wsp, last_bias=lb,
                    add_residual=True, router_packed=ops.prepack_router(wa, wb),
                    experts_packed=ops.prepack_experts(w1, b1, w2))
    wsp.check_status()
    m = O.unpack_mask(bits_of(wsp, c.N), c.E)
    k = m.sum(-1, keepdim=True).double()
    assert k.max().item() >= 3                                  # the case must have multi-expert tokens
    ex = O.experts_ffn_exact(x2d, m, t["w1"], t["b1"], t["w2"]) + t["last_bias"].double() \
        + x2d.double()
    err = (out.float().cpu().double() - ex).abs()
    # unit roundoff of bf16 is 2^-8; partial sums stay within the larger of |x| and |result|
    mag = torch.maximum(ex.abs(), x2d.double().abs()) + (ex - x2d.double()).abs()
    bound = (k + 1.0) * 2.0 ** -8 * mag + 2.0 ** -8 * (ex - x2d.double()).abs()
    assert (err <= bound * 1.5 + 2e-3).all(), float((err / (bound + 1e-12)).max())
    # and the upstream order (one rounding at the end) is not better than this by more than
    # the extra k roundings: compare the two max errors
    up = ((O.experts_ffn_naive(x2d, m, t["w1"], t["b1"], t["w2"]).float()
           + t["last_bias"].float()).bfloat16().float() + x2d.float()).bfloat16().double()
    e_up = (up - ex).abs().max().item()
    assert err.max().item() <= (k.max().item() + 1.0) * max(e_up, 2.0 ** -9)


def test_compact_zero_tokens_through_the_c_abi():
    """N = 0 through both compaction entry points, after a non-empty call that leaves the
    counts table and the outputs dirty: offsets must come back all zero, status clean."""
    import ctypes as CT
    from d2dmoe_b200 import ops, _capi
    E = 24
    wsp = ops.Workspace.allocate(1000, E, "cuda")
    m = torch.rand(1000, E) < 0.2
    load_mask(wsp, m)
    ops.compact(wsp, 1000, E)
    assert int(wsp.offsets[E]) == int(m.sum())
    p = lambda x: CT.c_void_p(x.data_ptr())                              # noqa: E731
    st = CT.c_void_p(torch.cuda.current_stream().cuda_stream)
    for fn in ("d2d_compact", "d2d_compact_noalloc"):
        wsp.offsets.fill_(77)
        if fn == "d2d_compact":
            rc = _capi.lib.d2d_compact(p(wsp.mask_bits), p(wsp.token_idx), p(wsp.offsets), 0, E,
                                       p(wsp.ws), wsp.ws.numel(), p(wsp.status), st)
        else:
            rc = _capi.lib.d2d_compact_noalloc(p(wsp.mask_bits), p(wsp.token_idx), p(wsp.offsets),
                                               0, E, p(wsp.status), st)
        assert rc == 0
        assert torch.equal(wsp.offsets, torch.zeros_like(wsp.offsets)), fn
        wsp.check_status()


def test_bounded_wait_runs_out_and_the_next_launch_is_clean():
    """A weight tile that never arrives (test hook) makes a bounded device wait run out: the
    kernel must report D2D_ERR_TIMEOUT in the status word and return, with its tensor memory
    freed, so that the same call right afterwards, hook off, gives the normal result."""
    from d2dmoe_b200 import ops, _capi
    c = C.LayerCase("timeout", 4, 197, 256, 64, 16, tau=0.2, dtype="bf16")
    t = C.make_tensors(c)
    x = dev(t["x"].reshape(c.N, c.d))
    w1, b1, w2 = dev(t["w1"]), dev(t["b1"]), dev(t["w2"])
    wa, wb, lb = dev(t["wa"]), dev(t["wb"]), dev(t["last_bias"].reshape(-1))
    rp, ep = ops.prepack_router(wa, wb), ops.prepack_experts(w1, b1, w2)
    wsp = ops.Workspace.allocate(c.N, c.E, "cuda")
    out = torch.empty_like(x)

    def call():
        ops.moe_forward(x, wa, wb, c.tau, w1, b1, w2, c.act, out, wsp, last_bias=lb,
                        router_packed=rp, experts_packed=ep)
    call()
    torch.cuda.synchronize()
    wsp.check_status()
    ref = out.clone()
    try:
        assert _capi.lib.d2d_debug_configure(12, 1) == 0
        call()
        torch.cuda.synchronize()                     # returns: nothing hangs
        with pytest.raises(_capi.D2DError, match="TIMEOUT"):
            wsp.check_status()
    finally:
        _capi.lib.d2d_debug_configure(0, 0)
    out.fill_(float("nan"))
    call()
    torch.cuda.synchronize()
    wsp.check_status()
    assert O.rel_err(out.float().cpu(), ref.float().cpu()) <= TOL["bf16"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_two_devices_driven_by_one_process():
    """One process, two GPUs, neither made current by the caller beforehand: the library keeps
    its launch facts (shared-memory opt-in, SM count) per device and the wrappers make the
    tensors' device current, so the same layer gives the same bits for mask and lists, and the
    same output within tolerance, on both."""
    import d2dmoe_b200 as D
    c = C.LayerCase("twodev", 4, 197, 256, 64, 16, tau=0.2, dtype="bf16")
    t = C.make_tensors(c)
    outs = []
    for dev_i in (1, 0, 1):                       # second device first
        dev_ = torch.device("cuda", dev_i)
        moe = D.MoeficationMoE(c.name, c.d, c.E, True, c.H, torch.nn.ReLU)
        moe.router = D.MoeficationRouter(c.d, c.E, width=c.R, depth=2, bias=False,
                                         activation="relu", output_activation="abs")
        moe = moe.to(torch.bfloat16)
        moe.load_state_dict({"experts.w1": t["w1"], "experts.b1": t["b1"], "experts.w2": t["w2"],
                             "last_bias": t["last_bias"], "router.layers.0.weight": t["wa"],
                             "router.layers.2.weight": t["wb"]})
        moe = moe.to(dev_)
        moe.forward_mode, moe.tau = "dynk_max", c.tau
        out, gd = moe(t["x"].to(dev_))            # current device stays cuda:0 throughout
        torch.cuda.synchronize(dev_)
        moe.last_workspace(c.N, dev_).check_status()
        outs.append((out.float().cpu(), gd[c.name][0].cpu()))
    assert torch.cuda.current_device() == 0
    for o, rt in outs[1:]:
        assert torch.equal(rt, outs[0][1])
        assert O.rel_err(o, outs[0][0]) <= TOL["bf16"]
