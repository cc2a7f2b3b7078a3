"""Router-training labels (per-expert activation norms captured while the layer runs every
expert on every token) against values captured from the unmodified upstream modules
(tests/golden/labels.npz, made by make_golden_labels.py)."""
import numpy as np
import pytest
import torch

from helpers import C, GOLDEN, O, TOL
import make_golden_labels as ML

CASES = ML.label_cases()
IDS = [c.name for c in CASES]
LAYERS = ("intermediate", "output")


def load(c):
    gz = np.load(GOLDEN / "labels.npz")
    g = {k.split("/", 1)[1]: gz[k] for k in gz.files if k.startswith(c.name + "/")}
    t = C.make_tensors(c)
    assert C.digest(t["x"]) == str(g["dg_x"]), "seeded generator drifted (x)"
    return g, t


@pytest.mark.parametrize("c", CASES, ids=IDS)
def test_oracle_norms_match_upstream(c):
    g, t = load(c)
    x2d = t["x"].reshape(c.N, c.d)
    for layer in LAYERS:
        for ordv in ML.ORDS:
            got = O.expert_activation_norms(x2d, t["w1"], None if c.glu else t["b1"], t["w2"],
                                            c.act, t.get("w_up") if c.glu else None,
                                            layer=layer, ord=ordv)
            ref = torch.from_numpy(g[f"{layer}_ord{ordv}"])
            assert got.shape == (c.E, c.N)
            assert O.rel_err(got.float(), ref) <= TOL[c.dtype], (layer, ordv)


def _module(c, t):
    import d2dmoe_b200 as D
    act = {"relu": torch.nn.ReLU, "gelu": torch.nn.GELU, "tanh": torch.nn.Tanh}[c.act]
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
    return moe.cuda().eval()


def _names(c):
    if c.glu:
        return {"intermediate": "experts.layers.0", "output": "experts.layers.1"}
    return {"intermediate": "experts.intermediate_activation_extraction_stub",
            "output": "experts.output_activation_extraction_stub"}


@pytest.mark.gpu
@pytest.mark.parametrize("c", CASES, ids=IDS)
def test_captured_norms_match_upstream(c):
    """The upstream recipe (mode 'all' + add_save_output_norm_hook on the named modules) on a
    layer of this package: norms from the expert kernel, output unchanged."""
    import d2dmoe_b200 as D
    g, t = load(c)
    moe = _module(c, t)
    moe.forward_mode = "all"
    x = t["x"].cuda()
    out_ref = torch.from_numpy(g["out"])
    for layer, nm in _names(c).items():
        for ordv in ML.ORDS:
            saved, handles = D.add_save_output_norm_hook(moe, [nm], ord=ordv, dim=-1)
            out, gd = moe(x)
            assert bool((gd[c.name][0] == 1).all())
            got = saved[nm]
            assert got.shape == (c.E, c.N) and got.dtype == x.dtype
            ref = torch.from_numpy(g[f"{layer}_ord{ordv}"])
            assert O.rel_err(got.float().cpu(), ref) <= TOL[c.dtype], (layer, ordv)
            assert O.rel_err(out.reshape(c.N, c.d).float().cpu(), out_ref) <= TOL[c.dtype]
            for h in handles:
                h.remove()
            assert moe.experts._capture is None
    moe.last_workspace(c.N, x.device).check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("c", CASES[:3], ids=IDS[:3])
def test_captured_norms_of_a_sparse_routing(c):
    """With a dynamic-k routing only the computed pairs carry a norm, the rest stay zero."""
    g, t = load(c)
    moe = _module(c, t)
    moe.forward_mode, moe.tau = "dynk_max", c.tau
    x = t["x"].cuda()
    out0, gd0 = moe(x)
    moe.experts.capture_norms("output", 2)
    out, gd = moe(x)
    norms = moe.experts.captured_norms.float().cpu()
    m = gd[c.name][0].reshape(c.N, c.E).cpu() > 0
    assert torch.equal(m, gd0[c.name][0].reshape(c.N, c.E).cpu() > 0)
    assert 0 < m.sum().item() < c.N * c.E
    ref = torch.from_numpy(g["output_ord2"])
    assert torch.all(norms[~m.T] == 0)
    assert O.rel_err(norms[m.T], ref[m.T]) <= TOL[c.dtype]
    assert O.rel_err(out.float().cpu(), out0.float().cpu()) <= TOL[c.dtype]
    moe.experts.capture_norms(None)
    # the experts module called directly (ExpertsLayer interface) captures as well
    moe.experts.capture_norms("intermediate", 1)
    rt = torch.ones(c.N, c.E, dtype=x.dtype, device="cuda")
    moe.experts(x.reshape(c.N, c.d), rt)
    got = moe.experts.captured_norms.float().cpu()
    assert O.rel_err(got, torch.from_numpy(g["intermediate_ord1"])) <= TOL[c.dtype]


@pytest.mark.gpu
def test_norm_capture_argument_checks():
    import d2dmoe_b200 as D
    c = CASES[1]
    g, t = load(c)
    moe = _module(c, t)
    with pytest.raises(ValueError):
        moe.experts.capture_norms("hidden")
    with pytest.raises(NotImplementedError):
        moe.experts.capture_norms("output", 3)
    with pytest.raises(NotImplementedError):
        D.add_save_output_norm_hook(moe, ["experts.output_activation_extraction_stub"], 2, dim=0)
    # a module outside an experts layer gets the ordinary hook
    saved, handles = D.add_save_output_norm_hook(moe, ["router"], ord=2, dim=-1)
    moe.forward_mode, moe.tau = "topk", None
    moe.k = 2
    x = t["x"].cuda()
    moe(x)
    assert saved["router"].shape == (c.B, c.S)
    handles[0].remove()


def test_norm_hook_helper_on_host_modules():
    """Host-side contract of the helper (no GPU): an ordinary module gets the upstream forward
    hook, an experts stub switches the capture of its experts module on, remove() undoes both."""
    import d2dmoe_b200 as D
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 6), torch.nn.ReLU())
    saved, handles = D.add_save_output_norm_hook(model, ["0"], ord=2, dim=-1)
    x = torch.randn(5, 8)
    model(x)
    assert torch.allclose(saved["0"], torch.linalg.vector_norm(model[0](x), ord=2, dim=-1))
    handles[0].remove()
    saved.clear()
    model(x)
    assert not saved

    moe = D.MoeficationMoE("m", 16, 4, True, 8, torch.nn.ReLU, experts_class="custom_kernel")
    name = "experts.output_activation_extraction_stub"
    saved, handles = D.add_save_output_norm_hook(moe, [name], ord=1, dim=-1)
    assert moe.experts._capture == ("output", 1)
    with pytest.raises(NotImplementedError):      # one layer / ord per experts module at a time
        D.add_save_output_norm_hook(moe, ["experts.intermediate_activation_extraction_stub"], 2)
    handles[0].remove()
    assert moe.experts._capture is None and not moe.experts._norm_sinks

    glu = D.MoeficationMoE("g", 16, 4, False, 8, torch.nn.GELU, experts_class="execute_all",
                           add_intermediate_gating=True)
    saved, handles = D.add_save_output_norm_hook(glu, ["experts.layers.0"], ord=2, dim=-1)
    assert glu.experts._capture == ("intermediate", 2)
    handles[0].remove()
    saved, handles = D.add_save_output_norm_hook(glu, ["experts.layers.1"], ord=2, dim=-1)
    assert glu.experts._capture == ("output", 2)
    handles[0].remove()
