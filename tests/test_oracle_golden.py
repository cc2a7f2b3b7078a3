"""The CPU oracle against the committed outputs of the upstream modules."""
import numpy as np
import pytest
import torch

from helpers import (O, TOL, WINDOW, all_cases, case_ids, gate_fixture_ids, gate_fixture_items,
                     golden_mask, golden_scores, load_golden)


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_mask_from_upstream_scores_is_bit_exact(c):
    g, t = load_golden(c)
    m = O.dynk_max_mask(golden_scores(g, c), c.tau)
    assert np.array_equal(O.pack_mask(m), g["mask_bits"])


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_router_scores_and_end_to_end_mask(c):
    g, t = load_golden(c)
    if c.score_override:
        pytest.skip("scores are given, no router")
    s = O.router_scores(t["x"].reshape(c.N, c.d), t["wa"], t["wb"])
    sg = golden_scores(g, c)
    err = O.rel_err(s, sg)
    assert err <= (1e-5 if c.dtype == "fp32" else 2.0 ** -7), err
    m = O.dynk_max_mask(s, c.tau)
    near = O.near_threshold(sg, c.tau, WINDOW[c.dtype])
    diff = (m != golden_mask(g, c)) & ~near
    assert diff.sum().item() == 0
    # the exclusion window must stay a rare event, not a loophole
    assert near.sum().item() <= max(4, 0.02 * c.N * c.E) or c.tau in (0.0, 1.0)


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_outputs_match_upstream(c):
    g, t = load_golden(c)
    m = golden_mask(g, c)
    x2d = t["x"].reshape(c.N, c.d)
    rows = torch.from_numpy(g["rows"])
    p = dict(t)
    if c.glu:
        p["b1"] = None
        p["last_bias"] = None
    exact = O.experts_ffn_exact(x2d, m, p["w1"], p["b1"], p["w2"], c.act, p.get("w_up"))
    if p.get("last_bias") is not None:
        exact = exact + p["last_bias"].double()
    if c.residual:
        exact = exact + x2d.double()
    key = "out_execute_all" if c.glu else "out_naive"
    ref = torch.from_numpy(g[key])
    assert O.rel_err(exact[rows], ref) <= TOL[c.dtype]
    if not c.glu:
        assert O.rel_err(exact[rows], torch.from_numpy(g["out_masked"])) <= TOL[c.dtype]
        out, _, _ = O.moe_forward(t["x"], p, c.tau, c.act, c.residual,
                                  scores=golden_scores(g, c))
        out = out.reshape(c.N, c.d).float()
        assert O.rel_err(out[rows], ref) <= (2e-6 if c.dtype == "fp32" else 2.0 ** -7)


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_token_lists(c):
    g, t = load_golden(c)
    m = golden_mask(g, c)
    off, idx = O.expert_token_lists(m)
    assert off[0] == 0 and off[-1] == m.sum().item() == len(idx)
    for e in range(c.E):
        seg = idx[off[e]:off[e + 1]]
        assert np.array_equal(seg, torch.nonzero(m[:, e]).flatten().numpy())


def test_gate_edge_cases():
    # all-zero row keeps every expert; NaN is never kept; arg-max always kept
    s = torch.tensor([[0.0, 0.0, 0.0], [1.0, float("nan"), 0.95], [3.0, 1.0, 2.0]])
    m = O.dynk_max_mask(s, 0.1)
    assert m[0].tolist() == [True, True, True]
    assert m[2].tolist() == [True, False, False]
    assert not m[1, 1]
    assert O.dynk_max_mask(s[2:], 1.0).all()


@pytest.mark.parametrize("item", gate_fixture_items(), ids=gate_fixture_ids())
def test_topk_and_dynk_rules_match_upstream_gate(item):
    """The oracle's restatement of the 'topk' and cumulative 'dynk' gates against what the
    upstream MoeficationMoE.gate returned for the same scores (tests/golden/gates.npz)."""
    c, rule, par, bits = item
    g, _ = load_golden(c)
    s = golden_scores(g, c).reshape(c.N, c.E)
    m = O.gate_topk(s, par) if rule == "topk" else O.gate_dynk_cumulative(s, par)
    assert torch.equal(m, O.unpack_mask(bits, c.E))


GLU_CASES = [c for c in all_cases() if c.glu]


@pytest.mark.parametrize("c", GLU_CASES, ids=[c.name for c in GLU_CASES])
def test_glu_module_port_matches_upstream_module_experts(c):
    """The restated sparse CPU path of a gated layer (experts_class='module': one GLUExpert of
    three nn.Linear per expert) against what the upstream module returned for the same
    parameters and routing tensor (fixture key out_module)."""
    g, t = load_golden(c)
    if "out_module" not in g:
        pytest.skip("fixture predates the module-experts output")
    m = golden_mask(g, c)
    x2d = t["x"].reshape(c.N, c.d)
    lin = O.glu_module_weights(t["w1"], t["w_up"], t["w2"])
    out = O.experts_glu_module(x2d, m.to(x2d.dtype), lin, c.act).float()
    rows = torch.from_numpy(g["rows"])
    ref = torch.from_numpy(g["out_module"])
    # same torch CPU calls in the same order on the same bits
    assert O.rel_err(out[rows], ref) <= (2e-6 if c.dtype == "fp32" else 2.0 ** -7)
    # and the sparse and dense upstream forms agree with each other within the tolerance
    assert O.rel_err(ref, torch.from_numpy(g["out_execute_all"])) <= TOL[c.dtype]
    # whole-layer form used as the timed CPU baseline of the gated configuration
    p = {"wa": t["wa"], "wb": t["wb"], "lin": lin}
    out2, rt = O.cpu_layer_forward_module_glu(t["x"], p, c.tau, c.act)
    near = O.near_threshold(golden_scores(g, c), c.tau, WINDOW[c.dtype])
    assert (((rt.reshape(c.N, c.E) > 0) != m) & ~near).sum().item() == 0
