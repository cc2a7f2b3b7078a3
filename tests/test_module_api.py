"""Host-side mirror of the upstream module interface (no GPU needed)."""
import inspect

import pytest
import torch

import d2dmoe_b200 as D
from oracle.ref_shim import load_reference

KEYS = {"last_bias": (1, 64), "experts.w1": (4, 64, 32), "experts.b1": (4, 32),
        "experts.w2": (4, 32, 64), "router.layers.0.weight": (128, 64),
        "router.layers.2.weight": (4, 128)}


def make(cls_moe=D.MoeficationMoE, cls_router=D.MoeficationRouter, **kw):
    # positional order as the upstream test builds it (scripts/test_moe_implementations.py:64-67)
    m = cls_moe("test_moe", 64, 4, True, 32, torch.nn.ReLU, **kw)
    m.router = cls_router(64, 4, width=128, depth=2, bias=False, activation="relu",
                          output_activation="abs")
    return m


def test_state_dict_layout():
    m = make()
    sd = m.state_dict()
    assert {k: tuple(v.shape) for k, v in sd.items()} == KEYS
    assert m.forward_mode == "all" and m.tau is None and m.k is None and m.router is not None
    for attr in ("name", "hidden_dim", "expert_dim", "num_experts", "bias", "experts",
                 "last_bias", "add_residual_connection"):
        assert hasattr(m, attr)
    e = m.experts
    for attr in ("num_experts", "depth", "expert_dim", "hidden_dim", "bias_mode", "act",
                 "activation_str", "forward_mode", "intermediate_activation_extraction_stub",
                 "output_activation_extraction_stub"):
        assert hasattr(e, attr)


def test_glu_state_dict_layout():
    m = D.MoeficationMoE("g", 64, 8, False, 32, torch.nn.GELU, experts_class="execute_all",
                         add_intermediate_gating=True)
    assert {k: tuple(v.shape) for k, v in m.state_dict().items()} == {
        "experts.layers.0.w": (8, 64, 32), "experts.layers.1.w": (8, 32, 64),
        "experts.layers.2.w": (8, 64, 32)}


def test_preconditions_raise_like_upstream():
    with pytest.raises(AssertionError):
        D.B200KernelExperts(64, 4, depth=3, expert_dim=32, bias="without_last",
                            activation=torch.nn.ReLU)
    with pytest.raises(AssertionError):
        D.B200KernelExperts(64, 4, expert_dim=32, bias=True, activation=torch.nn.ReLU)
    with pytest.raises(AssertionError):
        D.B200KernelExperts(64, 4, expert_dim=32, bias="without_last", activation=torch.nn.SiLU)
    with pytest.raises(NotImplementedError):
        D.B200KernelExperts(64, 4, expert_dim=32, bias="without_last", activation=torch.nn.ReLU,
                            intermediate_gating=True)


def test_no_cpu_path():
    m = make()
    m.forward_mode, m.tau = "dynk_max", 0.5
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        m(torch.randn(2, 3, 64))
    m.experts.forward_mode = "naive"
    with pytest.raises(NotImplementedError):
        m.experts(torch.randn(6, 64), torch.ones(6, 4))


def test_matches_upstream_signatures_and_checkpoint():
    ref = load_reference()
    if ref is None:
        pytest.skip("no upstream checkout on this machine")
    for ours, theirs in ((D.MoeficationMoE, ref.MoeficationMoE),
                         (D.MoeficationRouter, ref.MoeficationRouter),
                         (D.B200KernelExperts, ref.CustomKernelExperts)):
        a = inspect.signature(ours.__init__).parameters
        b = inspect.signature(theirs.__init__).parameters
        assert list(a) == list(b)
        for k in b:
            if k == "experts_class":
                continue
            assert a[k].default == b[k].default, (ours, k)
    r = make(ref.MoeficationMoE, ref.MoeficationRouter, experts_class="custom_kernel")
    m = make()
    m.load_state_dict(r.state_dict(), strict=True)      # an upstream checkpoint loads
    r.load_state_dict(m.state_dict(), strict=True)      # and ours loads upstream
    # the key under which upstream call sites build the layer resolves to the CUDA class
    assert D.MOE_IMPL_MAP["custom_kernel"] is D.B200KernelExperts
