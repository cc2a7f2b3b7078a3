"""Drop-in wiring inside the upstream code base (CPU; needs the read-only upstream checkout).

The upstream block and attention forwards dispatch on ``isinstance(module, MoELayer)`` and
build experts from ``MOE_IMPL_MAP``.  After ``bind_upstream()`` the classes of this package
must pass both, for FFN layers and for MoE-fied q/k/v/o attention projections
(architectures/moe/moe_models.py:13-76, architectures/moe/dsti.py:88-138).  The CUDA
arithmetic itself is covered by the GPU parity tests; here a CPU stand-in for ``forward``
shows which branch the upstream code takes.
"""
from functools import partial

import pytest
import torch
from torch import nn

from oracle.ref_shim import load_reference


@pytest.fixture(scope="module")
def upstream():
    ref = load_reference()
    if ref is None:
        pytest.skip("no upstream checkout")
    import d2dmoe_b200 as D
    assert D.bind_upstream()
    return ref, D


def test_classes_are_upstream_moe_layers(upstream):
    ref, D = upstream
    from architectures.moe import moe_layers
    assert issubclass(D.MoeficationMoE, moe_layers.MoELayer)
    assert issubclass(D.B200KernelExperts, moe_layers.ExpertsLayer)
    assert moe_layers.MOE_IMPL_MAP["b200_kernel"] is D.B200KernelExperts
    assert moe_layers.MOE_IMPL_MAP["b200_glu"] is D.B200GluExperts
    # the upstream layer builds this package's experts by key, with the upstream state_dict layout
    up = ref.MoeficationMoE("l", 64, 4, True, 32, nn.ReLU, experts_class="b200_kernel")
    assert isinstance(up.experts, D.B200KernelExperts)
    want = ref.MoeficationMoE("l", 64, 4, True, 32, nn.ReLU, experts_class="custom_kernel")
    assert {k: tuple(v.shape) for k, v in up.state_dict().items()} == \
           {k: tuple(v.shape) for k, v in want.state_dict().items()}
    ours = D.MoeficationMoE("l", 64, 4, True, 32, nn.ReLU, experts_class="custom_kernel")
    ours.load_state_dict(want.state_dict(), strict=True)


def test_upstream_block_and_attention_forwards_dispatch_to_these_layers(upstream):
    ref, D = upstream
    from architectures.custom import CustomMultiheadAttention
    from architectures.moe import moe_models

    class Echo(D.MoeficationMoE):
        """CPU stand-in for the CUDA forward: same return convention."""

        def forward(self, x):
            rt = torch.ones(*x.shape[:-1], self.num_experts)
            return x * 0.5 + (x if self.add_residual_connection else 0.0), {self.name: (rt,)}

    d = 64
    attn = CustomMultiheadAttention(d, 4)
    # MoE-fied projections: the same layer type with a residual connection (dsti.py:88-138)
    attn.q_proj = Echo("blk.q_proj", d, 4, True, 8, nn.GELU, add_residual_connection=True)
    attn.o_proj = Echo("blk.o_proj", d, 4, True, 8, nn.GELU, add_residual_connection=True)
    attn.forward = partial(moe_models.moe_attention_forward, attn)
    block = nn.Module()
    block.ln_1, block.ln_2 = nn.LayerNorm(d), nn.LayerNorm(d)
    block.dropout = nn.Identity()
    block.self_attention = attn
    block.mlp = Echo("blk.mlp", d, 4, True, 16, nn.ReLU)
    x = torch.randn(2, 5, d)
    out, gd = moe_models.moe_vit_block_forward(block, x)
    assert out.shape == x.shape
    assert set(gd) == {"blk.q_proj", "blk.o_proj", "blk.mlp"}       # all three taken as MoE layers
    assert gd["blk.mlp"][0].shape == (2, 5, 4)
    # the real class refuses CPU tensors loudly instead of computing something else
    real = D.MoeficationMoE("m", d, 4, True, 16, nn.ReLU)
    real.forward_mode, real.tau = "dynk_max", 0.1
    real.router = D.MoeficationRouter(d, 4, activation="relu", output_activation="abs")
    with pytest.raises(RuntimeError, match="CUDA"):
        real(x)
