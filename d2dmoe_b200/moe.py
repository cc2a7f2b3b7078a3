"""Drop-in PyTorch modules for the upstream MoE-FFN inference layer.

Same constructor arguments, attributes, ``state_dict`` keys/shapes and
``forward`` signatures as the upstream classes, with the computation done by the
sm_100a CUDA library:

  MoeficationMoE      <-> architectures/moe/moefication.py:28-101
  MoeficationRouter   <-> architectures/moe/moefication.py:309-339
  B200KernelExperts   <-> CustomKernelExperts, architectures/moe/moe_layers.py:136-264
  B200GluExperts      <-> ExecuteAllExperts with intermediate gating,
                          architectures/moe/moe_layers.py:50-101
  MOE_IMPL_MAP        <-> architectures/moe/moe_layers.py:402-407

state_dict of MoeficationMoE(bias=True, experts_class='b200_kernel') + router:
  last_bias [1,d], experts.w1 [E,d,H], experts.b1 [E,H], experts.w2 [E,H,d],
  router.layers.0.weight [R,d], router.layers.2.weight [E,R]
which is what an upstream checkpoint of the 'custom_kernel' layer holds.

There is no CPU path: a forward on CPU tensors raises.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from . import ops

ACTIVATION_TO_NAME = {nn.GELU: "gelu", nn.Tanh: "tanh", nn.ReLU: "relu", nn.LeakyReLU: "leaky_relu"}


def _function_module(fn):
    class _Fn(nn.Module):
        def forward(self, x):
            return fn(x)
    return _Fn


# name -> module class, as in common.py:159-169
ACTIVATION_NAME_MAP = {
    "relu": nn.ReLU, "gelu": nn.GELU, "sigmoid": nn.Sigmoid, "tanh": nn.Tanh,
    "leaky_relu": nn.LeakyReLU, "softplus": nn.Softplus, "silu": nn.SiLU,
    "abs": _function_module(torch.abs), "identity": nn.Identity,
}

# forward_mode strings of the upstream experts class that mean "the fast GPU path"
_KERNEL_MODES = ("b200", "triton_atomic", "triton")


def _uniform_init(p: torch.Tensor) -> torch.Tensor:
    """uniform(-1/sqrt(last dim), +1/sqrt(last dim)) (architectures/moe/moe_layers.py:19-24)."""
    with torch.no_grad():
        b = 1.0 / math.sqrt(p.size(-1))
        p.uniform_(-b, b)
    return p


class _WorkspaceCache:
    """Per-module cache of caller-owned buffers, keyed by (tokens, device)."""

    def __init__(self):
        self._w = {}

    def get(self, n: int, E: int, device) -> ops.Workspace:
        key = (n, E, str(device))
        w = self._w.get(key)
        if w is None:
            if len(self._w) > 8:
                self._w.clear()
            w = ops.Workspace.allocate(n, E, device)
            self._w[key] = w
        return w


class _PackedCache:
    """Packed weight images, rebuilt when a source parameter changes.

    A change is seen through the parameter's storage address, shape, dtype and version
    counter, i.e. ``load_state_dict``, ``.to()``, ``copy_`` and other in-place tensor ops.
    Writes that bypass the version counter (``p.data.copy_(...)``, raw pointer writes) are
    not seen: call ``invalidate()`` (``module.invalidate_packed()``) after those."""

    def __init__(self):
        self._key = None
        self._buf = None

    def invalidate(self):
        self._key = None
        self._buf = None

    def get(self, params, make):
        key = tuple((p.data_ptr(), p._version, p.dtype, tuple(p.shape)) for p in params
                    if p is not None)
        if key != self._key:
            self._buf = make()
            self._key = key
        return self._buf


class ExpertIntermediateActivationExtractionStub(nn.Module):
    """Parameter-free hook point kept for attribute compatibility
    (architectures/moe/moe_layers.py:116-125); the fused kernel does not call it."""


class ExpertOutputActivationExtractionStub(nn.Module):
    """Parameter-free hook point (architectures/moe/moe_layers.py:128-133)."""


class ExpertsLayer(nn.Module):
    pass


class B200KernelExperts(ExpertsLayer):
    """Experts of a two-layer FFN split (CustomKernelExperts-compatible).

    Parameters w1 [E,d,H], b1 [E,H], w2 [E,H,d]; ``forward(x[N,d], routing_tensor[N,E])``
    returns sum over the experts with a non-zero routing entry of
    act(x W1[e] + b1[e]) W2[e]  (architectures/moe/moe_layers.py:174-211).
    """

    def __init__(self, dim, num_experts, depth=2, expert_dim=None, bias=True, activation=nn.GELU,
                 intermediate_gating=False):
        if intermediate_gating:
            raise NotImplementedError("intermediate_gating: use experts_class='b200_glu'")
        super().__init__()
        assert depth == 2, "No support for depth != 2 for now"
        assert bias == "without_last", 'No support for bias != "without_last" for now'
        assert activation in ACTIVATION_TO_NAME, f"{activation} not supported by the kernel"
        self.num_experts = num_experts
        self.depth = depth
        self.expert_dim = dim * 2 if expert_dim is None else expert_dim
        self.hidden_dim = dim
        self.bias_mode = bias
        self.w1 = _uniform_init(nn.Parameter(torch.empty(num_experts, dim, self.expert_dim)))
        self.b1 = _uniform_init(nn.Parameter(torch.empty(num_experts, self.expert_dim)))
        self.w2 = _uniform_init(nn.Parameter(torch.empty(num_experts, self.expert_dim, dim)))
        self.act = activation()
        self.activation_str = ACTIVATION_TO_NAME[activation]
        self._forward_mode = "b200"
        self.intermediate_activation_extraction_stub = ExpertIntermediateActivationExtractionStub()
        self.output_activation_extraction_stub = ExpertOutputActivationExtractionStub()
        self._wsp = _WorkspaceCache()
        self._packed = _PackedCache()
        self._capture = None
        self._norm_sinks = []
        self.captured_norms = None

    @property
    def forward_mode(self):
        return self._forward_mode

    @forward_mode.setter
    def forward_mode(self, value):
        self._forward_mode = value

    # parameters in the order the kernels take them
    def kernel_params(self):
        return dict(w1=self.w1, b1=self.b1, w2=self.w2, w_up=None, act=self.activation_str)

    def packed(self):
        p = self.kernel_params()
        return self._packed.get((p["w1"], p["b1"], p["w2"], p["w_up"]),
                                lambda: ops.prepack_experts(p["w1"].detach(),
                                                            None if p["b1"] is None else p["b1"].detach(),
                                                            p["w2"].detach(),
                                                            None if p["w_up"] is None else p["w_up"].detach()))

    def invalidate_packed(self):
        """Drop the packed weight copy (needed only after writes through ``.data``)."""
        self._packed.invalidate()

    # -- router-training labels as a by-product of the expert kernel ----------------------
    def capture_norms(self, layer, ord=2):
        """Make every following forward also produce ``captured_norms`` [E, N]: the vector
        norm (ord 1 or 2, over the last dimension) of each expert's ``layer`` activations
        ('intermediate' = act(x W1 + b1), 'output' = the expert's output) for each token it
        runs on, zero elsewhere.  This is what router training reads through forward hooks
        on the extraction stubs upstream (methods/dynamic_sparsification/train_routers.py:
        49-82, utils.py:353-369) without the [E, N, d] activations being materialised.
        ``layer=None`` switches the capture off."""
        if layer is None:
            self._capture = None
            return
        if layer not in ops.NORM_OF:
            raise ValueError(f"Unknown layer for labels construction: {layer}")
        if ord not in (1, 2):
            raise NotImplementedError("vector norms of ord 1 and 2 are provided")
        self._capture = (layer, int(ord))

    def _norm_args(self, N, like):
        """Keyword arguments of ops.experts_ffn for the current capture setting."""
        if self._capture is None:
            return {}
        norms = torch.empty(self.num_experts, N, dtype=like.dtype, device=like.device)
        return dict(norms=norms, norm_layer=self._capture[0], norm_ord=self._capture[1])

    def _deliver_norms(self, kw):
        if kw:
            self.captured_norms = kw["norms"]
            for saved, key in self._norm_sinks:
                saved[key] = self.captured_norms

    def _check_mode(self):
        if self._forward_mode not in _KERNEL_MODES:
            raise NotImplementedError(
                f"Unsupported forward_mode: {self._forward_mode!r}; this class runs the CUDA "
                f"kernels only (modes {_KERNEL_MODES})")

    @torch.no_grad()
    def forward(self, x, routing_tensor):
        assert x.dim() == 2, f"{x.size()=}"
        self._check_mode()
        N, _ = x.shape
        E = self.num_experts
        x = x.contiguous()
        rt = routing_tensor.contiguous().to(x.dtype)
        wsp = self._wsp.get(N, E, x.device)
        out = torch.empty_like(x)
        if N == 0:
            return out
        p = self.kernel_params()
        ops.pack_mask(rt, wsp)
        ops.compact(wsp, N, E)
        kw = self._norm_args(N, x)
        ops.experts_ffn(x, wsp, p["w1"], p["b1"], p["w2"], p["act"], out, w_up=p["w_up"],
                        packed=self.packed(), accumulate=False, **kw)
        self._deliver_norms(kw)
        return out


class _GluLayer(nn.Module):
    """Holder of one stacked expert weight ``w [E, in, out]``, named like
    ExecuteAllExpertsLayer (architectures/moe/moe_layers.py:32-47) so that
    ``layers.{i}.w`` keys of an upstream state_dict load."""

    def __init__(self, in_dim, out_dim, num_experts):
        super().__init__()
        self.w = _uniform_init(nn.Parameter(torch.empty(num_experts, in_dim, out_dim)))


class B200GluExperts(B200KernelExperts):
    """Gated experts: down(act(gate(x)) * up(x)), no biases.  Parameter names follow
    ExecuteAllExperts with intermediate gating: layers.0 = gate, layers.1 = down,
    layers.2 = up (architectures/moe/moe_layers.py:71-78,91-96)."""

    def __init__(self, dim, num_experts, depth=2, expert_dim=None, bias=False, activation=nn.GELU,
                 intermediate_gating=True):
        ExpertsLayer.__init__(self)
        assert depth == 2, "Intermediate gating not supported for depth > 2"
        if bias not in (False, None):
            raise NotImplementedError("gated experts with biases are not supported by the kernel")
        if not intermediate_gating:
            raise NotImplementedError("use experts_class='b200_kernel' for ungated experts")
        assert activation in ACTIVATION_TO_NAME, f"{activation} not supported by the kernel"
        self.num_experts = num_experts
        self.depth = depth
        self.dim = dim
        self.hidden_dim = dim
        self.expert_dim = dim * 2 if expert_dim is None else expert_dim
        self.bias_mode = bias
        self.activation = activation
        self.intermediate_gating = True
        self.layers = nn.ModuleList([
            _GluLayer(dim, self.expert_dim, num_experts),
            _GluLayer(self.expert_dim, dim, num_experts),
            _GluLayer(dim, self.expert_dim, num_experts),
        ])
        self.act = activation()
        self.activation_str = ACTIVATION_TO_NAME[activation]
        self._forward_mode = "b200"
        self._wsp = _WorkspaceCache()
        self._packed = _PackedCache()
        self._capture = None
        self._norm_sinks = []
        self.captured_norms = None

    def kernel_params(self):
        return dict(w1=self.layers[0].w, b1=None, w2=self.layers[1].w, w_up=self.layers[2].w,
                    act=self.activation_str)


MOE_IMPL_MAP = {
    "b200_kernel": B200KernelExperts,
    "b200_glu": B200GluExperts,
    # upstream keys resolve to the CUDA classes so that existing call sites
    # (replace_with_moes(..., experts_class='custom_kernel')) pick them up
    "custom_kernel": B200KernelExperts,
}


# per device: (host-to-device, compute, device-to-host) streams shared by all layers
_HOST_STREAMS: dict = {}


class MoELayer(nn.Module):
    def __init__(self, name, num_experts):
        nn.Module.__init__(self)      # not super(): bind_upstream() may re-base this class
        self.name = name
        self.num_experts = num_experts


class MoeficationRouter(nn.Module):
    """Regression router MLP (architectures/moe/moefication.py:309-339): same
    constructor, same ``layers`` ModuleList (so the state_dict keys are
    ``layers.0.weight`` and ``layers.2.weight`` for depth 2) and the same cached
    Bernoulli override used by the upstream micro-benchmark."""

    def __init__(self, hidden_dim, num_experts, width=128, depth=2, bias=False, activation="tanh",
                 output_activation="identity", test_override_outputs_p=None):
        super().__init__()
        self.layers = nn.ModuleList()
        if depth == 1:
            self.layers.append(nn.Linear(hidden_dim, num_experts, bias=bias))
        else:
            self.layers.append(nn.Linear(hidden_dim, width, bias=bias))
            self.layers.append(ACTIVATION_NAME_MAP[activation]())
            for _ in range(depth - 2):
                self.layers.append(nn.Linear(width, width, bias=bias))
                self.layers.append(ACTIVATION_NAME_MAP[activation]())
            self.layers.append(nn.Linear(width, num_experts, bias=bias))
        self.layers.append(ACTIVATION_NAME_MAP[output_activation]())
        self.test_override_outputs_p = test_override_outputs_p
        if test_override_outputs_p is not None:
            self.response_cache = {}
        self._fusable = (depth == 2 and not bias and activation == "relu"
                         and output_activation == "abs" and test_override_outputs_p is None)
        self._packed = _PackedCache()

    def fusable(self) -> bool:
        """True when the router is the D2DMoE form (depth 2, ReLU, abs, no bias) that
        the fused router+mask kernel computes."""
        return self._fusable

    def packed(self):
        wa, wb = self.layers[0].weight, self.layers[2].weight
        return self._packed.get((wa, wb), lambda: ops.prepack_router(wa.detach(), wb.detach()))

    def invalidate_packed(self):
        """Drop the packed weight copy (needed only after writes through ``.data``)."""
        self._packed.invalidate()

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        if self.test_override_outputs_p is not None:
            key = (x.size(0), x.size(1))
            if key in self.response_cache:
                x = self.response_cache[key]
            else:
                with torch.no_grad():
                    x.bernoulli_(self.test_override_outputs_p)
                    self.response_cache[key] = x
        return x


class MoeficationMoE(MoELayer):
    """The MoE-FFN layer (architectures/moe/moefication.py:28-101).

    ``forward(x[B,S,d]) -> (out[B,S,d], {name: (routing_tensor[B,S,E],)})`` with
    ``forward_mode`` in {'all','topk','dynk','dynk_max'}, ``tau``/``k`` read at call
    time.  In 'dynk_max' mode with a D2DMoE router the whole layer is one library call
    (router + rule -> bit mask -> token lists -> expert FFN with scatter-add); other
    modes compute the routing tensor with device tensor ops and share the rest.
    ``tau`` keeps the upstream meaning: expert e runs iff score_e >= max_e(score)*(1.0-tau).
    """

    def __init__(self, name, hidden_dim, num_experts, bias, expert_dim, activation,
                 experts_class="b200_kernel", add_residual_connection=False,
                 add_intermediate_gating=False):
        super().__init__(name, num_experts)
        self.hidden_dim = hidden_dim
        self.expert_dim = expert_dim
        self.num_experts = num_experts
        self.bias = bias
        if add_intermediate_gating and experts_class in ("execute_all", "module", "custom_kernel",
                                                         "b200_kernel"):
            experts_class = "b200_glu"
        if experts_class not in MOE_IMPL_MAP:
            raise NotImplementedError(
                f"experts_class={experts_class!r}: this package provides {sorted(MOE_IMPL_MAP)}")
        self.experts = MOE_IMPL_MAP[experts_class](dim=hidden_dim, num_experts=num_experts, depth=2,
                                                   expert_dim=self.expert_dim,
                                                   bias=False if not bias else "without_last",
                                                   activation=activation,
                                                   intermediate_gating=add_intermediate_gating)
        if self.bias:
            self.last_bias = nn.Parameter(torch.zeros(1, hidden_dim))
        self.forward_mode = "all"
        self.router = None
        self.k = None
        self.tau = None
        self.add_residual_connection = add_residual_connection
        self._wsp = _WorkspaceCache()

    # -- routing for the modes that are not fused ---------------------------------
    def gate(self, x):
        """Routing tensor [B,S,E] of 0/1 in the router's dtype for the non-fused modes
        (architectures/moe/moefication.py:54-88), on the device."""
        if self.forward_mode == "all":
            return torch.ones(x.size(0), x.size(1), self.num_experts, dtype=x.dtype,
                              device=x.device)
        if self.forward_mode in ("topk", "dynk", "dynk_max"):
            s = self.router(x)
            wsp = self._wsp.get(s.numel() // s.size(-1), self.num_experts, x.device)
            s2 = s.reshape(-1, s.size(-1)).contiguous()
            self._rule_mask(s2, wsp)
            return ops.expand_mask(wsp, s2.size(0), s2.size(1), s.dtype).view(s.shape)
        raise ValueError(f"Unsupported forward_mode: {self.forward_mode}")

    def _rule_mask(self, s2, wsp):
        """Mask bits of the current routing rule from scores [N, E], on the device."""
        if self.forward_mode == "topk":
            if not 1 <= int(self.k) <= s2.size(1):
                raise RuntimeError("selected index k out of range")       # as torch.topk
            ops.mask_rule_from_scores(s2, "topk", wsp, k=self.k)
        elif self.forward_mode == "dynk":
            ops.mask_rule_from_scores(s2, "dynk", wsp, tau=self.tau)
        else:
            ops.mask_from_scores(s2, self.tau, wsp)

    @torch.no_grad()
    def forward(self, x):
        if not x.is_cuda:
            raise RuntimeError("d2dmoe_b200 runs on CUDA tensors only (there is no CPU path)")
        self.experts._check_mode()
        orig_size = x.size()
        E = self.num_experts
        x2d = x.reshape(-1, x.size(-1)).contiguous()
        N = x2d.size(0)
        p = self.experts.kernel_params()
        last_bias = self.last_bias.view(-1) if self.bias else None
        out = torch.empty_like(x2d)
        wsp = self._wsp.get(N, E, x.device)
        capture = getattr(self.experts, "_capture", None) is not None
        fused = (self.forward_mode == "dynk_max" and self.router is not None and not capture
                 and isinstance(self.router, MoeficationRouter) and self.router.fusable())
        if N == 0:
            rt = torch.zeros(*orig_size[:-1], E, dtype=x.dtype, device=x.device)
            return out.view(orig_size), {self.name: (rt,)}
        if fused:
            wa, wb = self.router.layers[0].weight, self.router.layers[2].weight
            rt = torch.empty(N, E, dtype=x.dtype, device=x.device)
            ops.moe_forward(x2d, wa, wb, self.tau, p["w1"], p["b1"], p["w2"], p["act"], out, wsp,
                            w_up=p["w_up"], last_bias=last_bias,
                            add_residual=self.add_residual_connection,
                            router_packed=self.router.packed(),
                            experts_packed=self.experts.packed(), routing_out=rt)
            rt = rt.view(*orig_size[:-1], E)
        elif self.forward_mode == "dynk_max" and not capture:
            # any other router: its scores come from device tensor ops, the rule and the
            # rest of the layer from the library
            s = self.router(x)
            s2 = s.reshape(N, E).contiguous()
            rt = torch.empty(N, E, dtype=s.dtype, device=x.device)
            ops.moe_forward(x2d, None, None, self.tau, p["w1"], p["b1"], p["w2"], p["act"], out,
                            wsp, w_up=p["w_up"], scores=s2, last_bias=last_bias,
                            add_residual=self.add_residual_connection,
                            experts_packed=self.experts.packed(), routing_out=rt)
            rt = rt.view(*orig_size[:-1], E)
        elif self.forward_mode in ("topk", "dynk") and not capture:
            s = self.router(x)
            self._rule_mask(s.reshape(N, E).contiguous(), wsp)
            ops.compact(wsp, N, E)
            ops.experts_ffn(x2d, wsp, p["w1"], p["b1"], p["w2"], p["act"], out, w_up=p["w_up"],
                            packed=self.experts.packed(), last_bias=last_bias,
                            add_residual=self.add_residual_connection, accumulate=False)
            rt = ops.expand_mask(wsp, N, E, s.dtype).view(*orig_size[:-1], E)
        else:
            # mode 'all' (every expert on every token: router training), and any mode while
            # the experts capture their activation norms
            rt = self.gate(x)
            ops.pack_mask(rt.reshape(N, E).contiguous(), wsp)
            ops.compact(wsp, N, E)
            kw = self.experts._norm_args(N, x2d) if capture else {}
            ops.experts_ffn(x2d, wsp, p["w1"], p["b1"], p["w2"], p["act"], out, w_up=p["w_up"],
                            packed=self.experts.packed(), last_bias=last_bias,
                            add_residual=self.add_residual_connection, accumulate=False, **kw)
            if capture:
                self.experts._deliver_norms(kw)
        return out.view(orig_size), {self.name: (rt,)}

    # -- pre-norm + residual fused around the layer -----------------------------------
    @staticmethod
    def _norm_args(norm):
        """(kind, gamma, beta, eps, gamma_offset) of a normalisation module the fused pre-norm
        pass can evaluate, or None: nn.LayerNorm over the last dimension with affine
        parameters, torch's RMSNorm, and Gemma-style RMSNorm modules (weight applied as
        1 + weight, transformers GemmaRMSNorm)."""
        if isinstance(norm, nn.LayerNorm):
            if norm.weight is None or len(norm.normalized_shape) != 1:
                return None
            return ops.NORM_LAYER, norm.weight, norm.bias, float(norm.eps), 0.0
        name = type(norm).__name__
        if "RMSNorm" in name and getattr(norm, "weight", None) is not None:
            eps = getattr(norm, "eps", None)
            if eps is None:
                eps = getattr(norm, "variance_epsilon", None)
            if eps is None:
                eps = torch.finfo(norm.weight.dtype).eps
            return ops.NORM_RMS, norm.weight, None, float(eps), 1.0 if "Gemma" in name else 0.0
        return None

    @torch.no_grad()
    def forward_block(self, x, norm):
        """``x + self(norm(x))``: the second half of an upstream transformer block
        (architectures/moe/moe_models.py:69-76 ViT, :91-100 GPT, :148-156 Gemma:
        ``y = ln_2(x); y, gd = mlp(y); return x + y``) with the normalisation pass and the
        residual add folded into the layer: one pass reads x once and writes the normalised
        rows and ``x + last_bias`` as the output's initial value, and the layer adds the expert
        outputs to that.  Returns ``(x + out, {name: (routing_tensor,)})``.  Falls back to the
        three separate steps when the layer is not in its fused form."""
        na = self._norm_args(norm)
        # (affine parameters in another dtype than x -- mixed-precision norms -- keep the
        # framework's own normalisation: the fused pass computes in the dtype of x)
        fused = (na is not None and x.is_cuda and self.forward_mode == "dynk_max"
                 and na[1].dtype == x.dtype and (na[2] is None or na[2].dtype == x.dtype)
                 and na[1].device == x.device
                 and getattr(self.experts, "_capture", None) is None
                 and isinstance(self.router, MoeficationRouter) and self.router.fusable()
                 and not self.add_residual_connection
                 and (x.size(-1) * x.element_size()) % 16 == 0
                 and x.size(-1) * x.element_size() <= 8192 and x.numel() > 0)
        if not fused:
            y, gd = self.forward(norm(x))
            return x + y, gd
        self.experts._check_mode()
        kind, gamma, beta, eps, goff = na
        orig_size = x.size()
        E = self.num_experts
        x2d = x.reshape(-1, x.size(-1)).contiguous()
        N = x2d.size(0)
        p = self.experts.kernel_params()
        xn = torch.empty_like(x2d)
        out = torch.empty_like(x2d)
        rt = torch.empty(N, E, dtype=x.dtype, device=x.device)
        wsp = self._wsp.get(N, E, x.device)
        ops.prenorm_init(x2d, gamma.detach().contiguous(),
                         None if beta is None else beta.detach().contiguous(), eps, kind, xn, out,
                         last_bias=self.last_bias.view(-1) if self.bias else None,
                         gamma_offset=goff)
        ops.moe_forward(xn, self.router.layers[0].weight, self.router.layers[2].weight, self.tau,
                        p["w1"], p["b1"], p["w2"], p["act"], out, wsp, w_up=p["w_up"],
                        add_residual=ops.OUT_PREINITIALISED, router_packed=self.router.packed(),
                        experts_packed=self.experts.packed(), routing_out=rt)
        return out.view(orig_size), {self.name: (rt.view(*orig_size[:-1], E),)}

    @torch.no_grad()
    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor | None = None,
                     chunks: int = 4, sync: bool = True) -> torch.Tensor:
        """``forward`` for host-resident activations: x_host [B,S,d] (pinned) -> out_host
        (pinned), pipelined over ``chunks`` slices of the batch so that the host-to-device
        copy of slice i+1, the kernels of slice i and the device-to-host copy of slice i-1
        overlap (three streams, ordered by events).  Tokens are independent, so slicing the
        batch does not change any result.  Returns out_host.

        All layers of a device share the three streams, so with ``sync=False`` consecutive
        calls (other layers, the next batch) queue behind each other without draining the
        pipeline; ``out_host`` is then complete only after ``MoeficationMoE.host_synchronize``.
        With ``sync=True`` (default) the call returns when ``out_host`` is complete.
        """
        if x_host.is_cuda:
            raise ValueError("forward_host takes a host tensor; use forward() for device tensors")
        dev = self.experts.kernel_params()["w1"].device
        B = x_host.shape[0]
        if out_host is None:
            out_host = torch.empty_like(x_host).pin_memory()
        chunks = max(1, min(chunks, B))
        st = _HOST_STREAMS.get(dev)
        if st is None:
            st = tuple(torch.cuda.Stream(device=dev) for _ in range(3))
            _HOST_STREAMS[dev] = st
        s_in, s_run, s_out = st
        cur = torch.cuda.current_stream(dev)
        if sync:
            for s_ in st:
                s_.wait_stream(cur)
        bounds = [(B * i // chunks, B * (i + 1) // chunks) for i in range(chunks)]
        bufs = getattr(self, "_host_bufs", None)
        rows = max(hi - lo for lo, hi in bounds)
        shape = (rows,) + tuple(x_host.shape[1:])
        if bufs is None or bufs[0].shape != shape or bufs[0].dtype != x_host.dtype:
            # Copies and kernels of earlier sync=False calls may still use the old staging
            # buffers: drain the three streams before they go back to the allocator (a host
            # wait, but only when the slice shape changes), and allocate the new ones on the
            # copy stream that writes them, telling the allocator which stream reads them.
            for s_ in st:
                s_.synchronize()
            with torch.cuda.stream(s_in):
                bufs = [torch.empty(shape, dtype=x_host.dtype, device=dev) for _ in range(2)]
            for b in bufs:
                b.record_stream(s_run)
            self._host_bufs = bufs
            self._host_done = [None, None]
        done_run = self._host_done        # kernels that last read each buffer (kept across calls)
        for i, (lo, hi) in enumerate(bounds):
            xb = bufs[i & 1][: hi - lo]
            with torch.cuda.stream(s_in):
                if done_run[i & 1] is not None:
                    s_in.wait_event(done_run[i & 1])       # buffer still read by slice i-2
                xb.copy_(x_host[lo:hi], non_blocking=True)
                ev_in = s_in.record_event()
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in)
                out, _ = self.forward(xb)
                ev_run = s_run.record_event()
                done_run[i & 1] = ev_run
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run)
                out_host[lo:hi].copy_(out, non_blocking=True)
                out.record_stream(s_out)
        if sync:
            for s_ in st:
                cur.wait_stream(s_)
            cur.synchronize()
        return out_host

    @staticmethod
    def host_synchronize(device=None) -> None:
        """Wait until every ``forward_host(..., sync=False)`` issued on ``device`` is complete."""
        for dev, st in _HOST_STREAMS.items():
            if device is None or torch.device(device) == dev:
                for s_ in st:
                    s_.synchronize()

    def last_workspace(self, n: int, device) -> ops.Workspace:
        """The cached buffers of the last call with ``n`` tokens: bit mask, token lists,
        offsets and the device status word (for tests and diagnostics)."""
        return self._wsp.get(n, self.num_experts, device)


def fused_vit_block_forward(self, input: torch.Tensor):
    """Replacement for the upstream ``moe_vit_block_forward``
    (architectures/moe/moe_models.py:56-76; bind with ``functools.partial`` like upstream does,
    moefication.py:169-176): same computation and return value, with the FFN half run as
    ``mlp.forward_block(x, ln_2)`` when ``mlp`` is a layer of this package."""
    gating_data = {}
    x = self.ln_1(input)
    res = self.self_attention(query=x, key=x, value=x, need_weights=False)
    if len(res) == 3:                     # MoE-fied attention returns its gating data as well
        x, _, attn_gating_data = res
        gating_data.update(attn_gating_data)
    else:
        x, _ = res
    x = self.dropout(x)
    x = x + input
    if isinstance(self.mlp, MoeficationMoE):
        out, ffn_gating_data = self.mlp.forward_block(x, self.ln_2)
        gating_data.update(ffn_gating_data)
        return out, gating_data
    y = self.ln_2(x)
    if isinstance(self.mlp, MoELayer):
        y, ffn_gating_data = self.mlp(y)
        gating_data.update(ffn_gating_data)
    else:
        y = self.mlp(y)
    return x + y, gating_data


def _dropout_is_identity(module) -> bool:
    drop = getattr(module, "dropout", None)
    return drop is None or not drop.training or getattr(drop, "p", 0.0) == 0.0


def fused_gpt_block_forward(self, input: torch.Tensor):
    """Replacement for the upstream ``moe_gpt_block_forward``
    (architectures/moe/moe_models.py:78-100): same computation and return value, with
    ``h + dropout(mlp(ln_2(h)))`` run as ``mlp.forward_block(h, ln_2)`` when ``mlp`` is a layer of
    this package and its dropout is inactive (evaluation mode)."""
    gating_data = {}
    ln1 = self.ln_1(input)
    res = self.attn(query=ln1, key=ln1, value=ln1, need_weights=False) \
        if hasattr(self.attn, "in_proj_weight") or hasattr(self.attn, "q_proj") else self.attn(ln1)
    if isinstance(res, tuple) and len(res) == 3:     # MoE-fied attention: gating data as well
        attn_output, _, attn_gating_data = res
        gating_data.update(attn_gating_data)
    else:
        attn_output = res[0] if isinstance(res, tuple) else res
    h = input + attn_output
    if isinstance(self.mlp, MoeficationMoE) and _dropout_is_identity(self.mlp):
        out, ffn_gating_data = self.mlp.forward_block(h, self.ln_2)
        gating_data.update(ffn_gating_data)
        return out, gating_data
    ln2 = self.ln_2(h)
    if isinstance(self.mlp, MoELayer):
        mlp_out, ffn_gating_data = self.mlp(ln2)
        if hasattr(self.mlp, "dropout"):
            mlp_out = self.mlp.dropout(mlp_out)
        gating_data.update(ffn_gating_data)
    else:
        mlp_out = self.mlp(ln2)
    return h + mlp_out, gating_data


def fused_gemma_decoder_forward(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor,
                                position_ids: torch.Tensor, cache_position: torch.Tensor):
    """Replacement for the upstream ``moe_gemma_decoder_forward``
    (architectures/moe/moe_models.py:132-160): same computation and return value, with
    ``residual + mlp(post_attention_layernorm(residual))`` run as
    ``mlp.forward_block(residual, post_attention_layernorm)`` (RMSNorm with the 1 + weight
    scale, gated experts) when ``mlp`` is a layer of this package."""
    gating_data = {}
    residual = hidden_states
    hidden_states = self.input_layernorm(hidden_states)
    hidden_states, _w, _kv = self.self_attn(hidden_states=hidden_states,
                                            attention_mask=attention_mask,
                                            position_ids=position_ids,
                                            cache_position=cache_position)
    hidden_states = residual + hidden_states
    if isinstance(self.mlp, MoeficationMoE):
        out, ffn_gating_data = self.mlp.forward_block(hidden_states, self.post_attention_layernorm)
        gating_data.update(ffn_gating_data)
        return out, gating_data
    residual = hidden_states
    hidden_states = self.post_attention_layernorm(hidden_states)
    if isinstance(self.mlp, MoELayer):
        hidden_states, ffn_gating_data = self.mlp(hidden_states)
        gating_data.update(ffn_gating_data)
    else:
        hidden_states = self.mlp(hidden_states)
    return residual + hidden_states, gating_data


class _NormCaptureHandle:
    """What add_save_output_norm_hook returns per module: ``remove()`` like a torch hook handle."""

    def __init__(self, experts, sink):
        self._experts, self._sink = experts, sink

    def remove(self):
        if self._sink in self._experts._norm_sinks:
            self._experts._norm_sinks.remove(self._sink)
        if not self._experts._norm_sinks:
            self._experts.capture_norms(None)


def add_save_output_norm_hook(model, module_names, ord, dim=-1):
    """Same contract as the upstream helper (utils.py:353-369): returns ``(saved, handles)``;
    after each forward of ``model``, ``saved[name]`` holds
    ``torch.linalg.vector_norm(output of module name, ord=ord, dim=dim)``.  For the modules
    router training names inside an experts layer of this package -- the two extraction stubs
    of B200KernelExperts, ``layers[0]`` / ``layers[1]`` of B200GluExperts
    (methods/dynamic_sparsification/train_routers.py:49-71) -- the [E, N] norms come out of the
    expert kernel itself; any other module gets an ordinary forward hook."""
    saved, handles = {}, []
    for name in module_names:
        module = model.get_submodule(name)
        parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
        experts, layer = None, None
        if isinstance(parent, B200KernelExperts):
            if module is getattr(parent, "intermediate_activation_extraction_stub", None):
                experts, layer = parent, "intermediate"
            elif module is getattr(parent, "output_activation_extraction_stub", None):
                experts, layer = parent, "output"
        elif isinstance(parent, nn.ModuleList) and name.count(".") >= 1:
            owner_name = name.rsplit(".", 2)[0] if name.count(".") >= 2 else ""
            owner = model.get_submodule(owner_name) if owner_name else model
            if isinstance(owner, B200GluExperts) and parent is owner.layers:
                idx = int(name.rsplit(".", 1)[1])
                if idx in (0, 1):
                    experts, layer = owner, ("intermediate", "output")[idx]
        if experts is None:
            def save_norm_hook(m, _input, output, _name=name):
                saved[_name] = torch.linalg.vector_norm(output, ord=ord, dim=dim)
            handles.append(module.register_forward_hook(save_norm_hook))
            continue
        if dim != -1:
            raise NotImplementedError("the expert kernel takes norms over the last dimension")
        if experts._capture is not None and experts._capture != (layer, int(ord)):
            raise NotImplementedError("one captured layer / ord per experts module at a time")
        experts.capture_norms(layer, ord)
        sink = (saved, name)
        experts._norm_sinks.append(sink)
        handles.append(_NormCaptureHandle(experts, sink))
    return saved, handles


def bind_upstream(moe_layers=None) -> bool:
    """Make these classes first-class citizens of the upstream code base when this package is
    used inside it.  The upstream block and attention forwards decide with
    ``isinstance(module, MoELayer)`` whether a sub-module returns ``(out, gating_data)``
    (architectures/moe/moe_models.py:20-46,71,93,150), and ``replace_with_moes`` builds experts
    from ``MOE_IMPL_MAP[experts_class]`` (architectures/moe/moefication.py:39,157-167).  This
    re-bases ``MoELayer`` / ``ExpertsLayer`` here onto the upstream classes of the same name and
    registers ``'b200_kernel'`` / ``'b200_glu'`` in the upstream map, so that a layer of this
    package dropped into an upstream model is dispatched exactly like an upstream one (FFN
    blocks and MoE-fied q/k/v/o attention projections alike).

    ``moe_layers``: the upstream module ``architectures.moe.moe_layers`` (imported here when
    None).  Returns False when the upstream package cannot be imported.  Called automatically at
    import when the upstream module is already loaded."""
    if moe_layers is None:
        try:
            import importlib
            moe_layers = importlib.import_module("architectures.moe.moe_layers")
        except Exception:      # noqa: BLE001  (not inside the upstream tree)
            return False
    up_moe, up_experts = moe_layers.MoELayer, moe_layers.ExpertsLayer
    if up_moe not in MoELayer.__mro__:
        MoELayer.__bases__ = (up_moe,)
    if up_experts not in ExpertsLayer.__mro__:
        ExpertsLayer.__bases__ = (up_experts,)
    moe_layers.MOE_IMPL_MAP.setdefault("b200_kernel", B200KernelExperts)
    moe_layers.MOE_IMPL_MAP.setdefault("b200_glu", B200GluExperts)
    return True


def add_routers(model: nn.Module, router_args: dict) -> dict:
    """Attach a MoeficationRouter to every MoeficationMoE of ``model``
    (architectures/moe/moefication.py:342-354)."""
    found = {}
    for name, m in model.named_modules():
        if isinstance(m, MoeficationMoE):
            m.router = MoeficationRouter(m.hidden_dim, m.num_experts, **router_args)
            found[name] = m
    assert len(found) > 0
    return found


import sys as _sys      # noqa: E402

if "architectures.moe.moe_layers" in _sys.modules:
    bind_upstream(_sys.modules["architectures.moe.moe_layers"])
