"""Tensor-level wrappers over the C ABI (include/d2dmoe.h).

PyTorch owns device memory and streams; every function here only checks its
arguments, takes ``tensor.data_ptr()`` and the current stream's handle, and calls
the library.  CUDA tensors only: a CPU tensor raises.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _capi
from ._capi import ACT, BF16, F32, check, lib

_DT = {torch.float32: F32, torch.bfloat16: BF16}


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise TypeError(f"d2dmoe_b200 supports float32 and bfloat16, got {t.dtype}")
    return _DT[t.dtype]


def _cu(*ts):
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("d2dmoe_b200 runs on CUDA tensors only (there is no CPU path)")
        if not t.is_contiguous():
            raise ValueError("d2dmoe_b200 needs contiguous tensors")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors of one call live on different devices: {dev} and {t.device}")


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class _on:
    """Make the device of ``t`` current for a library call (kernels launch on the current
    device) and hand out that device's current stream.  A no-op when it is current already."""

    __slots__ = ("dev", "ctx")

    def __init__(self, t):
        self.dev = t.device if isinstance(t, torch.Tensor) else torch.device(t)
        self.ctx = None

    def __enter__(self):
        if self.dev.index is not None and self.dev.index != torch.cuda.current_device():
            self.ctx = torch.cuda.device(self.dev)
            self.ctx.__enter__()
        return C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)
        return False


def threshold_multiplier(tau: float) -> float:
    """(1.0 - tau) evaluated in double and narrowed to fp32, as the tensor-scalar
    multiply of architectures/moe/moefication.py:83 does."""
    return float(np.float32(1.0 - float(tau)))


def workspace_bytes(n: int, E: int) -> int:
    out = C.c_size_t(0)
    check(lib.d2d_workspace_bytes(n, E, C.byref(out)), "d2d_workspace_bytes")
    return out.value


@dataclass
class Workspace:
    """Caller-owned buffers of one layer call for up to ``n`` tokens and ``E`` experts."""
    n: int
    E: int
    mask_bits: torch.Tensor      # [n, ceil(E/32)] int32 (bit pattern of u32 words)
    token_idx: torch.Tensor      # [n*E] int32
    offsets: torch.Tensor        # [E+1] int32
    ws: torch.Tensor             # bytes
    status: torch.Tensor         # [1] int32 device status word

    @staticmethod
    def allocate(n: int, E: int, device) -> "Workspace":
        nw = (E + 31) // 32
        i32 = dict(dtype=torch.int32, device=device)
        return Workspace(
            n, E,
            torch.empty(max(n, 1), nw, **i32),
            torch.empty(max(n * E, 1), **i32),
            torch.zeros(E + 1, **i32),
            torch.empty(max(workspace_bytes(n, E), 256), dtype=torch.uint8, device=device),
            torch.zeros(1, **i32),
        )

    def check_status(self) -> None:
        """Read the device status word (synchronises): raise if a kernel reported."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise _capi.D2DError(code, "device status")


def router_mask(x2d, wa, wb, tau, wsp: Workspace, *, packed=None, scores_out=None,
                last_bias=None, add_residual=False, out_init=None):
    _cu(x2d, wa, wb, packed, scores_out, last_bias, out_init)
    N, d = x2d.shape
    R, E = wa.shape[0], wb.shape[0]
    with _on(x2d) as st:
        check(lib.d2d_router_mask(_ptr(x2d), _ptr(wa), _ptr(wb), _ptr(packed),
                                  threshold_multiplier(tau), _ptr(wsp.mask_bits), _ptr(scores_out),
                                  _ptr(last_bias), int(add_residual), _ptr(out_init),
                                  N, d, R, E, _dt(x2d), _ptr(wsp.status), st),
              "d2d_router_mask")


RULE_TOPK, RULE_DYNK = 1, 2


def mask_rule_from_scores(scores2d, rule: str, wsp: Workspace, k=None, tau=None):
    """Mask bits for the 'topk' / 'dynk' (cumulative share) rules of the upstream gate
    (architectures/moe/moefication.py:59-79) on given scores [N, E]."""
    _cu(scores2d)
    N, E = scores2d.shape
    if rule == "topk":
        r, kk, tt = RULE_TOPK, int(k), 0.0
    elif rule == "dynk":
        r, kk, tt = RULE_DYNK, 0, float(tau)
    else:
        raise ValueError(f"unknown rule {rule!r}")
    with _on(scores2d) as st:
        check(lib.d2d_mask_rule_from_scores(_ptr(scores2d), r, kk, tt, _ptr(wsp.mask_bits), N, E,
                                            _dt(scores2d), _ptr(wsp.status), st),
              "d2d_mask_rule_from_scores")


def mask_from_scores(scores2d, tau, wsp: Workspace):
    _cu(scores2d)
    N, E = scores2d.shape
    with _on(scores2d) as st:
        check(lib.d2d_mask_from_scores(_ptr(scores2d), threshold_multiplier(tau),
                                       _ptr(wsp.mask_bits), N, E, _dt(scores2d), _ptr(wsp.status),
                                       st), "d2d_mask_from_scores")


def pack_mask(routing2d, wsp: Workspace):
    _cu(routing2d)
    N, E = routing2d.shape
    with _on(routing2d) as st:
        check(lib.d2d_pack_mask(_ptr(routing2d), _ptr(wsp.mask_bits), N, E, _dt(routing2d), st),
              "d2d_pack_mask")


def expand_mask(wsp: Workspace, N: int, E: int, dtype) -> torch.Tensor:
    rt = torch.empty(N, E, dtype=dtype, device=wsp.mask_bits.device)
    with _on(rt) as st:
        check(lib.d2d_expand_mask(_ptr(wsp.mask_bits), _ptr(rt), N, E, _DT[dtype], st),
              "d2d_expand_mask")
    return rt


def init_out(x2d, last_bias, add_residual, out):
    _cu(x2d, last_bias, out)
    N, d = out.shape
    with _on(out) as st:
        check(lib.d2d_init_out(_ptr(x2d), _ptr(last_bias), int(add_residual), _ptr(out), N, d,
                               _dt(out), st), "d2d_init_out")


NORM_LAYER, NORM_RMS = 0, 1
OUT_PREINITIALISED = 2      # add_residual value: ``out`` already holds its initial value


def prenorm_init(x2d, gamma, beta, eps: float, kind: int, xn, out_init=None, *, last_bias=None,
                 gamma_offset: float = 0.0):
    """One pass over x: ``xn = norm(x)`` (the layer's input) and ``out_init = x + last_bias``
    (the block's residual as the layer output's initial value).  Raises D2DError UNSUPPORTED for
    rows longer than 8192 bytes or not a multiple of 16 bytes."""
    _cu(x2d, gamma, beta, last_bias, xn, out_init)
    N, d = x2d.shape
    with _on(x2d) as st:
        check(lib.d2d_prenorm_init(_ptr(x2d), _ptr(gamma), _ptr(beta), float(eps), int(kind),
                                   float(gamma_offset), _ptr(last_bias), _ptr(xn), _ptr(out_init),
                                   N, d, _dt(x2d), st), "d2d_prenorm_init")


def compact(wsp: Workspace, N: int, E: int):
    with _on(wsp.mask_bits) as st:
        check(lib.d2d_compact(_ptr(wsp.mask_bits), _ptr(wsp.token_idx), _ptr(wsp.offsets), N, E,
                              _ptr(wsp.ws), wsp.ws.numel(), _ptr(wsp.status), st),
              "d2d_compact")


NORM_OF = {"intermediate": 1, "output": 2}


def experts_ffn(x2d, wsp: Workspace, w1, b1, w2, act: str, out, *, w_up=None, packed=None,
                last_bias=None, add_residual=False, accumulate=False, norms=None,
                norm_layer="output", norm_ord=2):
    """Grouped expert FFN over the token lists in ``wsp`` with scatter-add into ``out``.
    ``norms`` [E, N] (optional, dtype of x) receives the vector norm (``norm_ord`` 1 or 2) of
    every computed pair's ``norm_layer`` ('intermediate' | 'output') activations: the labels
    router training captures upstream (utils.py:353-369)."""
    _cu(x2d, w1, b1, w2, w_up, packed, last_bias, out, wsp.token_idx, norms)
    N, d = x2d.shape
    E, _, H = w1.shape
    with _on(x2d) as st:
        if norms is None:
            check(lib.d2d_experts_ffn(_ptr(x2d), _ptr(wsp.token_idx), _ptr(wsp.offsets), _ptr(w1),
                                      _ptr(b1), _ptr(w_up), _ptr(w2), _ptr(packed), _ptr(last_bias),
                                      int(add_residual), int(accumulate), _ptr(out), N, d, E, H,
                                      ACT[act], _dt(x2d), _ptr(wsp.status), st), "d2d_experts_ffn")
        else:
            if norms.shape != (E, N) or norms.dtype != x2d.dtype or not norms.is_contiguous():
                raise ValueError("norms must be a contiguous [E, N] tensor of x's dtype")
            check(lib.d2d_experts_ffn_norms(
                _ptr(x2d), _ptr(wsp.token_idx), _ptr(wsp.offsets), _ptr(w1), _ptr(b1), _ptr(w_up),
                _ptr(w2), _ptr(packed), _ptr(last_bias), int(add_residual), int(accumulate),
                _ptr(out), _ptr(norms), NORM_OF[norm_layer], int(norm_ord), N, d, E, H, ACT[act],
                _dt(x2d), _ptr(wsp.status), st), "d2d_experts_ffn_norms")


def moe_forward(x2d, wa, wb, tau, w1, b1, w2, act: str, out, wsp: Workspace, *, w_up=None,
                scores=None, last_bias=None, add_residual=False, router_packed=None,
                experts_packed=None, routing_out=None):
    """Whole layer in one library call: router+mask (or mask from ``scores``) ->
    compaction -> expert FFN with scatter-add into ``out``.  ``routing_out`` [N, E]
    (optional) receives the 0/1 routing tensor."""
    _cu(x2d, wa, wb, w1, b1, w2, w_up, scores, last_bias, out, router_packed, experts_packed,
        wsp.mask_bits, routing_out)
    N, d = x2d.shape
    E, _, H = w1.shape
    R = wa.shape[0] if wa is not None else 0
    with _on(x2d) as st:
        check(lib.d2d_moe_forward(_ptr(x2d), _ptr(wa), _ptr(wb), _ptr(router_packed), _ptr(scores),
                                  threshold_multiplier(tau), _ptr(w1), _ptr(b1), _ptr(w_up),
                                  _ptr(w2), _ptr(experts_packed), _ptr(last_bias),
                                  int(add_residual), _ptr(out), _ptr(wsp.mask_bits),
                                  _ptr(wsp.token_idx), _ptr(wsp.offsets), N, d, R, E, H, ACT[act],
                                  _dt(x2d), _ptr(wsp.ws), wsp.ws.numel(), _ptr(wsp.status),
                                  _ptr(routing_out), st),
              "d2d_moe_forward")


def prepack_experts(w1, b1, w2, w_up=None):
    """Packed tile images of the expert weights for the tensor-core kernel, or None
    when the shape/dtype has no tensor-core path."""
    _cu(w1, b1, w2, w_up)
    E, d, H = w1.shape
    n = C.c_size_t(0)
    check(lib.d2d_prepack_experts_bytes(d, E, H, int(w_up is not None), _dt(w1), C.byref(n)),
          "d2d_prepack_experts_bytes")
    if n.value == 0:
        return None
    buf = torch.empty(n.value + 1024, dtype=torch.uint8, device=w1.device)
    off = (-buf.data_ptr()) % 1024
    packed = buf[off:off + n.value]
    with _on(w1) as st:
        check(lib.d2d_prepack_experts(_ptr(w1), _ptr(b1), _ptr(w_up), _ptr(w2), _ptr(packed), d, E,
                                      H, _dt(w1), st), "d2d_prepack_experts")
    return packed


def prepack_router(wa, wb):
    _cu(wa, wb)
    R, d = wa.shape
    E = wb.shape[0]
    n = C.c_size_t(0)
    check(lib.d2d_prepack_router_bytes(d, R, E, _dt(wa), C.byref(n)), "d2d_prepack_router_bytes")
    if n.value == 0:
        return None
    buf = torch.empty(n.value + 1024, dtype=torch.uint8, device=wa.device)
    off = (-buf.data_ptr()) % 1024
    packed = buf[off:off + n.value]
    with _on(wa) as st:
        check(lib.d2d_prepack_router(_ptr(wa), _ptr(wb), _ptr(packed), d, R, E, _dt(wa), st),
              "d2d_prepack_router")
    return packed
