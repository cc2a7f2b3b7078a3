"""ctypes binding of the C ABI declared in include/d2dmoe.h.

The library is looked up in-tree (d2dmoe_b200/_lib).  There is no fallback: if it
is missing or does not load, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libd2dmoe_b200.so"

F32, BF16 = 0, 1
ACT = {"relu": 0, "gelu": 1, "tanh": 2, "leaky_relu": 3, "gelu_tanh": 4}

OK = 0
STATUS_NAMES = {0: "OK", 1: "BAD_ARG", 2: "UNSUPPORTED", 3: "LAUNCH", 4: "WORKSPACE",
                5: "INDEX_RANGE", 6: "TIMEOUT", 7: "NO_DEVICE", 8: "SCRATCH_LIMIT"}

_p, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes): must list every function of include/d2dmoe.h
SIGNATURES = {
    "d2d_abi_version": (_i, []),
    "d2d_strerror": (C.c_char_p, [_i]),
    "d2d_workspace_bytes": (_i, [_i64, _i, C.POINTER(_sz)]),
    "d2d_router_mask": (_i, [_p, _p, _p, _p, _f, _p, _p, _p, _i, _p, _i64, _i, _i, _i, _i, _p, _p]),
    "d2d_mask_from_scores": (_i, [_p, _f, _p, _i64, _i, _i, _p, _p]),
    "d2d_last_forward_launches": (_i, []),
    "d2d_debug_configure": (_i, [_i, _i]),
    "d2d_debug_select_experts_kernel": (_i, [_i]),
    "d2d_mask_rule_from_scores": (_i, [_p, _i, _i, _f, _p, _i64, _i, _i, _p, _p]),
    "d2d_init_out": (_i, [_p, _p, _i, _p, _i64, _i, _i, _p]),
    "d2d_expand_mask": (_i, [_p, _p, _i64, _i, _i, _p]),
    "d2d_prenorm_init": (_i, [_p, _p, _p, _f, _i, _f, _p, _p, _p, _i64, _i, _i, _p]),
    "d2d_pack_mask": (_i, [_p, _p, _i64, _i, _i, _p]),
    "d2d_compact": (_i, [_p, _p, _p, _i64, _i, _p, _sz, _p, _p]),
    "d2d_compact_noalloc": (_i, [_p, _p, _p, _i64, _i, _p, _p]),
    "d2d_experts_ffn": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p,
                             _i64, _i, _i, _i, _i, _i, _p, _p]),
    "d2d_experts_ffn_norms": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p, _p, _i, _i,
                                   _i64, _i, _i, _i, _i, _i, _p, _p]),
    "d2d_moe_forward": (_i, [_p, _p, _p, _p, _p, _f, _p, _p, _p, _p, _p, _p, _i, _p,
                             _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _p, _sz, _p, _p, _p]),
    "d2d_prepack_experts_bytes": (_i, [_i, _i, _i, _i, _i, C.POINTER(_sz)]),
    "d2d_prepack_experts": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "d2d_prepack_router_bytes": (_i, [_i, _i, _i, _i, C.POINTER(_sz)]),
    "d2d_prepack_router": (_i, [_p, _p, _p, _i, _i, _i, _i, _p]),
}


class D2DError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib.d2d_strerror(code).decode() if "lib" in globals() else str(code)
        super().__init__(f"{where}: {STATUS_NAMES.get(code, code)} ({msg})")


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python d2dmoe_b200/build.py` "
            "(this package has no non-CUDA path)")
    cdll = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(cdll, name)          # AttributeError if the library lacks a symbol
        fn.restype = res
        fn.argtypes = args
    return cdll


lib = _load()
if lib.d2d_abi_version() != 2:
    raise ImportError("libd2dmoe_b200.so: ABI version mismatch")


def check(code: int, where: str) -> None:
    if code != OK:
        raise D2DError(code, where)
