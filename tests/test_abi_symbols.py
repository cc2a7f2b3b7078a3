"""The shared library loads and exports every function include/d2dmoe.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "d2dmoe.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(d2d_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("d2d_router_mask", "d2d_mask_from_scores", "d2d_compact", "d2d_experts_ffn",
                 "d2d_moe_forward", "d2d_expand_mask", "d2d_strerror", "d2d_abi_version"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from d2dmoe_b200 import _capi
    cdll = ctypes.CDLL(str(_capi.LIB_PATH))
    for name in declared_functions():
        assert hasattr(cdll, name), f"{name} declared in d2dmoe.h but not exported"
        assert name in _capi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_capi.SIGNATURES) == set(declared_functions())


def test_host_only_entry_points():
    from d2dmoe_b200 import _capi
    assert _capi.lib.d2d_abi_version() == 2
    assert _capi.lib.d2d_strerror(0) == b"ok"
    assert b"workspace" in _capi.lib.d2d_strerror(4)
    n = ctypes.c_size_t(0)
    assert _capi.lib.d2d_workspace_bytes(50432, 24, ctypes.byref(n)) == 0
    assert n.value >= 50 * 24 * 4 and n.value % 256 == 0
    assert _capi.lib.d2d_workspace_bytes(-1, 24, ctypes.byref(n)) == 1      # BAD_ARG
    # null pointers are rejected on the host before anything is launched
    assert _capi.lib.d2d_compact(None, None, None, 10, 4, None, 0, None, None) == 1
    assert _capi.lib.d2d_mask_from_scores(None, 0.5, None, 10, 4, 0, None, None) == 1


def test_misaligned_buffers_are_rejected_before_any_launch():
    """x / out that do not start on a 16-byte boundary (a view with a storage offset) must be
    refused on the host with BAD_ARG: the checks of every stage run before the first launch,
    so nothing is enqueued.  The pointers are never dereferenced on the host."""
    import ctypes as C
    from d2dmoe_b200 import _capi
    lib = _capi.lib
    a = lambda v: C.c_void_p(v)                                             # noqa: E731
    base, ws = 0x7f0000000000, 0x7f0000100000
    good = dict(x=a(base), out=a(base + 0x10000))
    for bad in ("x", "out"):
        ptrs = dict(good)
        ptrs[bad] = a(ptrs[bad].value + 2)
        rc = lib.d2d_moe_forward(ptrs["x"], a(base), a(base), a(ws), None, 0.9, a(base), a(base),
                                 None, a(base), a(ws), None, 0, ptrs["out"], a(base), a(base),
                                 a(base), 256, 768, 128, 24, 128, 0, 1, a(ws), 1 << 20, None, None, None)
        assert rc == 1, (bad, rc)
    # experts entry point alone
    rc = lib.d2d_experts_ffn(a(base + 2), a(base), a(base), a(base), None, None, a(base), None,
                             None, 0, 1, a(base), 256, 768, 24, 128, 0, 1, None, None)
    assert rc == 1
    assert lib.d2d_debug_configure(0, 0) == 0


def test_argument_checks_of_the_block_level_and_label_entry_points():
    """d2d_prenorm_init and d2d_experts_ffn_norms refuse bad arguments on the host before any
    CUDA call (the pointers below are never dereferenced)."""
    import ctypes as C
    from d2dmoe_b200 import _capi
    lib = _capi.lib
    a = lambda v: C.c_void_p(v)                                             # noqa: E731
    base = 0x7f0000000000
    # labels: ord must be 1 or 2, the layer 1 or 2, the norms buffer present
    args = lambda norms, layer, ordv: (a(base), a(base), a(base), a(base), None, None, a(base),  # noqa: E731
                                       None, None, 0, 1, a(base), norms, layer, ordv,
                                       256, 768, 24, 128, 0, 1, None, None)
    assert lib.d2d_experts_ffn_norms(*args(a(base), 2, 3)) == 1
    assert lib.d2d_experts_ffn_norms(*args(a(base), 3, 2)) == 1
    assert lib.d2d_experts_ffn_norms(*args(a(base), 0, 2)) == 1
    assert lib.d2d_experts_ffn_norms(*args(None, 2, 2)) == 1
    # pre-norm: rows longer than 8 KB or not a multiple of 16 bytes are unsupported, pointers
    # must be 16-byte aligned
    pn = lambda x, d: lib.d2d_prenorm_init(x, a(base), None, 1e-6, 0, 0.0, None, a(base),   # noqa: E731
                                           a(base), 16, d, 1, None)
    assert pn(a(base), 8200) == 2                       # D2D_ERR_UNSUPPORTED
    assert pn(a(base), 100) == 2
    assert pn(a(base + 2), 768) == 1                    # D2D_ERR_BAD_ARG
