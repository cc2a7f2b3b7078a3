"""The C restatement of the integer stages against the upstream fixtures and the Python oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import (O, WINDOW, all_cases, case_ids, gate_fixture_ids, gate_fixture_items,
                     golden_mask, golden_scores, load_golden, rule_tie_tokens)
from oracle.build_c import build


@pytest.fixture(scope="module")
def lib():
    l = C.CDLL(str(build()))
    l.d2d_oracle_compact.restype = C.c_long
    return l


@pytest.mark.parametrize("c", all_cases(), ids=case_ids())
def test_c_rule_and_lists_match_upstream(lib, c):
    g, t = load_golden(c)
    s = golden_scores(g, c).reshape(c.N, c.E).contiguous()
    nw = (c.E + 31) // 32
    bits = np.zeros((c.N, nw), dtype=np.uint32)
    mult = C.c_float(O.threshold_multiplier(c.tau))
    if c.dtype == "fp32":
        a = s.numpy()
        lib.d2d_oracle_mask_f32(a.ctypes.data_as(C.c_void_p), mult, bits.ctypes.data_as(C.c_void_p),
                                C.c_long(c.N), c.E)
    else:
        a = s.view(torch.int16).numpy().view(np.uint16)
        lib.d2d_oracle_mask_bf16(a.ctypes.data_as(C.c_void_p), mult,
                                 bits.ctypes.data_as(C.c_void_p), C.c_long(c.N), c.E)
    assert np.array_equal(bits, g["mask_bits"])          # bit-exact with the upstream routing tensor
    off = np.zeros(c.E + 1, dtype=np.int32)
    idx = np.zeros(c.N * c.E, dtype=np.int32)
    total = lib.d2d_oracle_compact(bits.ctypes.data_as(C.c_void_p), C.c_long(c.N), c.E,
                                   off.ctypes.data_as(C.c_void_p), idx.ctypes.data_as(C.c_void_p))
    roff, ridx = O.expert_token_lists(golden_mask(g, c))
    assert total == len(ridx) and np.array_equal(off, roff) and np.array_equal(idx[:total], ridx)


@pytest.mark.parametrize("item", gate_fixture_items(), ids=gate_fixture_ids())
def test_c_topk_and_dynk_rules_match_upstream_gate(lib, item):
    """C restatement of the 'topk' / cumulative 'dynk' rules against the routing tensors the
    upstream gate returned: equal on every token outside the tie window (members of a group
    of equal scores are interchangeable upstream)."""
    c, rule, par, ref_bits = item
    g, _ = load_golden(c)
    s = golden_scores(g, c).reshape(c.N, c.E).contiguous()
    nw = (c.E + 31) // 32
    bits = np.zeros((c.N, nw), dtype=np.uint32)
    r, k, tau = (1, int(par), 0.0) if rule == "topk" else (2, 0, float(par))
    if c.dtype == "fp32":
        a = s.numpy()
        lib.d2d_oracle_rule_f32(a.ctypes.data_as(C.c_void_p), r, k, C.c_float(tau),
                                bits.ctypes.data_as(C.c_void_p), C.c_long(c.N), c.E)
    else:
        a = s.view(torch.int16).numpy().view(np.uint16)
        lib.d2d_oracle_rule_bf16(a.ctypes.data_as(C.c_void_p), r, k, C.c_float(tau),
                                 bits.ctypes.data_as(C.c_void_p), C.c_long(c.N), c.E)
    m, ref = O.unpack_mask(bits, c.E), O.unpack_mask(ref_bits, c.E)
    bad = (m != ref).any(-1)
    tie = rule_tie_tokens(s, rule, par, WINDOW[c.dtype], ref)
    assert (bad & ~tie).sum().item() == 0
