"""The C restatement of the integer stages against the upstream fixtures and the Python oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import O, all_cases, case_ids, golden_mask, golden_scores, load_golden
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
