"""d2d_compact_noalloc: the compaction entry point for callers that cannot allocate.

Some hosts of the library can pass only an operator's inputs and outputs, or run with
a memory pool that is frozen after start-up, so they have no workspace to give to
d2d_compact.  d2d_compact_noalloc keeps its counts table in a fixed array inside the
library instead.  This file checks, through the C ABI, that it produces exactly the
token lists and offsets of d2d_compact, on two calls in a row that share the array
(the second smaller than the first, so stale table contents would show), and that a
request beyond the array's capacity is refused.  It is collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest
import torch


def _run(lib, fn_noalloc, mask_bits, N, E):
    """Returns (offsets, token_idx) from d2d_compact and from d2d_compact_noalloc."""
    from d2dmoe_b200 import ops
    wsp = ops.Workspace.allocate(N, E, "cuda")
    wsp.mask_bits.copy_(mask_bits)
    p = lambda t: C.c_void_p(t.data_ptr())                               # noqa: E731
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ops.compact(wsp, N, E)
    off_a = wsp.offsets.clone()
    idx_a = wsp.token_idx.clone()
    off_b = torch.full_like(off_a, -1)
    idx_b = torch.full_like(idx_a, -1)
    rc = lib.d2d_compact_noalloc(p(wsp.mask_bits), p(idx_b), p(off_b), N, E, p(wsp.status), stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    wsp.check_status()
    total = int(off_a[E].item())
    return (off_a.cpu().numpy(), idx_a[:total].cpu().numpy()), (off_b.cpu().numpy(), idx_b[:total].cpu().numpy())


@pytest.mark.gpu
def test_noalloc_matches_workspace_entry_point_twice():
    from d2dmoe_b200 import _capi
    lib = _capi.lib
    g = torch.Generator().manual_seed(7)
    for N, E, p in ((50432, 24, 0.07), (3001, 96, 0.3)):      # second call: smaller table
        m = torch.rand(N, E, generator=g) < p
        nw = (E + 31) // 32
        words = np.zeros((N, nw), dtype=np.uint32)
        mm = m.numpy().astype(np.uint32)
        for e in range(E):
            words[:, e // 32] |= mm[:, e] << np.uint32(e % 32)
        bits = torch.from_numpy(words.view(np.int32)).cuda()
        (off_a, idx_a), (off_b, idx_b) = _run(lib, None, bits, N, E)
        assert np.array_equal(off_a, off_b)
        assert np.array_equal(idx_a, idx_b)                  # integer work: bit-exact
        assert off_a[E] == int(m.sum())
        for e in (0, E // 2, E - 1):                         # and both are the true lists
            assert np.array_equal(idx_b[off_b[e]:off_b[e + 1]],
                                  torch.nonzero(m[:, e]).flatten().numpy())
    # no tokens at all, right after calls that left the shared table full of counts:
    # every list is empty, so all E+1 offsets are zero and nothing is reported
    off = torch.full((E + 1,), 5, dtype=torch.int32, device="cuda")
    idx = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())                               # noqa: E731
    rc = lib.d2d_compact_noalloc(p(bits), p(idx), p(off), 0, E, p(status),
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0 and int(off.abs().sum()) == 0 and int(status.item()) == 0


def test_noalloc_rejects_sizes_beyond_its_table():
    from d2dmoe_b200 import _capi
    lib = _capi.lib
    one = C.c_void_p(16)      # never dereferenced: the size check comes first
    # ceil(N/128) * E = 8200 * 64 > 262144
    assert lib.d2d_compact_noalloc(one, one, one, 1025 * 1024, 64, None, None) == 8
    assert b"scratch" in lib.d2d_strerror(8)
    assert lib.d2d_compact_noalloc(None, one, one, 10, 4, None, None) == 1
