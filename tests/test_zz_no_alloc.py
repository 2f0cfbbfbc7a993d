"""The allocation-free entry point `intra_b200_fwd_llm_noalloc` against the regular one.

For hosts that keep all of HBM in their own arena (a library-side cudaMalloc would fail or stall
them) the library offers one launch path whose scratch is a fixed array inside the library image.
This test calls it through the C ABI twice in a row - the second call reuses the array the first one
left behind - and checks both outputs against `intra_b200_fwd_llm` on the same inputs. It lives in a
file that sorts last so that a run stopping at the first failure has already run everything else; it
needs nothing from the other tests and also passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

from oracle import intra_oracle as oracle
from tests import _util

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, q, k, v, pattern, group_num, window, prev=None):
    out = torch.empty_like(q)
    B, S, H, D = q.shape
    rc = lib.intra_b200_fwd_llm_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, H, k.shape[2],
        _util.strides3(q), _util.strides3(k), _util.strides3(v), _util.strides3(out),
        _util.PATTERN_ID[("llm", pattern)], group_num, window, D ** -0.5, q.device.index,
        torch.cuda.current_stream(q.device).cuda_stream, prev)
    return rc, out


def test_noalloc_matches_regular_entry_point_twice(lib):
    assert torch.cuda.is_available()
    q, k, v = oracle.make_inputs(2, 1500, 8, 2, seed=31, device="cuda")
    q2, k2, v2 = oracle.make_inputs(1, 2048, 4, 4, seed=32, device="cuda")

    prev = ctypes.c_int(-1)
    rc, out_a = _call_noalloc(lib, q, k, v, "scatter", 3, 576, ctypes.byref(prev))
    assert rc == 0 and prev.value == 0
    # second call straight after the first: same array, different shape and pattern
    rc, out_b = _call_noalloc(lib, q2, k2, v2, "window", 8, 576, None)
    assert rc == 0
    rc, out_c = _call_noalloc(lib, q, k, v, "scatter", 3, 576, ctypes.byref(prev))
    assert rc == 0 and prev.value == 0, "the previous allocation-free call reported a failed wait"
    torch.cuda.synchronize()

    rc, ref_a = _util.call_fwd(lib, "llm", "scatter", q, k, v, 3)
    assert rc == 0
    rc, ref_b = _util.call_fwd(lib, "llm", "window", q2, k2, v2, 576)
    assert rc == 0
    torch.cuda.synchronize()
    assert _util.device_status(lib, 0, reset=True) == 0
    for got, want in ((out_a, ref_a), (out_b, ref_b), (out_c, ref_a)):
        assert bool(torch.isfinite(got).all())
        assert _util.max_abs_err(got, want) <= _util.ATOL
    # and against the oracle itself, so the comparison above is not between two wrong results
    ref = _util.oracle_attention(q, k, v, oracle.llm_scatter_mask(1500, 3), on_device=True)
    assert _util.max_abs_err(out_a, ref) <= _util.ATOL


def test_noalloc_rejects_bad_arguments(lib):
    q = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16, device="cuda")
    s = _util.strides3(q)
    p = q.data_ptr()
    st = torch.cuda.current_stream().cuda_stream
    f = lib.intra_b200_fwd_llm_noalloc
    assert f(None, p, p, p, 1, 256, 2, 2, s, s, s, s, 0, 8, 576, 0.1, 0, st, None) == -1
    assert f(p, p, p, p, 1, 256, 2, 2, s, s, s, s, 9, 8, 576, 0.1, 0, st, None) == -2
    assert f(p, p, p, p, 1, 256, 2, 2, s, s, s, s, 4, 8, 32, 0.1, 0, st, None) == -2
    assert f(p + 2, p, p, p, 1, 256, 2, 2, s, s, s, s, 0, 8, 576, 0.1, 0, st, None) == -3
