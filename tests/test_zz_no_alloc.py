"""The allocation-free entry point `intra_b200_fwd_llm_noalloc` against the regular one.

For hosts that keep all of HBM in their own arena (a library-side cudaMalloc would fail or stall
them) the library offers one launch path whose scratch is a fixed array inside the library image.
This test calls it through the C ABI several times in a row - each call reuses the array the one
before left behind - checks the outputs against `intra_b200_fwd_llm` on the same inputs, and checks
that the device's free memory does not move across the calls. It lives in a
file that sorts last so that a run stopping at the first failure has already run everything else; it
needs nothing from the other tests and also passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

from oracle import intra_oracle as oracle
from tests import _util

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, q, k, v, out, pattern, group_num, window, prev=None):
    B, S, H, D = q.shape
    return lib.intra_b200_fwd_llm_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, H, k.shape[2],
        _util.strides3(q), _util.strides3(k), _util.strides3(v), _util.strides3(out),
        _util.PATTERN_ID[("llm", pattern)], group_num, window, D ** -0.5, q.device.index,
        torch.cuda.current_stream(q.device).cuda_stream, prev)


def _noalloc_against_regular(lib):
    """Three allocation-free calls in a row, then the regular entry point on the same inputs. Every
    tensor exists before the first call, and the free device memory the driver reports must not move
    across the second and third calls (the first may pay one-time costs such as loading the kernels)."""
    assert torch.cuda.is_available()
    q, k, v = oracle.make_inputs(2, 1500, 8, 2, seed=31, device="cuda")
    q2, k2, v2 = oracle.make_inputs(1, 2048, 4, 4, seed=32, device="cuda")
    out_a, out_c, ref_a = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    out_b, ref_b = torch.empty_like(q2), torch.empty_like(q2)
    torch.cuda.synchronize()

    prev = ctypes.c_int(-1)
    assert _call_noalloc(lib, q, k, v, out_a, "scatter", 3, 576, ctypes.byref(prev)) == 0 and prev.value == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    # second call straight after the first: same array, different shape and pattern
    assert _call_noalloc(lib, q2, k2, v2, out_b, "window", 8, 576, None) == 0
    assert _call_noalloc(lib, q, k, v, out_c, "scatter", 3, 576, ctypes.byref(prev)) == 0
    assert prev.value == 0, "the previous allocation-free call reported a failed wait"
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "an allocation-free call changed the free device memory"

    assert _util.call_fwd(lib, "llm", "scatter", q, k, v, 3, out=ref_a)[0] == 0
    assert _util.call_fwd(lib, "llm", "window", q2, k2, v2, 576, out=ref_b)[0] == 0
    torch.cuda.synchronize()
    assert _util.device_status(lib, 0, reset=True) == 0
    for got, want in ((out_a, ref_a), (out_b, ref_b), (out_c, ref_a)):
        assert bool(torch.isfinite(got).all())
        assert _util.max_abs_err(got, want) <= _util.ATOL
    # and against the oracle itself, so the comparison above is not between two wrong results
    _util.check_against_oracle(out_a, q, k, v, oracle.llm_scatter_mask(1500, 3))


def test_noalloc_matches_regular_entry_point_twice(lib):
    _noalloc_against_regular(lib)


def test_noalloc_first_thing_in_a_fresh_process():
    """The same sequence in a child process whose very first library call is the allocation-free one,
    so that no regular entry point has set the device up (or allocated) before it."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys; sys.path.insert(0, sys.argv[1])\n"
            "from intra_b200 import _loader\n"
            "from tests.test_zz_no_alloc import _noalloc_against_regular\n"
            "_noalloc_against_regular(_loader.lib)\nprint('NOALLOC-OK')\n")
    proc = subprocess.run([sys.executable, "-c", code, root], capture_output=True, text=True, timeout=600, cwd=root)
    assert proc.returncode == 0 and "NOALLOC-OK" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-2000:]


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
