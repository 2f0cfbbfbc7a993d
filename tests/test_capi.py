"""The C-ABI library loads, exports every symbol the public header declares, and rejects bad
arguments before touching a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from tests import _util

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "intra_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(intra_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from intra_b200 import _loader
    names = declared_symbols()
    assert len(names) >= 8
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/intra_b200.h but not exported"
        assert name in _loader.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_loader.SIGNATURES) == names


def test_strerror(lib):
    assert lib.intra_b200_strerror(0) == b"ok"
    for code in range(-6, 0):
        assert len(lib.intra_b200_strerror(code)) > 10
    assert lib.intra_b200_strerror(-99) == b"unknown status"


def test_bad_arguments_are_rejected_without_a_gpu(lib):
    q = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16)
    s = _util.strides3(q)
    ptr = q.data_ptr()
    args = lambda **kw: dict(dict(q=ptr, k=ptr, v=ptr, out=ptr, B=1, S=256, H=2, Hkv=1, pattern=0, G=8, W=576,
                                  scale=0.088), **kw)

    def call(a):
        return lib.intra_b200_fwd_llm(a["q"], a["k"], a["v"], a["out"], a["B"], a["S"], a["H"], a["Hkv"], s, s, s, s,
                                      a["pattern"], a["G"], a["W"], a["scale"], 0, None)

    assert call(args(q=None)) == -1
    assert call(args(S=0)) == -1
    assert call(args(H=3, Hkv=2)) == -1
    assert call(args(scale=0.0)) == -1
    assert call(args(scale=float("nan"))) == -1
    assert call(args(pattern=7)) == -2
    assert call(args(pattern=4, W=63)) == -2
    assert call(args(G=0)) == -2
    assert call(args(q=ptr + 2)) == -3
    bad = (ctypes.c_int64 * 3)(q.stride(0), q.stride(1) + 4, q.stride(2))
    assert lib.intra_b200_fwd_llm(ptr, ptr, ptr, ptr, 1, 256, 2, 1, bad, s, s, s, 0, 8, 576, 0.088, 0, None) == -3
    # an output whose heads (or tokens) share memory: different tiles would write the same rows
    expanded = (ctypes.c_int64 * 3)(q.stride(0), q.stride(1), 0)
    assert lib.intra_b200_fwd_llm(ptr, ptr, ptr, ptr, 1, 256, 2, 1, s, s, s, expanded, 0, 8, 576, 0.088, 0, None) == -1
    negative = (ctypes.c_int64 * 3)(q.stride(0), -q.stride(1), q.stride(2))
    assert lib.intra_b200_fwd_llm(ptr, ptr, ptr, ptr, 1, 256, 2, 1, s, s, s, negative, 0, 8, 576, 0.088, 0, None) == -1
    assert lib.intra_b200_fwd_image(ptr, ptr, ptr, ptr, 1, 256, 2, s, s, s, s, 0, 64, 0.088, 0, None) == -2
    assert lib.intra_b200_fwd_image(ptr, ptr, ptr, ptr, 1, 512 + 4096, 2, s, s, s, s, 1, 64, 0.088, 0, None) == -2


def test_python_entry_points_validate_like_the_reference():
    from intra_b200 import intra_image_attn, intra_llm_attn
    q = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA bfloat16"):
        intra_llm_attn(q, q, q)
    with pytest.raises(ValueError, match="CUDA bfloat16"):
        intra_image_attn(q, q, q)


@pytest.mark.skipif(torch.cuda.is_available(), reason="only meaningful on a machine without a GPU")
def test_no_cpu_fallback(lib):
    """Without a GPU a well-formed call must fail with a CUDA error status, never compute."""
    q = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16)
    s = _util.strides3(q)
    out = torch.full_like(q, 7.0)
    rc = lib.intra_b200_fwd_llm(q.data_ptr(), q.data_ptr(), q.data_ptr(), out.data_ptr(), 1, 256, 2, 2, s, s, s, s,
                                0, 8, 576, 0.088, 0, None)
    assert rc in (-4, -5)
    assert bool((out == 7.0).all())


def test_helper_entry_points_reject_bad_arguments(lib):
    """The head-interleave entry point and the test hooks check their arguments before touching a GPU."""
    buf = torch.zeros(1024, dtype=torch.uint8)
    p = buf.data_ptr()
    assert p % 16 == 0
    f = lib.intra_b200_interleave_heads
    assert f(None, p, 2, 4, 256, 0, None) == -1
    assert f(p, p, 0, 4, 256, 0, None) == -1
    assert f(p, p, 2, 0, 256, 0, None) == -1
    assert f(p, p, 2, 4, 8, 0, None) == -3                  # blocks must be multiples of 16 bytes
    assert f(p + 4, p, 2, 4, 256, 0, None) == -3
    assert lib.intra_b200_test_force_path(0, 3) == -1
    assert lib.intra_b200_test_force_path(0, 0) == 0
    assert lib.intra_b200_test_wait_timeout(0, p, 0, None) == -1       # limit out of range
    assert lib.intra_b200_test_wait_timeout(5000, p, 0, None) == -1
    assert lib.intra_b200_test_wait_timeout(5, None, 0, None) == -1
    n = ctypes.c_int64(0)
    assert lib.intra_b200_test_tma_rows(p, p, p, 1, 256, 2, 1, None, None, None, 0, 0, 8, None, None, None, None, None,
                                        ctypes.byref(n), ctypes.byref(n), 0, None) == -1   # no strides


def test_launcher_picks_the_kernel_form_by_item_length(lib):
    """Host arithmetic only: long items that share their key tiles go to the row-owner form, short ones
    (window: 5 key tiles, Gather-0: 7, S=4096) to the 4-way column split; a forced form is honoured, with
    the 2-way split standing in for the row-owner form on split key lists."""
    form = lib.intra_b200_test_kernel_form
    LLM, IMG = 0, 1
    SCATTER, GATHER1, WINDOW, GATHER0 = 0, 1, 4, 4
    assert form(LLM, SCATTER, 4096, 8, 32, 8) == 4            # 2.5 key tiles per item
    assert form(LLM, GATHER1, 16384, 8, 32, 8) == 1           # 8.5
    assert form(LLM, WINDOW, 16384, 576, 32, 8) == 4
    assert form(LLM, SCATTER, 32768, 2, 32, 8) == 1
    assert form(LLM, SCATTER, 65536, 8, 32, 8) == 1
    assert form(LLM, WINDOW, 65536, 576, 32, 8) == 4
    assert form(IMG, SCATTER, 512 + 64 * 64, 64, 24, 24) == 1     # 8 key tiles
    assert form(IMG, SCATTER, 512 + 128 * 128, 128, 24, 24) == 1  # 20
    assert form(IMG, GATHER0, 512 + 128 * 128, 128, 24, 24) == 4  # 7, split key lists
    assert form(LLM, SCATTER, 4096, 8, 32, 5) == -1           # heads not a multiple of KV heads
    assert form(LLM, 7, 4096, 8, 32, 8) < 0                   # no such pattern
    try:
        assert lib.intra_b200_test_force_path(0, 1) == 0
        assert form(LLM, SCATTER, 4096, 8, 32, 8) == 1
        assert form(IMG, GATHER0, 512 + 128 * 128, 128, 24, 24) == 2
        assert lib.intra_b200_test_force_path(0, 4) == 0
        assert form(LLM, SCATTER, 65536, 8, 32, 8) == 4
    finally:
        assert lib.intra_b200_test_force_path(0, 0) == 0
