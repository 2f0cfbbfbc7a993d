"""The library's closed-form index maps, evaluated on the host, against the oracle's dense masks:
the visited (query, key) sets must match bit for bit, every pair visited exactly once."""
import ctypes

import numpy as np
import pytest

from oracle import intra_oracle as oracle
from tests import _util

MASK_CASES = _util.load_mask_goldens()


@pytest.mark.parametrize("case", MASK_CASES, ids=_util.case_id)
def test_visited_set_equals_mask(lib, case):
    S = case["S"]
    counts = np.zeros((S, S), dtype=np.uint8)
    rc = lib.intra_b200_visited_host(_util.FAMILY[case["family"]], _util.PATTERN_ID[(case["family"], case["pattern"])],
                                     S, _util.case_param(case), counts.ctypes.data)
    assert rc == 0
    assert counts.max() <= 1, "a (query, key) pair is visited more than once"
    mask = oracle.build_mask(case["family"], case["pattern"], S, **_util.case_kwargs(case))
    assert np.array_equal(counts.view(bool), mask)
    assert int(counts.sum(dtype=np.int64)) == case["pairs"]


@pytest.mark.parametrize("family,pattern,S,param", [
    ("llm", "scatter", 65536, 8), ("llm", "window", 65536, 576), ("llm", "scatter", 32768, 2),
    ("llm", "gather1", 16384, 8), ("image", "scatter", 16896, 128), ("image", "gather0", 16896, 128)])
def test_tile_counts_cover_pairs(lib, family, pattern, S, param):
    """At benchmark sizes: the score slots the launch computes (128 x 128 per key tile) are at least
    the attended pairs, and padding stays bounded."""
    nt, nkv = ctypes.c_int64(0), ctypes.c_int64(0)
    rc = lib.intra_b200_tile_counts(_util.FAMILY[family], _util.PATTERN_ID[(family, pattern)], S, param,
                                    ctypes.byref(nt), ctypes.byref(nkv))
    assert rc == 0 and nt.value > 0
    kw = {"group_num": param} if pattern in ("scatter", "gather1") and family == "llm" else (
        {"window": param} if family == "llm" else {"width": param})
    pairs = oracle.pair_count(family, pattern, S, **kw)
    slots = nkv.value * 128 * 128
    assert pairs <= slots <= 2.6 * pairs


def test_unsupported_shapes_are_rejected(lib):
    buf = np.zeros(16, dtype=np.uint8)
    assert lib.intra_b200_visited_host(0, 2, 64, 8, buf.ctypes.data) == -2       # unknown llm pattern id
    assert lib.intra_b200_visited_host(0, 4, 64, 32, buf.ctypes.data) == -2      # window below one block
    assert lib.intra_b200_visited_host(1, 0, 512 + 64, 8, buf.ctypes.data) == -2   # width too small
    assert lib.intra_b200_visited_host(1, 4, 512 + 64 * 64 + 1, 64, buf.ctypes.data) == -2
    assert lib.intra_b200_visited_host(0, 0, 4, 8, buf.ctypes.data) == -2        # more groups than tokens


@pytest.mark.parametrize("case", MASK_CASES, ids=_util.case_id)
def test_row_pair_visited_set_equals_mask(lib, case):
    """The decomposition into pairs of row tiles (sharing their key tiles, or for Gather-0 keeping
    their own) visits the same set."""
    S = case["S"]
    counts = np.zeros((S, S), dtype=np.uint8)
    rc = lib.intra_b200_visited_pairs_host(_util.FAMILY[case["family"]],
                                           _util.PATTERN_ID[(case["family"], case["pattern"])], S,
                                           _util.case_param(case), counts.ctypes.data)
    assert rc == 0
    assert counts.max() <= 1
    mask = oracle.build_mask(case["family"], case["pattern"], S, **_util.case_kwargs(case))
    assert np.array_equal(counts.view(bool), mask)


def _check_random_shape(lib, family, pattern, S, param):
    kw = ({"width": param} if family == "image" else
          {"window": param} if pattern == "window" else {"group_num": param})
    mask = oracle.build_mask(family, pattern, S, **kw)
    for fn in (lib.intra_b200_visited_host, lib.intra_b200_visited_pairs_host):
        counts = np.zeros((S, S), dtype=np.uint8)
        rc = fn(_util.FAMILY[family], _util.PATTERN_ID[(family, pattern)], S, param, counts.ctypes.data)
        assert rc == 0, (family, pattern, S, param, rc)
        assert counts.max() <= 1
        assert np.array_equal(counts.view(bool), mask), (family, pattern, S, param)


def test_random_llm_shapes_visit_exactly_the_mask(lib):
    """Seeded sweep over shapes the fixed matrix does not hold: ragged group lengths, sequences
    shorter than a tile, group counts that do not divide anything, windows that are not block
    multiples - both the tile and the pair-tile decomposition."""
    rng = np.random.default_rng(20240611)
    for _ in range(60):
        S = int(rng.integers(1, 900))
        G = int(rng.integers(1, min(S, 13) + 1))
        _check_random_shape(lib, "llm", "scatter", S, G)
        _check_random_shape(lib, "llm", "gather1", S, G)
        W = int(rng.integers(64, 1100))
        _check_random_shape(lib, "llm", "window", S, W)


@pytest.mark.parametrize("width", [16, 24, 40, 56])
def test_odd_image_widths_visit_exactly_the_mask(lib, width):
    """Widths beyond the reference's 64 and 128: an odd number of patches per row leaves a patch
    without a partner, and width / 4 need not divide a tile."""
    S = 512 + width * width
    _check_random_shape(lib, "image", "scatter", S, width)
    _check_random_shape(lib, "image", "gather0", S, width)
