"""The CPU oracle against the fixtures generated from the reference's own Python code."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import intra_oracle as oracle
from tests import _util

MASK_CASES = _util.load_mask_goldens()
ATTN_META, ATTN = _util.load_attention_goldens()


@pytest.mark.parametrize("case", MASK_CASES, ids=_util.case_id)
def test_mask_matches_reference_digest(case):
    m = oracle.build_mask(case["family"], case["pattern"], case["S"], **_util.case_kwargs(case))
    d = oracle.mask_digest(m)
    assert d["shape"] == case["shape"]
    assert d["pairs"] == case["pairs"]
    assert d["row_checksum"] == case["row_checksum"]
    assert d["sha256"] == case["sha256"]
    assert oracle.pair_count(case["family"], case["pattern"], case["S"], **_util.case_kwargs(case)) == case["pairs"]


def test_pair_counts_at_benchmark_sizes():
    # Closed forms at sizes whose dense masks are too large to build in a unit test.
    assert oracle.pair_count("llm", "scatter", 4096, group_num=8) == 1050624
    assert oracle.pair_count("llm", "gather1", 16384, group_num=8) == 16785408
    assert oracle.pair_count("llm", "window", 16384, window=576) == 8773632
    assert oracle.pair_count("llm", "scatter", 65536, group_num=8) == 268468224
    assert oracle.pair_count("llm", "window", 65536, window=576) == 35536896
    assert oracle.pair_count("llm", "scatter", 32768, group_num=2) == 268451840
    assert oracle.pair_count("image", "scatter", 512 + 128 * 128, width=128) == 43253760
    assert oracle.pair_count("image", "gather0", 512 + 128 * 128, width=128) == 13893632


@pytest.mark.parametrize("meta", ATTN_META, ids=lambda m: m["name"])
def test_attention_matches_reference_output(meta):
    q, k, v = oracle.make_inputs(meta["B"], meta["S"], meta["H"], meta["Hkv"], seed=meta["seed"])
    h = hashlib.sha256()
    for x in (q, k, v):
        h.update(x.contiguous().view(torch.int16).numpy().view(np.uint16).tobytes())
    assert h.hexdigest() == meta["inputs_sha256"], "seeded inputs differ from the ones the fixture was made with"
    mask = oracle.build_mask(meta["family"], meta["pattern"], meta["S"], **_util.case_kwargs(meta))
    want = _util.bf16_from_bits(ATTN[meta["name"]])
    got = oracle.masked_attention(q, k, v, mask)
    # Same algorithm as the fixture's generator; one bf16 ulp of slack for a different CPU's SDPA.
    assert torch.allclose(got.float(), want.float(), atol=2e-3, rtol=8e-3)
    rows = oracle.masked_attention_rows(q, k, v, mask, rows=200)
    assert torch.allclose(rows.float(), want.float(), atol=2e-3, rtol=8e-3)


def test_masked_lse_matches_direct_logsumexp_and_softmax():
    """The log-sum-exp oracle: equal to a direct logsumexp over the masked scores, slab size
    irrelevant, and consistent with masked_attention (exp(s - lse) are its probabilities)."""
    q, k, v = oracle.make_inputs(1, 300, 4, 2, seed=1)
    mask = torch.from_numpy(oracle.llm_scatter_mask(300, 3))
    lse = oracle.masked_lse(q, k, mask, rows=128)
    assert lse.shape == (1, 4, 300) and lse.dtype == torch.float32
    kf = k.float().repeat_interleave(2, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) * 128 ** -0.5
    s = s.masked_fill(~mask, float("-inf"))
    assert float((torch.logsumexp(s, -1) - lse).abs().max()) <= 1e-5
    assert torch.equal(lse, oracle.masked_lse(q, k, mask, rows=77))
    p = torch.exp(s - lse[..., None])
    out = torch.einsum("bhqk,bkhd->bqhd", p, v.float().repeat_interleave(2, dim=2))
    ref = oracle.masked_attention(q, k, v, mask).float()
    assert float((out - ref).abs().max()) <= 1e-2


@pytest.mark.parametrize("case", [c for c in MASK_CASES if c["S"] <= 4608], ids=_util.case_id)
def test_mask_row_slabs_equal_slices_of_the_full_mask(case):
    """The row-slab form of every mask builder (what the parity tests at S = 32768 and 65536 use, where
    the S x S mask cannot be built) is bit for bit the corresponding slice of the pinned full mask."""
    S, kw = case["S"], _util.case_kwargs(case)
    full = oracle.build_mask(case["family"], case["pattern"], S, **kw)
    for r0, r1 in ((0, min(S, 100)), (S // 3, min(S, S // 3 + 517)), (max(S - 129, 0), S), (500, min(S, 700))):
        if r0 >= r1:
            continue
        assert np.array_equal(oracle.build_mask(case["family"], case["pattern"], S, rows=(r0, r1), **kw), full[r0:r1])
    picked = np.arange(3, S, 37)
    assert np.array_equal(oracle.build_mask(case["family"], case["pattern"], S, rows=picked, **kw), full[picked])


def test_slab_attention_matches_sdpa_form():
    """masked_attention_slab (explicit softmax, one slab of query rows) against the SDPA form that is
    pinned to the reference's outputs, including its log-sum-exp against masked_lse."""
    q, k, v = oracle.make_inputs(2, 700, 4, 2, seed=3)
    for mask in (oracle.llm_window_mask(700, 200), oracle.llm_gather1_mask(700, 4)):
        ref = oracle.masked_attention_fp32(q, k, v, mask)
        lse_ref = oracle.masked_lse(q, k, torch.from_numpy(mask))
        for r0, r1 in ((0, 128), (300, 700)):
            out, lse = oracle.masked_attention_slab(q[:, r0:r1], k, v, mask[r0:r1])
            assert out.dtype == torch.float32 and out.shape == (2, r1 - r0, 4, 128)
            assert float((out - ref[:, r0:r1]).abs().max()) <= 2e-5
            assert float((lse - lse_ref[:, :, r0:r1]).abs().max()) <= 2e-5
