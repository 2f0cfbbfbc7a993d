"""GPU parity: the CUDA path, called through the C ABI, against the oracle and the golden fixtures."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import intra_oracle as oracle
from tests import _util

pytestmark = pytest.mark.gpu

MASK_CASES = _util.load_mask_goldens()
ATTN_META, ATTN = _util.load_attention_goldens()


@pytest.fixture(autouse=True)
def _status_clean(lib):
    """Every test starts and ends with a healthy device status word."""
    assert torch.cuda.is_available()
    _util.device_status(lib, 0, reset=True)
    yield
    assert _util.device_status(lib, 0, reset=True) == 0, "a kernel gave up on a bounded wait"


def test_library_is_native(lib):
    """The tests must exercise the in-tree CUDA library, on an sm_100 device."""
    from intra_b200 import _loader
    assert _loader.LIB_PATH.endswith("intra_b200/_lib/libintra_b200.so")
    assert torch.cuda.get_device_capability(0)[0] == 10


def test_umma_single_tile(lib):
    """One 128x128x128 tile through both tensor-core contractions (operand layouts, descriptors,
    TMEM load/store paths) against fp32 matmuls of the same bf16 data."""
    g = torch.Generator().manual_seed(5)
    a, b, v = (torch.randn(128, 128, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    s_out = torch.zeros(128, 128, device="cuda")
    o_out = torch.zeros(128, 128, device="cuda")
    p_scale = 1.0 / 16
    rc = lib.intra_b200_selftest_umma(a.data_ptr(), b.data_ptr(), v.data_ptr(), p_scale, s_out.data_ptr(),
                                      o_out.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    s_ref = a.float() @ b.float().t()
    assert torch.allclose(s_out, s_ref, atol=1e-3, rtol=1e-4)
    p_ref = (s_out * p_scale).to(torch.bfloat16).float()
    o_ref = p_ref @ v.float()
    assert torch.allclose(o_out, o_ref, atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("case", [c for c in MASK_CASES if c["S"] <= 8192], ids=_util.case_id)
def test_device_visited_set_equals_mask(lib, case):
    """The index maps as the device evaluates them: visited (query, key) pairs == oracle mask."""
    S = case["S"]
    counts = torch.zeros(S, S, dtype=torch.uint8, device="cuda")
    rc = lib.intra_b200_visited_device(_util.FAMILY[case["family"]],
                                       _util.PATTERN_ID[(case["family"], case["pattern"])], S,
                                       _util.case_param(case), counts.data_ptr(), 0,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    mask = oracle.build_mask(case["family"], case["pattern"], S, **_util.case_kwargs(case))
    got = counts.cpu().numpy()
    assert got.max() <= 1
    assert np.array_equal(got.view(bool), mask)


@pytest.mark.parametrize("meta", ATTN_META, ids=lambda m: m["name"])
def test_golden_outputs(lib, meta):
    """Outputs of the reference's own oracle on seeded inputs (committed fixtures)."""
    q, k, v = oracle.make_inputs(meta["B"], meta["S"], meta["H"], meta["Hkv"], seed=meta["seed"], device="cuda")
    rc, out = _util.call_fwd(lib, meta["family"], meta["pattern"], q, k, v, _util.case_param(meta))
    assert rc == 0
    torch.cuda.synchronize()
    want = _util.bf16_from_bits(ATTN[meta["name"]])
    assert bool(torch.isfinite(out).all())
    assert _util.max_abs_err(out, want) <= _util.ATOL


def _llm_matrix():
    cases = []
    for S in (1000, 2048, 3000, 4096, 8192, 16384):
        for B, H, Hkv in ((1, 32, 8), (2, 32, 32)):
            for G in (2, 3, 8):
                cases.append(("scatter", S, B, H, Hkv, G))
            if S % 64 == 0:
                cases.append(("gather1", S, B, H, Hkv, 8))
            for W in (576, 1000):
                cases.append(("window", S, B, H, Hkv, W))
    return cases


@pytest.mark.parametrize("pattern,S,B,H,Hkv,param", _llm_matrix(),
                         ids=lambda x: str(x))
def test_llm_matrix(lib, pattern, S, B, H, Hkv, param):
    """The shape matrix of the reference's kernel test (tests/test_kernel.py:33-44), seed 0."""
    q, k, v = oracle.make_inputs(B, S, H, Hkv, seed=0, device="cuda")
    rc, out = _util.call_fwd(lib, "llm", pattern, q, k, v, param)
    assert rc == 0
    kw = {"window": param} if pattern == "window" else {"group_num": param}
    mask = oracle.build_mask("llm", pattern, S, **kw)
    _util.check_against_oracle(out, q, k, v, mask)


@pytest.mark.parametrize("width,H", [(64, 24), (128, 8)])
@pytest.mark.parametrize("B", [1, 2])
@pytest.mark.parametrize("pattern", ["scatter", "gather0"])
def test_image_matrix(lib, pattern, B, width, H):
    """Image shapes of the reference's kernel test (tests/test_kernel.py:45-51)."""
    S = 512 + width * width
    q, k, v = oracle.make_inputs(B, S, H, H, seed=0, device="cuda")
    rc, out = _util.call_fwd(lib, "image", pattern, q, k, v, width)
    assert rc == 0
    mask = oracle.build_mask("image", pattern, S, width=width)
    _util.check_against_oracle(out, q, k, v, mask)


# The five BASELINE configurations at their full sizes. Their S x S masks do not fit anywhere, so the
# oracle runs on the GPU over slabs of query rows whose mask rows are built per slab from the same
# predicates (tests/test_oracle.py pins slab == slice of the full mask): every query head on slabs at
# the start, the middle, the end and an odd offset of the sequence (the odd one straddles tile, group
# and block boundaries), plus, where `group_rows` is set, every row of the first KV-head group.
BASELINE_CASES = [
    # name, family, pattern, S, H, Hkv, kwargs, all rows of KV-head group 0?
    ("c4-scatter-g2-32k", "llm", "scatter", 32768, 32, 8, {"group_num": 2}, False),
    ("c4-window-32k", "llm", "window", 32768, 32, 8, {"window": 576}, True),
    ("c5-scatter-g8-64k", "llm", "scatter", 65536, 32, 8, {"group_num": 8}, False),
    ("c5-window-64k", "llm", "window", 65536, 32, 8, {"window": 576}, True),
    ("c2-gather1-16k", "llm", "gather1", 16384, 32, 8, {"group_num": 8}, True),
    ("c3-scatter-w128-h24", "image", "scatter", 512 + 128 * 128, 24, 24, {"width": 128}, True),
    ("c3-gather0-w128-h24", "image", "gather0", 512 + 128 * 128, 24, 24, {"width": 128}, True),
]
SLAB = 1024


@pytest.mark.parametrize("name,family,pattern,S,H,Hkv,kw,group_rows", BASELINE_CASES, ids=[c[0] for c in BASELINE_CASES])
def test_baseline_configs_full_size(lib, name, family, pattern, S, H, Hkv, kw, group_rows):
    from intra_b200 import intra_image_attn, intra_llm_attn
    q, k, v = oracle.make_inputs(1, S, H, Hkv, seed=0, device="cuda")
    fn = intra_image_attn if family == "image" else intra_llm_attn
    with torch.no_grad():
        out, lse = fn(q, k, v, pattern, return_lse=True, **kw)
        plain = fn(q, k, v, pattern, **kw)
    torch.cuda.synchronize()
    assert torch.equal(out, plain), "asking for the log-sum-exp changed the output"
    rep = H // Hkv
    starts = sorted({0, S // 2 - SLAB // 2, S - SLAB, min(128 * 37 + 71, S - SLAB)})
    worst = 0.0
    checked = 0
    first_groups = 1 if family == "llm" else 3
    plan = [(r0, range(Hkv)) for r0 in starts]
    if group_rows:
        plan += [(r0, range(first_groups)) for r0 in range(0, S, SLAB)]
    for r0, groups in plan:
        r1 = min(r0 + SLAB, S)
        mask_rows = torch.from_numpy(oracle.build_mask(family, pattern, S, rows=(r0, r1), **kw)).cuda()
        for g in groups:
            hs = slice(g * rep, (g + 1) * rep)
            ref, ref_lse, spread = oracle.masked_attention_slab(q[:, r0:r1, hs], k[:, :, g:g + 1], v[:, :, g:g + 1],
                                                                mask_rows, with_spread=True)
            worst = max(worst, _util.check_parity(out[:, r0:r1, hs], ref, spread))
            assert float((lse[:, hs, r0:r1] - ref_lse).abs().max()) <= LSE_ATOL
            checked += (r1 - r0) * rep
    assert checked >= 4 * SLAB * H
    print(f"{name}: {checked} query rows x heads checked, max |err| {worst:.3e}")


def _encoded_rows(B, S, H, tensor_id):
    """(B, S, H, 128) bf16 whose row for token t holds (t + 1) in base 256, the head, the batch and the
    tensor id in elements 0..5 of both 64-element halves (all exact in bfloat16)."""
    x = torch.zeros(B, S, H, 128, dtype=torch.float32)
    t = torch.arange(S) + 1
    for half in (0, 64):
        x[..., half + 0] = (t % 256)[None, :, None]
        x[..., half + 1] = ((t // 256) % 256)[None, :, None]
        x[..., half + 2] = (t // 65536)[None, :, None]
        x[..., half + 3] = torch.arange(H)[None, None, :]
        x[..., half + 4] = torch.arange(B)[:, None, None]
        x[..., half + 5] = tensor_id
    return x.to(torch.bfloat16).cuda()


@pytest.mark.parametrize("case", MASK_CASES + [
    {"family": "llm", "pattern": "scatter", "S": 65536, "group_num": 8},
    {"family": "llm", "pattern": "scatter", "S": 32768, "group_num": 2},
    {"family": "llm", "pattern": "window", "S": 65536, "window": 576}], ids=_util.case_id)
@pytest.mark.parametrize("heads", [(2, 1), (3, 3)], ids=["head-pairs", "row-pairs"])
def test_tma_tiles_hold_the_rows_the_index_maps_name(lib, case, heads):
    """The production TMA path, bit-exact: every query tile and every key / value tile of every item is
    fetched by the attention kernel's own planning and load code from tensors whose rows encode their
    token id, head, batch and tensor, and the rows that arrive in shared memory are compared with the
    closed-form index maps (whose visited sets the CPU tests pin to the masks). Covers the tensor maps
    (capi.cu build_maps), the box coordinates (tma_maps.h) and the per-item affine plan of the key tiles."""
    family, pattern, S = case["family"], case["pattern"], case["S"]
    H, Hkv = heads if family == "llm" else (heads[0], heads[0])
    B = 2 if S <= 4608 else 1
    q, k, v = _encoded_rows(B, S, H, 0), _encoded_rows(B, S, Hkv, 1), _encoded_rows(B, S, Hkv, 2)
    n_items, max_kv = ctypes.c_int64(0), ctypes.c_int64(0)
    args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), B, S, H, Hkv, _util.strides3(q), _util.strides3(k),
            _util.strides3(v), _util.FAMILY[family], _util.PATTERN_ID[(family, pattern)], _util.case_param(case))
    rc = lib.intra_b200_test_tma_rows(*args, None, None, None, None, None, ctypes.byref(n_items), ctypes.byref(max_kv),
                                      0, torch.cuda.current_stream().cuda_stream)
    if rc == -2:
        pytest.skip("shape takes the cp.async gathers, not TMA boxes")
    assert rc == 0 and n_items.value > 0 and max_kv.value > 0
    nq, nk = n_items.value * 2 * 128, n_items.value * 2 * max_kv.value * 128
    q_got = torch.full((nq,), -3, dtype=torch.int32, device="cuda")
    k_got = torch.full((nk,), -3, dtype=torch.int32, device="cuda")
    v_got = torch.full((nk,), -3, dtype=torch.int32, device="cuda")
    q_want = np.zeros(nq, dtype=np.int32)
    k_want = np.zeros(nk, dtype=np.int32)
    rc = lib.intra_b200_test_tma_rows(*args, q_got.data_ptr(), k_got.data_ptr(), v_got.data_ptr(), q_want.ctypes.data,
                                      k_want.ctypes.data, ctypes.byref(n_items), ctypes.byref(max_kv), 0,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert (q_want >= 0).sum() == B * H * S, "every query token belongs to exactly one tile row"
    for got, want, what in ((q_got, q_want, "query"), (k_got, k_want, "key"), (v_got, k_want, "value")):
        got = got.cpu().numpy()
        used = want != -9
        assert used.any()
        bad = np.nonzero(used & (got != want))[0]
        assert bad.size == 0, f"{what} rows differ at {bad[:8]}: got {got[bad[:8]]}, want {want[bad[:8]]}"


@pytest.mark.parametrize("world,B,S,Hl", [(2, 1, 4096, 16), (8, 2, 1000, 4), (3, 1, 77, 1)])
def test_interleave_heads_kernel(lib, world, B, S, Hl):
    """The multi-GPU launcher's reorder kernel on one GPU: rank-major blocks of an all-gather into
    (batch, token, head, 128) order, bit for bit against a torch permute."""
    from intra_b200 import sharded
    parts = torch.randn(world, B, S, Hl, 128, device="cuda").to(torch.bfloat16)
    got = sharded.interleave_heads(parts)
    want = parts.permute(1, 2, 0, 3, 4).reshape(B, S, world * Hl, 128)
    torch.cuda.synchronize()
    assert got.shape == want.shape and torch.equal(got, want)


def test_status_word_is_sticky_but_launches_go_on(lib):
    """The documented behaviour of the status word: a recorded failure stays until it is reset and is
    reported by intra_b200_device_status, and launches made meanwhile still compute their outputs. The
    failure is written from the host; no kernel misbehaves."""
    q, k, v = oracle.make_inputs(1, 1024, 4, 2, seed=41, device="cuda")
    rc, want = _util.call_fwd(lib, "llm", "scatter", q, k, v, 4)
    assert rc == 0
    assert lib.intra_b200_test_poke_status(0, 133) == 0
    rc, got = _util.call_fwd(lib, "llm", "scatter", q, k, v, 4)
    assert rc == 0, "entry points do not poll the status word"
    torch.cuda.synchronize()
    assert torch.equal(got, want), "a recorded failure must not turn later launches into no-ops"
    word = ctypes.c_int(0)
    assert lib.intra_b200_device_status(0, ctypes.byref(word), 0) == -6 and word.value == 133
    assert lib.intra_b200_device_status(0, ctypes.byref(word), 1) == -6 and word.value == 133
    assert lib.intra_b200_device_status(0, ctypes.byref(word), 0) == 0 and word.value == 0


def test_bounded_wait_gives_up_and_reports(lib):
    """The abort protocol end to end on a wait that nothing satisfies: the wait runs out after its
    limit (20 ms here), the give-up releases the other warp long before its own 2 s limit, tensor memory
    is freed, the kernel returns normally, the status word names the wait site, the context stays usable."""
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    assert lib.intra_b200_test_wait_timeout(20, waited.data_ptr(), 0, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()                                # returns: the kernel ended by itself
    ns = int(waited.item())
    assert 15e6 <= ns <= 500e6, f"the second warp waited {ns / 1e6:.1f} ms"
    word = ctypes.c_int(0)
    assert lib.intra_b200_device_status(0, ctypes.byref(word), 1) == -6
    assert word.value in (100 + 92, 100 + 1), word.value
    assert lib.intra_b200_device_status(0, ctypes.byref(word), 0) == 0 and word.value == 0
    q, k, v = oracle.make_inputs(1, 512, 2, 2, seed=43, device="cuda")      # the device still works
    rc, out = _util.call_fwd(lib, "llm", "window", q, k, v, 576)
    assert rc == 0
    _util.check_against_oracle(out, q, k, v, oracle.llm_window_mask(512, 576))


@pytest.mark.parametrize("family,pattern,S,param", [
    ("llm", "scatter", 1111, 5), ("llm", "gather1", 777, 4), ("llm", "gather1", 1000, 8),
    ("llm", "window", 130, 64), ("llm", "window", 129, 200), ("llm", "scatter", 1, 1),
    ("image", "scatter", 512 + 24 * 24, 24), ("image", "gather0", 512 + 24 * 24, 24),
    ("image", "gather0", 512 + 40 * 40, 40)])
def test_ragged_and_small_shapes_vs_cpu_oracle(lib, family, pattern, S, param):
    """Shapes beyond the reference's restrictions; oracle on the CPU."""
    H, Hkv = (4, 2) if family == "llm" else (2, 2)
    q, k, v = oracle.make_inputs(1, S, H, Hkv, seed=3, device="cuda")
    rc, out = _util.call_fwd(lib, family, pattern, q, k, v, param, scale=0.11)
    assert rc == 0
    kw = {"width": param} if family == "image" else ({"window": param} if pattern == "window" else {"group_num": param})
    mask = oracle.build_mask(family, pattern, S, **kw)
    ref = _util.oracle_attention(q, k, v, mask, scale=0.11)
    assert bool(torch.isfinite(out).all())
    assert _util.max_abs_err(out, ref) <= _util.ATOL


def test_python_api_strided_views_and_errors(lib):
    """The reference-shaped Python API: transposed (B, H, S, D)-storage views as the FLUX caller
    passes them (experiments/flux/intra_processor.py:128-135), canary rows, run-twice determinism,
    and the reference's exceptions."""
    from intra_b200 import intra_image_attn, intra_llm_attn
    B, S, H, Hkv = 1, 2048, 8, 2
    g = torch.Generator().manual_seed(9)
    qs = torch.randn(B, H, S + 2, 128, generator=g).to(torch.bfloat16).cuda()
    ks = torch.randn(B, Hkv, S + 2, 128, generator=g).to(torch.bfloat16).cuda()
    vs = torch.randn(B, Hkv, S + 2, 128, generator=g).to(torch.bfloat16).cuda()
    qs[:, :, 0] = float("nan"); qs[:, :, -1] = float("nan")        # guard rows around the views
    ks[:, :, 0] = float("nan"); ks[:, :, -1] = float("nan")
    vs[:, :, 0] = float("nan"); vs[:, :, -1] = float("nan")
    q, k, v = (x[:, :, 1:-1].transpose(1, 2) for x in (qs, ks, vs))
    assert not q.is_contiguous() and q.stride(-1) == 1
    with torch.no_grad():
        out1 = intra_llm_attn(q, k, v, "scatter", group_num=8)
        out2 = intra_llm_attn(q, k, v, "scatter", group_num=8)
        outw = intra_llm_attn(q, k, v, "window", window=576)
    assert out1.shape == q.shape and out1.dtype == q.dtype
    assert torch.equal(out1, out2), "two runs differ bitwise"
    ref = _util.oracle_attention(q, k, v, oracle.llm_scatter_mask(S, 8), on_device=True)
    assert _util.max_abs_err(out1, ref) <= _util.ATOL
    refw = _util.oracle_attention(q, k, v, oracle.llm_window_mask(S, 576), on_device=True)
    assert _util.max_abs_err(outw, refw) <= _util.ATOL

    width = 64
    Si = 512 + width * width
    qi = torch.randn(1, 2, Si, 128, generator=g).to(torch.bfloat16).cuda().transpose(1, 2)
    with torch.no_grad():
        oi = intra_image_attn(qi, qi, qi, "gather0", width)
    refi = _util.oracle_attention(qi, qi, qi, oracle.image_gather0_mask(width), on_device=True)
    assert _util.max_abs_err(oi, refi) <= _util.ATOL

    x = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        intra_llm_attn(x.float(), x.float(), x.float())
    with pytest.raises(ValueError):
        intra_llm_attn(x[..., :64], x[..., :64], x[..., :64])
    with pytest.raises(ValueError, match="gather1"):
        intra_llm_attn(x, x, x, "gather1", group_num=4)
    with pytest.raises(ValueError, match="gather1"):
        intra_llm_attn(x[:, :200], x[:, :200], x[:, :200], "gather1", group_num=8)
    with pytest.raises(KeyError):
        intra_llm_attn(x, x, x, "nope")
    with pytest.raises(ValueError, match="width"):
        intra_image_attn(x, x, x, "scatter", 32)
    with pytest.raises(ValueError, match="expected"):
        intra_image_attn(x, x, x, "scatter", 64)
    xr = x.clone().requires_grad_(True)
    with pytest.raises(RuntimeError, match="forward-only"):
        intra_llm_attn(xr, x, x)


def test_non_default_stream_and_scale(lib):
    q, k, v = oracle.make_inputs(2, 1536, 4, 4, seed=21, device="cuda")
    st = torch.cuda.Stream()
    from intra_b200 import intra_llm_attn
    with torch.no_grad(), torch.cuda.stream(st):
        out = intra_llm_attn(q, k, v, "gather1", group_num=8, softmax_scale=0.05)
    st.synchronize()
    ref = _util.oracle_attention(q, k, v, oracle.llm_gather1_mask(1536, 8), scale=0.05, on_device=True)
    assert _util.max_abs_err(out, ref) <= _util.ATOL


def test_flux_caller_and_relaxed_shapes(lib):
    """The FLUX processor's call shape ((B, H, S, D) tensors, alternating patterns) and the shapes the
    reference's wrapper refuses but the kernels handle (strict=False)."""
    from intra_b200 import flux, intra_image_attn, intra_llm_attn
    assert [flux.layer_pattern(i) for i in range(6)] == ["scatter", "scatter", "gather0", "gather0", "scatter", "scatter"]
    assert flux.latent_width(512 + 64 * 64) == 64
    with pytest.raises(ValueError):
        flux.latent_width(512 + 60 * 60 + 1)
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(1, 3, 512 + 64 * 64, 128, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    with torch.no_grad():
        for layer in (0, 2):
            pattern = flux.layer_pattern(layer)
            out = flux.flux_joint_attention(q, k, v, pattern)
            assert out.shape == q.shape
            mask = oracle.build_mask("image", pattern, q.shape[2], width=64)
            ref = _util.oracle_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), mask, on_device=True)
            assert _util.max_abs_err(out.transpose(1, 2), ref) <= _util.ATOL
        # relaxed shapes through the Python API
        ql, kl, vl = oracle.make_inputs(1, 1000, 4, 2, seed=8, device="cuda")
        out = intra_llm_attn(ql, kl, vl, "gather1", group_num=5, strict=False)
        ref = _util.oracle_attention(ql, kl, vl, oracle.llm_gather1_mask(1000, 5), on_device=True)
        assert _util.max_abs_err(out, ref) <= _util.ATOL
        qi, ki, vi = oracle.make_inputs(1, 512 + 48 * 48, 2, 2, seed=9, device="cuda")
        for pattern in ("scatter", "gather0"):
            out = intra_image_attn(qi, ki, vi, pattern, 48, strict=False)
            ref = _util.oracle_attention(qi, ki, vi, oracle.build_mask("image", pattern, qi.shape[1], width=48), on_device=True)
            assert _util.max_abs_err(out, ref) <= _util.ATOL
        with pytest.raises(ValueError):
            intra_image_attn(qi, ki, vi, "scatter", 48)


@pytest.mark.parametrize("gain", [6.0, 24.0])
def test_large_logits_exercise_rescaling(lib, gain):
    """Scores spread over hundreds of units (large-magnitude q): the running maximum moves many times,
    accumulators are rescaled in tensor memory, and most probabilities underflow to zero."""
    q, k, v = oracle.make_inputs(1, 3072, 4, 2, seed=17, device="cuda")
    q = (q.float() * gain).to(torch.bfloat16)
    for pattern, param, mask in (("scatter", 2, oracle.llm_scatter_mask(3072, 2)),
                                 ("window", 576, oracle.llm_window_mask(3072, 576))):
        rc, out = _util.call_fwd(lib, "llm", pattern, q, k, v, param)
        assert rc == 0
        ref = _util.oracle_attention(q, k, v, mask, on_device=True)
        assert bool(torch.isfinite(out).all())
        assert _util.max_abs_err(out, ref) <= 2 * _util.ATOL   # near one-hot rows: a bf16 ulp of |v| <= 4


def test_llm_backend_callable(lib):
    """The transformers-style attention callable: layer schedule, (B, H, S, D) inputs, prefill on the
    kernels, dense decode step."""
    from intra_b200 import llm_backend

    class Layer:
        def __init__(self, idx):
            self.layer_idx = idx

    assert [llm_backend.layer_masktype(i) for i in range(6)] == [0, 0, 4, 4, 0, 0]
    fn = llm_backend.make_intra_attention()
    g = torch.Generator().manual_seed(12)
    q = torch.randn(1, 8, 1024, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(1, 2, 1024, 128, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(1, 2, 1024, 128, generator=g).to(torch.bfloat16).cuda()
    for idx, mask in ((1, oracle.llm_scatter_mask(1024, 8)), (2, oracle.llm_window_mask(1024, 576))):
        out, w = fn(Layer(idx), q, k, v, scaling=128 ** -0.5)
        assert w is None and out.shape == (1, 1024, 8, 128)
        ref = _util.oracle_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), mask, on_device=True)
        assert _util.max_abs_err(out, ref) <= _util.ATOL
    out, _ = fn(Layer(0), q[:, :, -1:], k, v, scaling=128 ** -0.5)     # decode step: dense over the cache
    kk, vv = k.repeat_interleave(4, 1).float(), v.repeat_interleave(4, 1).float()
    att = torch.softmax(q[:, :, -1:].float() @ kk.transpose(-1, -2) * 128 ** -0.5, -1) @ vv
    assert _util.max_abs_err(out, att.transpose(1, 2)) <= _util.ATOL


LSE_ATOL = 2e-3   # fp32 scores and sums; exponentials are ex2.approx / a cubic, both far below this


@pytest.mark.parametrize("family,pattern,S,H,Hkv,param", [
    ("llm", "scatter", 3000, 4, 2, 3),      # ragged groups, head pairs
    ("llm", "gather1", 2048, 3, 3, 8),      # odd head count: row pairs
    ("llm", "window", 2500, 4, 1, 576),
    ("image", "scatter", 512 + 32 * 32, 2, 2, 32),
    ("image", "gather0", 512 + 32 * 32, 2, 2, 32),
])
def test_lse_output(lib, family, pattern, S, H, Hkv, param):
    """The optional log-sum-exp output against the oracle on every pattern; asking for it does not
    change the attention output."""
    from intra_b200 import intra_image_attn, intra_llm_attn
    q, k, v = oracle.make_inputs(2, S, H, Hkv, seed=23, device="cuda")
    kw = {"width": param} if family == "image" else ({"window": param} if pattern == "window" else {"group_num": param})
    mask = oracle.build_mask(family, pattern, S, **kw)
    ref = oracle.masked_lse(q, k, torch.from_numpy(mask).cuda())
    fn = intra_image_attn if family == "image" else intra_llm_attn
    with torch.no_grad():
        plain = fn(q, k, v, pattern, strict=False, **kw)
        out, lse = fn(q, k, v, pattern, strict=False, return_lse=True, **kw)
    assert lse.shape == (2, H, S) and lse.dtype == torch.float32
    assert torch.equal(out, plain)
    assert bool(torch.isfinite(lse).all())
    assert float((lse - ref).abs().max()) <= LSE_ATOL


def test_lse_merges_disjoint_key_sets(lib):
    """Two nested windows: the log-sum-exp grows with the key set, and by the log of the added mass,
    which is the property a caller merging partial results relies on."""
    from intra_b200 import intra_llm_attn
    q, k, v = oracle.make_inputs(1, 2048, 2, 2, seed=29, device="cuda")
    with torch.no_grad():
        _, lse_small = intra_llm_attn(q, k, v, "window", window=256, return_lse=True)
        _, lse_big = intra_llm_attn(q, k, v, "window", window=1024, return_lse=True)
    assert bool((lse_big >= lse_small - 1e-4).all())
    ref_small = oracle.masked_lse(q, k, torch.from_numpy(oracle.llm_window_mask(2048, 256)).cuda())
    ref_big = oracle.masked_lse(q, k, torch.from_numpy(oracle.llm_window_mask(2048, 1024)).cuda())
    assert float(((lse_big - lse_small) - (ref_big - ref_small)).abs().max()) <= 2 * LSE_ATOL


@pytest.fixture
def _launcher_choice_restored(lib):
    yield
    assert lib.intra_b200_test_force_path(0, 0) == 0


@pytest.mark.parametrize("no_tma,split", [(0, 1), (0, 2), (0, 4), (1, 0), (1, 1), (1, 2), (1, 4)],
                         ids=["row-owner", "split2", "split4", "no-tma", "no-tma-row-owner", "no-tma-split2", "no-tma-split4"])
def test_forced_kernel_paths(lib, _launcher_choice_restored, no_tma, split):
    """Every kernel variant the launcher can choose, forced through the library's test hook: the
    row-owner form and both softmax column splits for every pattern, including the combinations its
    heuristic never picks, and the cp.async row gathers where TMA boxes would have been used."""
    from intra_b200 import intra_image_attn, intra_llm_attn
    assert lib.intra_b200_test_force_path(no_tma, split) == 0
    with torch.no_grad():
        for family, pattern, S, H, Hkv, kw in (
                ("llm", "scatter", 2048, 4, 2, {"group_num": 2}), ("llm", "gather1", 2048, 3, 3, {"group_num": 8}),
                ("llm", "window", 1536, 4, 1, {"window": 576}), ("image", "scatter", 512 + 32 * 32, 2, 2, {"width": 32}),
                ("image", "gather0", 512 + 32 * 32, 2, 2, {"width": 32})):
            q, k, v = oracle.make_inputs(1, S, H, Hkv, seed=31, device="cuda")
            fn = intra_image_attn if family == "image" else intra_llm_attn
            out, lse = fn(q, k, v, pattern, strict=False, return_lse=True, **kw)
            mask = torch.from_numpy(oracle.build_mask(family, pattern, S, **kw)).cuda()
            _util.check_parity(out, oracle.masked_attention_fp32(q, k, v, mask), oracle.masked_attention_fp32(q, k, v.abs(), mask))
            assert float((lse - oracle.masked_lse(q, k, mask)).abs().max()) <= LSE_ATOL, (family, pattern)


@pytest.mark.parametrize("split", [1, 2, 4], ids=["row-owner", "split2", "split4"])
def test_items_of_one_key_tile_back_to_back(lib, _launcher_choice_restored, split):
    """Scatter with 128-token groups: every item of every CTA has a single key tile, so nothing but the
    hand-offs between the softmax warps, the MMA warps and the epilogue warps paces the pipeline from
    item to item (the case in which a role can run furthest ahead of another). Output and log-sum-exp
    against the oracle, and no bounded wait gave up."""
    from intra_b200 import intra_llm_attn
    assert lib.intra_b200_test_force_path(0, split) == 0
    S, G = 2048, 16
    q, k, v = oracle.make_inputs(4, S, 16, 8, seed=41, device="cuda")
    mask = torch.from_numpy(oracle.build_mask("llm", "scatter", S, group_num=G)).cuda()
    with torch.no_grad():
        for _ in range(3):
            out, lse = intra_llm_attn(q, k, v, "scatter", group_num=G, strict=False, return_lse=True)
    _util.check_parity(out, oracle.masked_attention_fp32(q, k, v, mask), oracle.masked_attention_fp32(q, k, v.abs(), mask))
    assert float((lse - oracle.masked_lse(q, k, mask)).abs().max()) <= LSE_ATOL
    assert _util.device_status(lib, 0, reset=True) == 0


def test_out_argument(lib):
    """out= writes into the caller's tensor (any layout the kernels accept) and refuses one that
    does not match."""
    from intra_b200 import intra_image_attn, intra_llm_attn
    q, k, v = oracle.make_inputs(1, 1024, 4, 2, seed=37, device="cuda")
    with torch.no_grad():
        want = intra_llm_attn(q, k, v, "scatter", group_num=4)
        out = torch.full_like(q, float("nan"))
        got = intra_llm_attn(q, k, v, "scatter", group_num=4, out=out)
        assert got is out and torch.equal(out, want)
        view = torch.zeros(1, 4, 1024, 128, dtype=torch.bfloat16, device="cuda").transpose(1, 2)   # (B, H, S, D) storage
        intra_llm_attn(q, k, v, "scatter", group_num=4, out=view)
        assert torch.equal(view, want)
        with pytest.raises(ValueError):
            intra_llm_attn(q, k, v, "scatter", group_num=4, out=torch.empty(1, 1024, 4, 64, dtype=torch.bfloat16, device="cuda"))
        with pytest.raises(ValueError):
            intra_llm_attn(q, k, v, "scatter", group_num=4, out=torch.empty_like(q, dtype=torch.float16))
        with pytest.raises(ValueError):
            intra_llm_attn(q, k, v, "scatter", group_num=4, out=q)
        both = torch.empty(2, 1024, 4, 128, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(ValueError, match="overlap"):             # an offset view of q's own storage
            intra_llm_attn(both[:1], k, v, "scatter", group_num=4, out=both.view(-1)[64:64 + q.numel()].view(q.shape))
        with pytest.raises(ValueError):                              # every head would write the same rows
            intra_llm_attn(q, k, v, "scatter", group_num=4, out=torch.empty(1, 1024, 1, 128, dtype=torch.bfloat16, device="cuda").expand(1, 1024, 4, 128))
        qi, ki, vi = oracle.make_inputs(1, 512 + 16 * 16, 2, 2, seed=38, device="cuda")
        wi = intra_image_attn(qi, ki, vi, "gather0", 16, strict=False)
        oi = torch.empty_like(qi)
        intra_image_attn(qi, ki, vi, "gather0", 16, strict=False, out=oi)
        assert torch.equal(oi, wi)
