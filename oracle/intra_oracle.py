"""CPU oracle for the INTRA forward sparse-attention path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, what the reference specifies for the path: the five dense
boolean attention masks and fp32 masked attention. Only the tests, the smoke check and the
CPU-baseline leg of the benchmark may import it; the product (the `intra_b200` package and its
CUDA library) never does.

Each function cites the reference lines it follows. The masks here are written from the
per-token predicates (group ids, window bounds) rather than from the reference's expressions, and
they are pinned to the reference: `tests/golden/make_golden.py` runs the reference's own
`intra_attn/reference.py` and stores digests of its masks and its attention outputs on seeded
inputs; `tests/test_oracle.py` checks this module against those stored values.
"""
from __future__ import annotations

import hashlib
import math

import numpy as np
import torch
import torch.nn.functional as F

TEXT_LEN = 512  # intra_attn/reference.py:10


# ------------------------------------------------------------------------------------- masks
# Every builder takes an optional `rows` ((r0, r1) or an array of query ids): only those mask rows are
# built, against all S keys, so that sequences whose S x S mask does not fit in memory can be checked slab by slab. The
# predicates are the same expressions either way; tests/test_oracle.py checks slab == slice of the full
# mask bit for bit.
def _query_ids(S: int, rows):
    """Query token ids of the mask rows to build: all, a (r0, r1) range, or an explicit index array."""
    if rows is None:
        return np.arange(S)
    if isinstance(rows, tuple):
        r0, r1 = rows
        assert 0 <= r0 <= r1 <= S
        return np.arange(r0, r1)
    qi = np.asarray(rows, dtype=np.int64)
    assert qi.ndim == 1 and (qi.size == 0 or (qi.min() >= 0 and qi.max() < S))
    return qi


def llm_scatter_mask(S: int, group_num: int = 8, rows=None) -> np.ndarray:
    """mask[q, k] = k <= q and k % G == q % G   (intra_attn/reference.py:14-17)."""
    qi, ki = _query_ids(S, rows), np.arange(S)
    return ((qi % group_num)[:, None] == (ki % group_num)[None, :]) & (ki[None, :] <= qi[:, None])


def llm_gather1_mask(S: int, group_num: int = 8, rows=None) -> np.ndarray:
    """Segments of G tokens, segment s in group s % G, causal  (intra_attn/reference.py:20-24)."""
    qi, ki = _query_ids(S, rows), np.arange(S)
    grp = lambda i: (i // group_num) % group_num
    return (grp(qi)[:, None] == grp(ki)[None, :]) & (ki[None, :] <= qi[:, None])


def llm_window_mask(S: int, window: int = 576, block: int = 64, rows=None) -> np.ndarray:
    """Each `block`-query block sees keys from (block start - (window - block)), clamped at 0, up
    to the query itself  (intra_attn/reference.py:27-32)."""
    qi, ki = _query_ids(S, rows), np.arange(S)
    first = np.maximum((qi // block) * block - (window - block), 0)
    return (ki[None, :] >= first[:, None]) & (ki[None, :] <= qi[:, None])


def image_group_ids(width: int, text_len: int = TEXT_LEN) -> np.ndarray:
    """Group of every token: text chunk j (text_len/8 tokens) rides with image group j; image
    token (r, c) is in group (r % 2) * 4 + c % 4  (intra_attn/reference.py:36-46)."""
    text = np.arange(text_len) // (text_len // 8)
    r, c = np.divmod(np.arange(width * width), width)
    return np.concatenate([text, (r % 2) * 4 + (c % 4)])


def image_scatter_mask(width: int, text_len: int = TEXT_LEN, rows=None) -> np.ndarray:
    """Every query sees all text keys plus the image keys of its own group
    (intra_attn/reference.py:49-53)."""
    g = image_group_ids(width, text_len)
    S = g.size
    qi = _query_ids(S, rows)
    key_is_text = np.arange(S) < text_len
    return key_is_text[None, :] | (g[qi][:, None] == g[None, :])


def gather0_window_start(idx: np.ndarray, n_patch: int, patch: int = 8, window: int = 16) -> np.ndarray:
    """First row/column of the window of patch index idx  (intra_attn/reference.py:65-68)."""
    s = idx * patch - (window - patch) // 2
    s = np.where(idx == 0, 0, s)
    return np.where(idx == n_patch - 1, idx * patch - (window - patch), s)


def image_gather0_mask(width: int, text_len: int = TEXT_LEN, patch: int = 8, window: int = 16, rows=None) -> np.ndarray:
    """Image queries: all text keys + a window x window block of image keys around their patch;
    text queries keep their Scatter rows  (intra_attn/reference.py:56-74)."""
    S = text_len + width * width
    qi = _query_ids(S, rows)
    m = image_scatter_mask(width, text_len, rows=rows)
    n_patch = width // patch
    r, c = np.divmod(np.arange(width * width), width)
    r0 = gather0_window_start(r // patch, n_patch, patch, window)
    c0 = gather0_window_start(c // patch, n_patch, patch, window)
    img = qi[qi >= text_len] - text_len                     # image queries of the slab
    rows_ok = (r[None, :] >= r0[img][:, None]) & (r[None, :] < r0[img][:, None] + window)
    cols_ok = (c[None, :] >= c0[img][:, None]) & (c[None, :] < c0[img][:, None] + window)
    m[qi >= text_len, text_len:] = rows_ok & cols_ok
    return m


def build_mask(family: str, pattern: str, S: int, group_num: int = 8, window: int = 576,
               width: int = 64, rows=None) -> np.ndarray:
    """Mask for the public API's (family, pattern) names (intra_attn/interface.py:12-13)."""
    if family == "llm":
        if pattern == "scatter":
            return llm_scatter_mask(S, group_num, rows=rows)
        if pattern == "gather1":
            return llm_gather1_mask(S, group_num, rows=rows)
        if pattern == "window":
            return llm_window_mask(S, window, rows=rows)
    elif family == "image":
        assert S == TEXT_LEN + width * width
        if pattern == "scatter":
            return image_scatter_mask(width, rows=rows)
        if pattern == "gather0":
            return image_gather0_mask(width, rows=rows)
    raise KeyError((family, pattern))


def mask_digest(mask: np.ndarray) -> dict:
    """Order-sensitive digest of a boolean mask: sha256 of its packed bits, popcount, and a
    weighted row-sum checksum."""
    m = np.ascontiguousarray(mask, dtype=bool)
    rows = m.sum(axis=1, dtype=np.int64)
    return {
        "shape": list(m.shape),
        "pairs": int(rows.sum()),
        "row_checksum": int((rows * (np.arange(m.shape[0], dtype=np.int64) + 1)).sum()),
        "sha256": hashlib.sha256(np.packbits(m, axis=None).tobytes()).hexdigest(),
    }


# ------------------------------------------------------------------------- attended pair counts
def pair_count(family: str, pattern: str, S: int, group_num: int = 8, window: int = 576,
               width: int = 64) -> int:
    """Number of attended (query, key) pairs = popcount of the mask, in closed form."""
    if family == "llm":
        if pattern in ("scatter", "gather1"):
            total = 0
            for g in range(group_num):
                if pattern == "scatter":
                    n = S // group_num + (1 if g < S % group_num else 0)
                else:
                    span = group_num * group_num
                    n = (S // span) * group_num + min(max(S % span - g * group_num, 0), group_num)
                total += n * (n + 1) // 2
            return total
        if pattern == "window":
            total = 0
            for b in range((S + 63) // 64):
                first = max(64 * b - (window - 64), 0)
                lo, hi = 64 * b, min(64 * b + 64, S)
                n = hi - lo
                total += n * (lo - first) + n * (n + 1) // 2
            return total
    else:
        n_img = width * width // 8
        if pattern == "scatter":
            return S * (TEXT_LEN + n_img)
        if pattern == "gather0":
            return TEXT_LEN * (TEXT_LEN + n_img) + width * width * (TEXT_LEN + 256)
    raise KeyError((family, pattern))


# -------------------------------------------------------------------------------- attention
def masked_attention_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask, softmax_scale=None):
    """fp32 dense-mask attention as the reference's oracle computes it (intra_attn/reference.py:78-82),
    before its final rounding to the input dtype: q, k, v are (B, S, H, D) with H % H_kv == 0; mask is
    (S, S) bool; fp32 result (B, S, H, D)."""
    if not torch.is_tensor(mask):
        mask = torch.from_numpy(np.ascontiguousarray(mask))
    mask = mask.to(q.device)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    out = F.scaled_dot_product_attention(qf, kf, vf, attn_mask=mask, scale=softmax_scale,
                                         enable_gqa=qf.shape[1] != kf.shape[1])
    return out.permute(0, 2, 1, 3)


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask, softmax_scale=None):
    """The reference's oracle  (intra_attn/reference.py:78-83): the above, rounded to q's dtype."""
    return masked_attention_fp32(q, k, v, mask, softmax_scale).to(q.dtype)


def masked_attention_slab(q_rows, k, v, mask_rows, softmax_scale=None, with_spread=False):
    """Attention of a slab of query rows against all keys with an explicit fp32 softmax:
    q_rows (B, R, H, D), k / v (B, S, H_kv, D), mask_rows (R, S) bool. Returns (out fp32 (B, R, H, D),
    lse fp32 (B, H, R)). Needs no S x S mask, so it reaches sequence lengths the SDPA form cannot, and
    it is an independent statement of the same arithmetic (tests/test_oracle.py compares the two).
    with_spread=True appends sum_j p_j |v_j| (fp32, shaped like out): the scale of the terms that were
    added up, against which a rounding error of the probabilities has to be judged."""
    if not torch.is_tensor(mask_rows):
        mask_rows = torch.from_numpy(np.ascontiguousarray(mask_rows))
    B, R, H, D = q_rows.shape
    Hkv = k.shape[2]
    rep = H // Hkv
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
    kf = k.float().permute(0, 2, 3, 1)                       # B, Hkv, D, S
    vf = v.float().permute(0, 2, 1, 3)                       # B, Hkv, S, D
    qs = q_rows.float().permute(0, 2, 1, 3).reshape(B, Hkv, rep, R, D)
    s = torch.matmul(qs, kf[:, :, None]) * scale             # B, Hkv, rep, R, S
    s = s.masked_fill(~mask_rows.to(s.device), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    shape = lambda o: o.reshape(B, H, R, D).permute(0, 2, 1, 3)
    out = shape(torch.matmul(p, vf[:, :, None]))             # B, R, H, D
    if with_spread:
        return out, lse.reshape(B, H, R), shape(torch.matmul(p, vf.abs()[:, :, None]))
    return out, lse.reshape(B, H, R)


def masked_attention_rows(q, k, v, mask, softmax_scale=None, rows: int = 1024):
    """Same result as masked_attention computed slab by slab with the explicit softmax above, so that
    long sequences fit in memory and the SDPA call has an independent cross-check."""
    if not torch.is_tensor(mask):
        mask = torch.from_numpy(np.ascontiguousarray(mask))
    S = q.shape[1]
    out = torch.empty_like(q)
    for r0 in range(0, S, rows):
        r1 = min(r0 + rows, S)
        out[:, r0:r1] = masked_attention_slab(q[:, r0:r1], k, v, mask[r0:r1], softmax_scale)[0].to(q.dtype)
    return out


def masked_lse(q, k, mask, softmax_scale=None, rows: int = 1024):
    """log(sum_j exp(scale * q_i . k_j)) over the keys the mask lets query i attend, fp32, shape
    (B, H, S): the `softmax_lse` the reference's bindings return (csrc/flash_attn/flash_api.cpp:470,
    551) in the layout of its dense kernels."""
    if not torch.is_tensor(mask):
        mask = torch.from_numpy(np.ascontiguousarray(mask))
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
    kf = k.float().permute(0, 2, 3, 1)                       # B, Hkv, D, S
    rep = H // Hkv
    out = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    for r0 in range(0, S, rows):
        r1 = min(r0 + rows, S)
        qs = q[:, r0:r1].float().permute(0, 2, 1, 3).reshape(B, Hkv, rep, r1 - r0, D)
        s = torch.matmul(qs, kf[:, :, None]) * scale         # B, Hkv, rep, rows, S
        s = s.masked_fill(~mask[r0:r1].to(s.device), float("-inf"))
        out[:, :, r0:r1] = torch.logsumexp(s, dim=-1).reshape(B, H, r1 - r0)
    return out


def make_inputs(B, S, H, Hkv, seed=0, device="cpu", D=128):
    """Seeded i.i.d. N(0, 1) bf16 q, k, v like the reference's test and benchmark inputs
    (tests/test_kernel.py:17-20, benchmarks/bench_kernel.py:45-49). Always drawn on the CPU so the
    same seed gives the same tensors on every machine."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, S, H, D, generator=g, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, generator=g, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, generator=g, dtype=torch.float32).to(torch.bfloat16)
    return q.to(device), k.to(device), v.to(device)
