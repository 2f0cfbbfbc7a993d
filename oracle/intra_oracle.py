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
def llm_scatter_mask(S: int, group_num: int = 8) -> np.ndarray:
    """mask[q, k] = k <= q and k % G == q % G   (intra_attn/reference.py:14-17)."""
    i = np.arange(S)
    grp = i % group_num
    return (grp[:, None] == grp[None, :]) & (i[None, :] <= i[:, None])


def llm_gather1_mask(S: int, group_num: int = 8) -> np.ndarray:
    """Segments of G tokens, segment s in group s % G, causal  (intra_attn/reference.py:20-24)."""
    i = np.arange(S)
    grp = (i // group_num) % group_num
    return (grp[:, None] == grp[None, :]) & (i[None, :] <= i[:, None])


def llm_window_mask(S: int, window: int = 576, block: int = 64) -> np.ndarray:
    """Each `block`-query block sees keys from (block start - (window - block)), clamped at 0, up
    to the query itself  (intra_attn/reference.py:27-32)."""
    i = np.arange(S)
    first = np.maximum((i // block) * block - (window - block), 0)
    k = i[None, :]
    return (k >= first[:, None]) & (k <= i[:, None])


def image_group_ids(width: int, text_len: int = TEXT_LEN) -> np.ndarray:
    """Group of every token: text chunk j (text_len/8 tokens) rides with image group j; image
    token (r, c) is in group (r % 2) * 4 + c % 4  (intra_attn/reference.py:36-46)."""
    text = np.arange(text_len) // (text_len // 8)
    r, c = np.divmod(np.arange(width * width), width)
    return np.concatenate([text, (r % 2) * 4 + (c % 4)])


def image_scatter_mask(width: int, text_len: int = TEXT_LEN) -> np.ndarray:
    """Every query sees all text keys plus the image keys of its own group
    (intra_attn/reference.py:49-53)."""
    g = image_group_ids(width, text_len)
    S = g.size
    key_is_text = np.arange(S) < text_len
    return key_is_text[None, :] | (g[:, None] == g[None, :])


def gather0_window_start(idx: np.ndarray, n_patch: int, patch: int = 8, window: int = 16) -> np.ndarray:
    """First row/column of the window of patch index idx  (intra_attn/reference.py:65-68)."""
    s = idx * patch - (window - patch) // 2
    s = np.where(idx == 0, 0, s)
    return np.where(idx == n_patch - 1, idx * patch - (window - patch), s)


def image_gather0_mask(width: int, text_len: int = TEXT_LEN, patch: int = 8, window: int = 16) -> np.ndarray:
    """Image queries: all text keys + a window x window block of image keys around their patch;
    text queries keep their Scatter rows  (intra_attn/reference.py:56-74)."""
    m = image_scatter_mask(width, text_len)
    n_patch = width // patch
    r, c = np.divmod(np.arange(width * width), width)
    r0 = gather0_window_start(r // patch, n_patch, patch, window)
    c0 = gather0_window_start(c // patch, n_patch, patch, window)
    rows_ok = (r[None, :] >= r0[:, None]) & (r[None, :] < r0[:, None] + window)
    cols_ok = (c[None, :] >= c0[:, None]) & (c[None, :] < c0[:, None] + window)
    m[text_len:, text_len:] = rows_ok & cols_ok
    return m


def build_mask(family: str, pattern: str, S: int, group_num: int = 8, window: int = 576,
               width: int = 64) -> np.ndarray:
    """Mask for the public API's (family, pattern) names (intra_attn/interface.py:12-13)."""
    if family == "llm":
        if pattern == "scatter":
            return llm_scatter_mask(S, group_num)
        if pattern == "gather1":
            return llm_gather1_mask(S, group_num)
        if pattern == "window":
            return llm_window_mask(S, window)
    elif family == "image":
        assert S == TEXT_LEN + width * width
        if pattern == "scatter":
            return image_scatter_mask(width)
        if pattern == "gather0":
            return image_gather0_mask(width)
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
def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask, softmax_scale=None):
    """fp32 dense-mask attention, the reference's oracle  (intra_attn/reference.py:78-83):
    q, k, v are (B, S, H, D) with H % H_kv == 0; mask is (S, S) bool; result in q's dtype."""
    if not torch.is_tensor(mask):
        mask = torch.from_numpy(np.ascontiguousarray(mask))
    mask = mask.to(q.device)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    out = F.scaled_dot_product_attention(qf, kf, vf, attn_mask=mask, scale=softmax_scale,
                                         enable_gqa=qf.shape[1] != kf.shape[1])
    return out.permute(0, 2, 1, 3).to(q.dtype)


def masked_attention_rows(q, k, v, mask, softmax_scale=None, rows: int = 1024):
    """Same result computed with an explicit softmax over row slabs of the mask, so that long
    sequences fit in memory and the SDPA call above has an independent cross-check."""
    if not torch.is_tensor(mask):
        mask = torch.from_numpy(np.ascontiguousarray(mask))
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
    kf = k.float().permute(0, 2, 3, 1)                       # B, Hkv, D, S
    vf = v.float().permute(0, 2, 1, 3)                       # B, Hkv, S, D
    rep = H // Hkv
    out = torch.empty_like(q)
    for r0 in range(0, S, rows):
        r1 = min(r0 + rows, S)
        qs = q[:, r0:r1].float().permute(0, 2, 1, 3).reshape(B, Hkv, rep, r1 - r0, D)
        s = torch.matmul(qs, kf[:, :, None]) * scale         # B, Hkv, rep, rows, S
        s = s.masked_fill(~mask[r0:r1].to(s.device), float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.matmul(p, vf[:, :, None])                  # B, Hkv, rep, rows, D
        out[:, r0:r1] = o.reshape(B, H, r1 - r0, D).permute(0, 2, 1, 3).to(q.dtype)
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
