"""Python entry points, drop-in for the reference's `intra_attn/interface.py`.

Same names, defaults, argument meaning and exceptions as the reference
(intra_attn/interface.py:17-66); the work is done by libintra_b200.so through its C ABI.
All functions take q, k, v of shape (batch, seqlen, heads, 128) in bfloat16 on a B200 and return the
attention output shaped, typed and laid out like q. k/v may have fewer heads than q (GQA) as long as
they divide the query heads. Forward only.
"""
from __future__ import annotations

import torch

from . import _loader
from ._loader import lib, strides3

LLM_PATTERNS = {"scatter": 0, "gather1": 1, "window": 4}
IMAGE_PATTERNS = {"scatter": 0, "gather0": 4}
TEXT_LEN = 512


def _check(q, k, v):
    """Argument checks of the reference (intra_attn/interface.py:17-23), plus the layout the
    library needs: the reference's kernels silently assume 128-element head stride and equal q/k row
    strides; here any batch/token/head strides are honoured as long as rows stay 16-byte aligned,
    and tensors that break that are made contiguous first."""
    for x in (q, k, v):
        if not x.is_cuda or x.dtype != torch.bfloat16 or x.shape[-1] != 128:
            raise ValueError("INTRA kernels need CUDA bfloat16 tensors with head_dim 128")
    if torch.is_grad_enabled() and any(x.requires_grad for x in (q, k, v)):
        raise RuntimeError("INTRA kernels are forward-only; call them under torch.no_grad()")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be (batch, seqlen, heads, 128)")
    if k.shape != v.shape or k.shape[:2] != q.shape[:2] or q.shape[2] % k.shape[2] != 0:
        raise ValueError(f"incompatible shapes q={tuple(q.shape)} k={tuple(k.shape)} v={tuple(v.shape)}")
    if k.device != q.device or v.device != q.device:
        raise ValueError("q, k, v must be on the same device")

    def usable(x):
        return (x.stride(-1) == 1 and x.data_ptr() % 16 == 0
                and all(x.stride(d) % 8 == 0 and x.stride(d) >= 0 for d in range(3)))

    return [x if usable(x) else x.contiguous() for x in (q, k, v)]


def _scale(q, softmax_scale):
    return q.shape[-1] ** -0.5 if softmax_scale is None else float(softmax_scale)


def _raise(status):
    msg = _loader.strerror(status)
    if status == _loader.ERR_CUDA:
        raise RuntimeError(f"intra_b200: {msg} (cudaError {lib.intra_b200_last_cuda_error()})")
    if status in (_loader.ERR_DEVICE, _loader.ERR_KERNEL):
        raise RuntimeError(f"intra_b200: {msg}")
    raise ValueError(f"intra_b200: {msg}")


def _byte_span(x):
    """[first, last) byte addresses a tensor with non-negative strides can touch."""
    last = sum((n - 1) * st for n, st in zip(x.shape, x.stride()) if n > 0)
    return x.data_ptr(), x.data_ptr() + (last + 1) * x.element_size()


def _empty_like(q, out=None, inputs=()):
    """The output tensor: the caller's `out` after checks, else a fresh tensor laid out like q."""
    if out is not None:
        if out.shape != q.shape or out.dtype != q.dtype or out.device != q.device:
            raise ValueError("out must match q in shape, dtype and device")
        if out.stride(-1) != 1 or any(out.stride(d) % 8 or out.stride(d) <= 0 for d in range(3)) or out.data_ptr() % 16:
            raise ValueError("out needs unit stride in the last dim, positive strides and 16-byte aligned rows")
        lo, hi = _byte_span(out)
        for x in inputs:
            xlo, xhi = _byte_span(x)
            if lo < xhi and xlo < hi:
                raise ValueError("out must not overlap q, k or v: other tiles still read them while it is written")
        return out
    out = torch.empty_like(q)
    if out.stride(-1) != 1 or any(out.stride(d) % 8 or out.stride(d) <= 0 for d in range(3)):
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    return out


# Validated call plans, keyed by everything the checks above look at (addresses, shapes, strides,
# dtypes, device, requires_grad). A serving loop or a layer stack calls with the same tensors over and
# over; at S = 4096 a call is 40 us of GPU time and the checks would cost as much on the host again.
_PLANS = {}
_PLANS_MAX = 512


def _plan(q, k, v, out):
    """(q, k, v, out or None, B, S, H, Hkv, q/k/v/out stride arrays or None for out) after the checks."""
    rg = q.requires_grad or k.requires_grad or v.requires_grad
    if rg and torch.is_grad_enabled():
        raise RuntimeError("INTRA kernels are forward-only; call them under torch.no_grad()")
    key = (q.data_ptr(), k.data_ptr(), v.data_ptr(), None if out is None else (out.data_ptr(), out.shape, out.stride(), out.dtype, out.device),
           q.shape, k.shape, v.shape, q.stride(), k.stride(), v.stride(), q.dtype, k.dtype, v.dtype, q.device, k.device, v.device)
    plan = _PLANS.get(key)
    if plan is not None:
        return (q, k, v) + plan
    q2, k2, v2 = _check(q, k, v)
    copied = q2 is not q or k2 is not k or v2 is not v        # fresh contiguous copies: nothing to remember
    if out is not None:
        _empty_like(q2, out, (q2, k2, v2))
    B, S, H, _ = q2.shape
    plan = (B, S, H, k2.shape[2], strides3(q2), strides3(k2), strides3(v2), None if out is None else strides3(out))
    if not copied:
        if len(_PLANS) >= _PLANS_MAX:
            _PLANS.clear()
        _PLANS[key] = plan
    return (q2, k2, v2) + plan


def intra_llm_attn(q, k, v, pattern="scatter", group_num=8, window=576, softmax_scale=None, *, strict=True,
                   return_lse=False, out=None):
    """Causal prefill attention for language models.

    pattern="scatter": token i attends to earlier tokens j with j % group_num == i % group_num.
    pattern="gather1": groups are segments of group_num tokens, segment s in group s % group_num.
    pattern="window":  each 64-query block attends to itself and the preceding window - 64 tokens.

    Any seqlen works for scatter and window; gather1 keeps the reference's contract of
    group_num=8 and seqlen % 64 == 0 (intra_attn/interface.py:41-42). `strict=False` (not in the
    reference) lifts that restriction: the kernels handle Gather-1 for any group_num and seqlen.
    `return_lse=True` (not in the reference, whose kernels compute the value and drop it) returns
    `(out, lse)` with lse of shape (batch, heads, seqlen), float32: the log of each query's softmax
    denominator, which is what merging attention over disjoint key sets needs. `out=` (not in the
    reference, which always allocates) writes into a tensor of the caller's; it must not alias q, k, v.
    """
    q, k, v, B, S, H, Hkv, qs, ks, vs, os_ = _plan(q, k, v, out)
    if strict and pattern == "gather1" and (group_num != 8 or S % (group_num * group_num)):
        raise ValueError(f"gather1 needs group_num=8 and seqlen % 64 == 0, got G={group_num}, S={S}")
    pid = LLM_PATTERNS[pattern]
    if out is None:
        out = _empty_like(q)
        os_ = strides3(out)
    dev = q.device
    tail = (qs, ks, vs, os_, pid, int(group_num), int(window), _scale(q, softmax_scale), dev.index,
            torch.cuda.current_stream(dev).cuda_stream)
    if return_lse:
        lse = torch.empty((B, H, S), dtype=torch.float32, device=dev)
        rc = lib.intra_b200_fwd_llm_lse(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                        B, S, H, Hkv, *tail)
    else:
        rc = lib.intra_b200_fwd_llm(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, H, Hkv, *tail)
    if rc != 0:
        _raise(rc)
    return (out, lse) if return_lse else out


def intra_image_attn(q, k, v, pattern="scatter", width=64, softmax_scale=None, *, strict=True, return_lse=False,
                     out=None):
    """Bidirectional attention for FLUX-style sequences: 512 text tokens followed by a
    width x width grid of image tokens.

    pattern="scatter": 8 groups, image token (r, c) in group (r % 2) * 4 + c % 4; text chunks of
                       64 tokens ride with groups 0..7; all text keys are always visible.
    pattern="gather0": each 8 x 8 image patch attends to a 16 x 16 window around it plus all text.

    width must be 64 or 128 as in the reference (intra_attn/interface.py:60-63); `strict=False` (not in
    the reference) accepts any width that is a multiple of 8 and at least 16. `return_lse=True` returns
    `(out, lse)` and `out=` writes into the caller's tensor, as in intra_llm_attn.
    """
    q, k, v, B, S, H, Hkv, qs, ks, vs, os_ = _plan(q, k, v, out)
    if not strict and (width < 16 or width % 8):
        raise ValueError("width must be a multiple of 8 and at least 16")
    if strict and width not in (64, 128):
        raise ValueError("image kernels are compiled for width 64 and 128")
    if S != TEXT_LEN + width * width:
        raise ValueError(f"expected {TEXT_LEN} text + {width}x{width} image tokens, got {S}")
    if Hkv != H:
        raise ValueError("image attention is multi-head: k/v need as many heads as q")
    pid = IMAGE_PATTERNS[pattern]
    if out is None:
        out = _empty_like(q)
        os_ = strides3(out)
    dev = q.device
    tail = (qs, ks, vs, os_, pid, int(width), _scale(q, softmax_scale), dev.index,
            torch.cuda.current_stream(dev).cuda_stream)
    if return_lse:
        lse = torch.empty((B, H, S), dtype=torch.float32, device=dev)
        rc = lib.intra_b200_fwd_image_lse(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                          B, S, H, *tail)
    else:
        rc = lib.intra_b200_fwd_image(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, H, *tail)
    if rc != 0:
        _raise(rc)
    return (out, lse) if return_lse else out


def device_status(device=None, reset=False):
    """Synchronise `device` and return the status word its kernels write when a bounded wait gives
    up (0 = healthy; otherwise 100 + the id of the first wait that ran out since the last reset). The
    attention calls never poll it, and a recorded failure does not change later launches: a caller that
    wants to know checks here, e.g. once per step. Raises nothing; callers decide."""
    import ctypes
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    word = ctypes.c_int(0)
    lib.intra_b200_device_status(dev, ctypes.byref(word), 1 if reset else 0)
    return word.value
