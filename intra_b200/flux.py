"""Attention call of a FLUX-style joint-attention layer on top of `intra_image_attn`.

The reference's only production caller is its diffusers attention processor
(experiments/flux/intra_processor.py:54-169): after projections, QK-norm and RoPE it holds
query/key/value as (B, H, S, D) tensors, S = 512 text + width^2 image tokens, hands (B, S, H, D)
*views* of them to the kernel and alternates the two image patterns every two layers. This module
carries exactly that part - shape checks, the layer schedule and the view-based call - so that a
processor can be pointed at this package without diffusers being involved here. The kernel reads the
transposed views in place (every batch/token/head stride is honoured); nothing is copied.
Training paths of the reference processor (masked SDPA under autograd) are out of scope.
"""
from __future__ import annotations

import math

import torch

from .interface import TEXT_LEN, intra_image_attn

KERNEL_WIDTHS = (64, 128)   # latent sides of 1024^2 and 2048^2 images (intra_processor.py:30)


def latent_width(seq_len: int) -> int:
    """Side of the square latent grid behind the 512 text tokens (intra_processor.py:47-51)."""
    width = math.isqrt(seq_len - TEXT_LEN)
    if width * width != seq_len - TEXT_LEN or width % 8:
        raise ValueError(f"expected 512 text + a square latent grid with side % 8 == 0, got {seq_len}")
    return width


def layer_pattern(layer_index: int) -> str:
    """Pattern of attention layer `layer_index`: Scatter, Scatter, Gather 0, Gather 0, ...
    (intra_processor.py:162-169)."""
    return "gather0" if layer_index % 4 in (2, 3) else "scatter"


def flux_joint_attention(query, key, value, pattern: str, softmax_scale=None):
    """query, key, value: (B, H, S, 128) bf16 CUDA tensors as a FLUX attention processor holds them.
    Returns the attention output in the same (B, H, S, 128) layout (a view of a (B, S, H, 128) tensor).
    Forward only; call under torch.no_grad()."""
    if query.dim() != 4:
        raise ValueError("expected (batch, heads, seq, head_dim) tensors")
    width = latent_width(query.shape[2])
    scale = 1.0 / math.sqrt(query.shape[-1]) if softmax_scale is None else softmax_scale
    out = intra_image_attn(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2),
                           pattern=pattern, width=width, softmax_scale=scale)
    return out.transpose(1, 2)
