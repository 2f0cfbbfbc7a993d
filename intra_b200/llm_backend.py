"""`transformers` attention-backend callable built on `intra_llm_attn`.

The reference ships a PyTorch restatement of the kernel's language-model patterns as an
ALL_ATTENTION_FUNCTIONS-style callable (experiments/llm/intra_token_attn.py:112-134): two Scatter
layers, then two 64-aligned-window layers, repeating, with dense attention for single-token decode
steps because the patterns are prefill-only. This module offers the same callable with the prefill
running on the B200 kernels: query/key/value arrive as (B, H, S, D) and are handed to the kernel as
(B, S, H, D) views without copies. The decode step stays what it is in the reference - one dense SDPA
call over the cache, outside the scope of the sparse kernels.

    from transformers import AttentionInterface
    AttentionInterface.register("intra_b200", make_intra_attention())
    model = AutoModelForCausalLM.from_pretrained(..., attn_implementation="intra_b200")
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .interface import intra_llm_attn

NUM_GROUPS = 8          # intra_token_attn.py:22-24
WINDOW_BACK = 512
WINDOW_CHUNK = 64


def layer_masktype(layer_idx: int) -> int:
    """Kernel mask id of a layer: 0 (Scatter) for layer_idx % 4 in {0, 1}, 4 (window) otherwise
    (intra_token_attn.py:112-114)."""
    return 0 if layer_idx % 4 in (0, 1) else 4


def make_intra_attention(num_groups: int = NUM_GROUPS, back: int = WINDOW_BACK, chunk: int = WINDOW_CHUNK,
                         force_masktype=None):
    """Returns `fn(module, query, key, value, attention_mask=None, scaling=None, dropout=0.0, **kw)`
    -> (output (B, S, H, D), None), the signature transformers expects of an attention backend."""
    if chunk != 64:
        raise ValueError("the window kernel aligns its lookback to 64-query blocks")
    window = back + chunk      # a 64-query block sees itself plus `back` earlier tokens

    def intra_attention_forward(module, query, key, value, attention_mask=None, scaling=None, dropout=0.0,
                                **kwargs):
        if query.shape[2] == 1:          # decode step: dense over the cache, as the reference does
            rep = query.shape[1] // key.shape[1]
            k2 = key.repeat_interleave(rep, dim=1) if rep > 1 else key
            v2 = value.repeat_interleave(rep, dim=1) if rep > 1 else value
            am = attention_mask[:, :, :, : k2.shape[-2]] if attention_mask is not None else None
            o = F.scaled_dot_product_attention(query, k2, v2, attn_mask=am, scale=scaling, is_causal=False)
            return o.transpose(1, 2).contiguous(), None
        mt = force_masktype if force_masktype is not None else layer_masktype(getattr(module, "layer_idx", 0))
        q, k, v = (x.transpose(1, 2) for x in (query, key, value))
        with torch.no_grad():
            if mt == 0:
                out = intra_llm_attn(q, k, v, "scatter", group_num=num_groups, softmax_scale=scaling)
            else:
                out = intra_llm_attn(q, k, v, "window", window=window, softmax_scale=scaling)
        return out, None

    return intra_attention_forward
