"""Head-sharded launcher: one process per GPU, each owning a contiguous block of KV-head groups.

Attention is independent per (batch, query head) and a KV head is shared only by its H / H_kv query
heads (the reference indexes it as `bidh / h_h_k_ratio`, csrc/flash_attn/src/flash_fwd_kernel.h:5338),
so sharding by KV-head group needs no exchange step: every rank runs the single-GPU kernel on its
own heads. Outputs stay head-sharded unless the caller asks for the full tensor, in which case one
NCCL all-gather over NVLink assembles it. The reference has no multi-GPU path; this is new.

Failures are agreed on the host: before any collective the ranks reduce a success flag, so a rank whose
local launch failed makes every rank raise instead of leaving the others stuck in the all-gather.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def head_slices(H: int, Hkv: int, rank: int, world: int) -> Tuple[slice, slice]:
    """Query-head and KV-head slices owned by `rank`. KV-head groups are dealt in contiguous blocks."""
    if Hkv % world != 0:
        raise ValueError(f"{Hkv} KV heads cannot be split over {world} ranks")
    if H % Hkv != 0:
        raise ValueError("query heads must be a multiple of KV heads")
    kv_per = Hkv // world
    rep = H // Hkv
    return (slice(rank * kv_per * rep, (rank + 1) * kv_per * rep), slice(rank * kv_per, (rank + 1) * kv_per))


def shard_heads(q, k, v, rank: int, world: int):
    """This rank's head block of full (B, S, H, D) / (B, S, H_kv, D) tensors (views, no copy)."""
    qs, ks = head_slices(q.shape[2], k.shape[2], rank, world)
    return q[:, :, qs], k[:, :, ks], v[:, :, ks]


def _agree_ok(ok: bool, group) -> bool:
    if group is None and not (dist.is_available() and dist.is_initialized()):
        return ok
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
    backend = dist.get_backend(group)
    if backend == "nccl":
        flag = flag.cuda()
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())


def gather_heads(out_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather head-sharded outputs (B, S, H/n, D) into the full (B, S, H, D) tensor."""
    world = dist.get_world_size(group)
    B, S, Hl, D = out_local.shape
    parts = torch.empty((world * B, S, Hl, D), dtype=out_local.dtype, device=out_local.device)
    dist.all_gather_into_tensor(parts, out_local.contiguous(), group=group)
    return parts.view(world, B, S, Hl, D).permute(1, 2, 0, 3, 4).reshape(B, S, world * Hl, D)


def sharded_attn(local_fn: Callable[..., torch.Tensor], q_local, k_local, v_local, *args,
                 group=None, gather_output: bool = False, **kwargs) -> torch.Tensor:
    """Run `local_fn(q_local, k_local, v_local, *args, **kwargs)` on this rank's heads.

    `local_fn` is `intra_llm_attn` or `intra_image_attn` (tests inject a stand-in). With
    gather_output=True every rank returns the full-head tensor; otherwise its own block.
    """
    err: Optional[BaseException] = None
    out_local = None
    try:
        out_local = local_fn(q_local, k_local, v_local, *args, **kwargs)
    except Exception as e:  # agreed on below, then re-raised on every rank
        err = e
    distributed = dist.is_available() and dist.is_initialized()
    if distributed and not _agree_ok(err is None, group):
        raise RuntimeError("head-sharded attention failed on at least one rank"
                           + (f" (this rank: {err})" if err is not None else "")) from err
    if err is not None:
        raise err
    if gather_output and distributed and dist.get_world_size(group) > 1:
        return gather_heads(out_local, group)
    return out_local


def intra_llm_attn_sharded(q_local, k_local, v_local, pattern="scatter", group_num=8, window=576, softmax_scale=None,
                           group=None, gather_output=False):
    """`intra_llm_attn` on this rank's KV-head groups; see `sharded_attn`."""
    from .interface import intra_llm_attn
    return sharded_attn(intra_llm_attn, q_local, k_local, v_local, pattern, group_num=group_num, window=window,
                        softmax_scale=softmax_scale, group=group, gather_output=gather_output)


def intra_image_attn_sharded(q_local, k_local, v_local, pattern="scatter", width=64, softmax_scale=None,
                             group=None, gather_output=False):
    """`intra_image_attn` on this rank's heads; see `sharded_attn`."""
    from .interface import intra_image_attn
    return sharded_attn(intra_image_attn, q_local, k_local, v_local, pattern, width=width,
                        softmax_scale=softmax_scale, group=group, gather_output=gather_output)
