"""Head-sharded launcher: one process per GPU, each owning a contiguous block of KV-head groups.

Attention is independent per (batch, query head) and a KV head is shared only by its H / H_kv query
heads (the reference indexes it as `bidh / h_h_k_ratio`, csrc/flash_attn/src/flash_fwd_kernel.h:5338),
so sharding by KV-head group needs no exchange step: every rank runs the single-GPU kernel on its
own heads. Outputs stay head-sharded unless the caller asks for the full tensor, in which case one
NCCL all-gather over NVLink brings the blocks together and a copy kernel of this library puts them in
(batch, token, head, 128) order. The reference has no multi-GPU path; this is new.

Without `gather_output` a call is exactly the local launch: no collective, no host synchronisation.
With it, the ranks first agree (one small all-reduce, read on the host) that every local launch was
accepted, so that a rank whose call raised makes every rank raise instead of leaving the others stuck
in the all-gather. The agreement sees only errors raised before the launch; a kernel that gives up on
a bounded wait reports asynchronously through `intra_b200.interface.device_status`, which callers poll
when they choose to (e.g. once per step).
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


def _distributed(group) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def _agree_ok(ok: bool, group) -> bool:
    """True iff every rank of the group passed ok=True. One all-reduce and one host read."""
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
    if dist.get_backend(group) == "nccl":
        flag = flag.cuda()
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())


def interleave_heads(parts: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(world, B, S, Hl, D) rank-major blocks -> (B, S, world * Hl, D). On a GPU the copy is the library's
    own kernel (`intra_b200_interleave_heads`); on the CPU (tests with gloo ranks) it is a torch copy."""
    world, B, S, Hl, D = parts.shape
    if out is None:
        out = torch.empty((B, S, world * Hl, D), dtype=parts.dtype, device=parts.device)
    if parts.is_cuda:
        from ._loader import lib
        rc = lib.intra_b200_interleave_heads(parts.data_ptr(), out.data_ptr(), world, B * S, Hl * D * parts.element_size(),
                                             parts.device.index, torch.cuda.current_stream(parts.device).cuda_stream)
        if rc != 0:
            from .interface import _raise
            _raise(rc)
    else:
        out.view(B, S, world, Hl, D).copy_(parts.permute(1, 2, 0, 3, 4))
    return out


class GatherHandle:
    """An all-gather of head-sharded outputs running on a side stream. `wait()` makes the caller's
    current stream wait for it (no host synchronisation) and returns the full (B, S, H, D) tensor."""

    def __init__(self, full, event, keep):
        self._full, self._event, self._keep = full, event, keep

    def wait(self) -> torch.Tensor:
        if self._event is not None:
            torch.cuda.current_stream(self._full.device).wait_event(self._event)
            for t in self._keep:                        # their memory may be reused from this stream on
                t.record_stream(torch.cuda.current_stream(self._full.device))
        self._keep = ()
        return self._full


_side_streams = {}


def gather_heads_async(out_local: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> GatherHandle:
    """Start all-gathering head-sharded outputs (B, S, H/n, D) into the full (B, S, H, D) tensor on a side
    stream, so that the caller's next attention call overlaps the transfer. The side stream first waits
    for the work already queued on the caller's stream (the call that produced out_local)."""
    world = dist.get_world_size(group)
    B, S, Hl, D = out_local.shape
    src = out_local.contiguous()
    if not out_local.is_cuda:
        parts = torch.empty((world, B, S, Hl, D), dtype=src.dtype)
        dist.all_gather_into_tensor(parts.view(world * B, S, Hl, D), src, group=group)
        return GatherHandle(interleave_heads(parts, out), None, ())
    dev = out_local.device
    cur = torch.cuda.current_stream(dev)
    side = _side_streams.get(dev.index)
    if side is None:
        side = _side_streams[dev.index] = torch.cuda.Stream(dev)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        parts = torch.empty((world, B, S, Hl, D), dtype=src.dtype, device=dev)
        dist.all_gather_into_tensor(parts.view(world * B, S, Hl, D), src, group=group)
        full = interleave_heads(parts, out)
        event = torch.cuda.Event()
        event.record(side)
    src.record_stream(side)
    return GatherHandle(full, event, (parts, full))


def gather_heads(out_local: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather head-sharded outputs (B, S, H/n, D) into the full (B, S, H, D) tensor, ordered on the
    caller's current stream."""
    return gather_heads_async(out_local, group, out).wait()


def sharded_attn(local_fn: Callable[..., torch.Tensor], q_local, k_local, v_local, *args,
                 group=None, gather_output: bool = False, async_gather: bool = False, **kwargs):
    """Run `local_fn(q_local, k_local, v_local, *args, **kwargs)` on this rank's heads.

    `local_fn` is `intra_llm_attn` or `intra_image_attn` (tests inject a stand-in). Without
    gather_output the result is this rank's block and nothing but the local launch happens. With
    gather_output=True every rank returns the full-head tensor (a `GatherHandle` if async_gather).
    """
    if not (gather_output and _distributed(group)):
        return local_fn(q_local, k_local, v_local, *args, **kwargs)
    err: Optional[BaseException] = None
    out_local = None
    try:
        out_local = local_fn(q_local, k_local, v_local, *args, **kwargs)
    except Exception as e:  # agreed on below, then re-raised on every rank
        err = e
    if not _agree_ok(err is None, group):
        raise RuntimeError("head-sharded attention failed on at least one rank"
                           + (f" (this rank: {err})" if err is not None else "")) from err
    handle = gather_heads_async(out_local, group)
    return handle if async_gather else handle.wait()


def intra_llm_attn_sharded(q_local, k_local, v_local, pattern="scatter", group_num=8, window=576, softmax_scale=None,
                           group=None, gather_output=False, async_gather=False, out=None):
    """`intra_llm_attn` on this rank's KV-head groups; see `sharded_attn`. `out=` receives the local block."""
    from .interface import intra_llm_attn
    return sharded_attn(intra_llm_attn, q_local, k_local, v_local, pattern, group_num=group_num, window=window,
                        softmax_scale=softmax_scale, out=out, group=group, gather_output=gather_output,
                        async_gather=async_gather)


def intra_image_attn_sharded(q_local, k_local, v_local, pattern="scatter", width=64, softmax_scale=None,
                             group=None, gather_output=False, async_gather=False, out=None):
    """`intra_image_attn` on this rank's heads; see `sharded_attn`. `out=` receives the local block."""
    from .interface import intra_image_attn
    return sharded_attn(intra_image_attn, q_local, k_local, v_local, pattern, width=width,
                        softmax_scale=softmax_scale, out=out, group=group, gather_output=gather_output,
                        async_gather=async_gather)
