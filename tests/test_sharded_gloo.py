"""Head-sharded launcher on CPU ranks (gloo, world size 2): head partition, output all-gather and
host-side failure agreement. The local attention is a stand-in (the CPU oracle), since the host logic
under test is independent of the kernel."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from intra_b200 import sharded
from oracle import intra_oracle as oracle


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_local(mask):
    def fn(q, k, v, *a, **kw):
        return oracle.masked_attention(q, k, v, mask)
    return fn


def _worker(rank, world, port, mode, result_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        B, S, H, Hkv = 1, 256, 8, 4
        q, k, v = oracle.make_inputs(B, S, H, Hkv, seed=5)
        mask = oracle.llm_scatter_mask(S, 4)
        ql, kl, vl = sharded.shard_heads(q, k, v, rank, world)
        assert ql.shape[2] == H // world and kl.shape[2] == Hkv // world
        if mode == "gather":
            full = sharded.sharded_attn(_oracle_local(mask), ql, kl, vl, gather_output=True)
            ref = oracle.masked_attention(q, k, v, mask)
            result_q.put((rank, bool(torch.equal(full, ref))))
        elif mode == "local":
            out = sharded.sharded_attn(_oracle_local(mask), ql, kl, vl, gather_output=False)
            ref = oracle.masked_attention(q, k, v, mask)
            qs, _ = sharded.head_slices(H, Hkv, rank, world)
            result_q.put((rank, bool(torch.equal(out, ref[:, :, qs]))))
        elif mode == "async":
            handle = sharded.sharded_attn(_oracle_local(mask), ql, kl, vl, gather_output=True, async_gather=True)
            ref = oracle.masked_attention(q, k, v, mask)
            result_q.put((rank, bool(torch.equal(handle.wait(), ref))))
        elif mode == "fail-local":
            # without a collective to protect there is no agreement: the failing rank raises its own
            # error, the healthy one returns its block, nobody waits for anybody
            def bad_local(qq, kk, vv, *a, **kw):
                if rank == 1:
                    raise RuntimeError("injected launch failure")
                return oracle.masked_attention(qq, kk, vv, mask)
            try:
                out = sharded.sharded_attn(bad_local, ql, kl, vl, gather_output=False)
                result_q.put((rank, rank == 0 and out.shape[2] == H // world))
            except RuntimeError as e:
                result_q.put((rank, rank == 1 and "injected" in str(e)))
        elif mode == "fail":
            def bad(qq, kk, vv, *a, **kw):
                if rank == 1:
                    raise RuntimeError("injected launch failure")
                return oracle.masked_attention(qq, kk, vv, mask)
            try:
                sharded.sharded_attn(bad, ql, kl, vl, gather_output=True)
                result_q.put((rank, False))
            except RuntimeError as e:
                result_q.put((rank, "failed on at least one rank" in str(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["gather", "local", "async", "fail", "fail-local"])
def test_sharded_world2(mode):
    world = 2
    ctx = mp.get_context("spawn")
    result_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, result_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [result_q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in results) == [0, 1]
    assert all(ok for _, ok in results), results


def test_head_slices():
    assert sharded.head_slices(32, 8, 0, 8) == (slice(0, 4), slice(0, 1))
    assert sharded.head_slices(32, 8, 7, 8) == (slice(28, 32), slice(7, 8))
    assert sharded.head_slices(32, 8, 1, 2) == (slice(16, 32), slice(4, 8))
    assert sharded.head_slices(24, 24, 3, 8) == (slice(9, 12), slice(9, 12))
    with pytest.raises(ValueError):
        sharded.head_slices(32, 8, 0, 3)
