"""Head-sharded launch on 2+ real GPUs: each rank's output equals the same heads of a one-GPU run,
and the all-gathered tensor equals the full one. Skipped on boxes with a single GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, result_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from intra_b200 import intra_llm_attn, sharded
        from oracle import intra_oracle as oracle
        q, k, v = oracle.make_inputs(1, 4096, 32, 8, seed=2, device=f"cuda:{rank}")
        with torch.no_grad():
            full = intra_llm_attn(q, k, v, "gather1", group_num=8)
            ql, kl, vl = (x.contiguous() for x in sharded.shard_heads(q, k, v, rank, world))
            local = sharded.intra_llm_attn_sharded(ql, kl, vl, "gather1", group_num=8)
            gathered = sharded.intra_llm_attn_sharded(ql, kl, vl, "gather1", group_num=8, gather_output=True)
            # the all-gather of one call running on its side stream under the next call
            handle = sharded.intra_llm_attn_sharded(ql, kl, vl, "window", window=576, gather_output=True, async_gather=True)
            again = sharded.intra_llm_attn_sharded(ql, kl, vl, "gather1", group_num=8)
            full_w = intra_llm_attn(q, k, v, "window", window=576)
            gathered_w = handle.wait()
        qs, _ = sharded.head_slices(32, 8, rank, world)
        torch.cuda.synchronize()
        result_q.put((rank, bool(torch.equal(local, full[:, :, qs])) and bool(torch.equal(again, local)),
                      bool(torch.equal(gathered, full)) and bool(torch.equal(gathered_w, full_w))))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_head_sharded_matches_single_gpu():
    world = min(torch.cuda.device_count(), 8)
    while 8 % world:
        world -= 1
    ctx = mp.get_context("spawn")
    result_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, result_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [result_q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(a and b for _, a, b in results), results
