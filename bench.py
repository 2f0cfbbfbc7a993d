"""Benchmark of the INTRA forward sparse-attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c5|c1|c2|c3|c3s|c4]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One step = one pass of the hot path over one batch of seeded synthetic q/k/v. The default workload is
the long-context configuration (B=1, S=65536, 32 query / 8 KV heads, head dim 128, bf16 N(0,1)): one
Scatter G=8 call and one window-576 call per step. On N GPUs the KV-head groups of that ONE workload are
split over the ranks through the head-sharded launcher (intra_b200.sharded; no data-path collective),
so the total work is fixed: strong scaling, "one KV-head group per GPU at 8". `--replicas` gives every
rank the whole workload instead (weak scaling). Rank 0 prints ONE JSON line:

  value       effective sparse TFLOP/s = 4*128*H*attended_pairs per step / device time per step over all
              ranks' heads, inputs resident in HBM, CUDA events on the launching stream, max over ranks
  e2e         the same metric through the public Python API with pinned HOST buffers: per step the
              host->device copies of the rank's q/k/v heads, both calls, and the device->host copy of
              both outputs; steps are pipelined over three streams (copy-in, kernels, copy-out)
  roofline    tensor-core roofline of the dominant launch of the step: algorithmic FLOPs per launch /
              its mean CUDA-event duration inside the timed region, against the measured bf16 dense
              peak of MEASURED_PEAKS.json; config.calls carries the same fraction for every call, and,
              on one GPU, for the two calls of the S=16384 configuration (Gather-1 G=8, window 576)
              timed right after the timed region
  cpu_baseline  the CPU oracle (fp32 dense-mask SDPA, the reference's reference.py algorithm) timed on
              this box's host cores on a bounded sample of the same workload (rank 0, N=1 only)

`--impl reference` times that CPU path alone (all host threads, bounded sample per step).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HEAD_DIM = 128
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of each workload's dominant kernel (c1 and
# c5: Scatter G=8, c2: Gather-1, c3: image Scatter, c4: Scatter G=2), from the full-size ncu captures
# summarised under profiles/ (a profiler cannot run inside the timed region).
NCU_TRAFFIC_BYTES = {"c1": 50432768 + 5723136, "c2": 279402240 + 99670016, "c3": 381974272 + 90594048,
                     "c4": 1967612000 + 238374912, "c5": 6485108000 + 507752704}
DEFAULT_WORKLOAD = "c5"

WORKLOADS = {
    # name: (description, B, S, H, Hkv, [(family, pattern, kwargs)])
    "c1": ("LLM Scatter G=8 causal, B=1 S=4096 32q/8kv d=128", 1, 4096, 32, 8,
           [("llm", "scatter", {"group_num": 8})]),
    "c2": ("LLM Gather-1 G=8 + window 576 causal, B=1 S=16384 32q/8kv d=128", 1, 16384, 32, 8,
           [("llm", "gather1", {"group_num": 8}), ("llm", "window", {"window": 576})]),
    "c3": ("FLUX image Scatter + Gather-0, B=1 24 heads d=128, 512 text + 128x128 grid", 1, 512 + 128 * 128, 24, 24,
           [("image", "scatter", {"width": 128}), ("image", "gather0", {"width": 128})]),
    "c3s": ("FLUX image Scatter + Gather-0, B=1 24 heads d=128, 512 text + 64x64 grid", 1, 512 + 64 * 64, 24, 24,
            [("image", "scatter", {"width": 64}), ("image", "gather0", {"width": 64})]),
    "c4": ("g2s4 layer pair: Scatter G=2 + window 576 causal, B=1 S=32768 32q/8kv d=128", 1, 32768, 32, 8,
           [("llm", "scatter", {"group_num": 2}), ("llm", "window", {"window": 576})]),
    "c5": ("LLM Scatter G=8 + window 576 causal, B=1 S=65536 32q/8kv d=128", 1, 65536, 32, 8,
           [("llm", "scatter", {"group_num": 8}), ("llm", "window", {"window": 576})]),
}


def pair_count(family, pattern, S, group_num=8, window=576, width=64):
    """Attended (query, key) pairs of a pattern in closed form (popcount of its mask)."""
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
        total = 0
        for b in range((S + 63) // 64):
            first = max(64 * b - (window - 64), 0)
            n = min(64 * b + 64, S) - 64 * b
            total += n * (64 * b - first) + n * (n + 1) // 2
        return total
    n_img = width * width // 8
    if pattern == "scatter":
        return S * (512 + n_img)
    return 512 * (512 + n_img) + width * width * (512 + 256)


def call_flops(family, pattern, kw, S, H):
    return 4 * HEAD_DIM * H * pair_count(family, pattern, S, **kw)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


CLOCK_TAIL_S = 0.25   # how long the timed launches are kept running past the end event for the clock sampler


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a timed region runs (read-only)."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n = self._nvml
        sm = n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(self._handle, n.NVML_CLOCK_SM)
        r = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle) if hasattr(
            n, "nvmlDeviceGetCurrentClocksEventReasons") else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
        reasons = []
        if r & 0x8:
            reasons.append("hw_slowdown")
        if r & 0x40:
            reasons.append("hw_thermal_slowdown")
        if r & 0x20:
            reasons.append("sw_thermal_slowdown")
        if r & 0x4:
            reasons.append("sw_power_cap")
        return sm, mx, reasons

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                              "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
        f = [x.strip() for x in out.strip().split(",")]
        reasons = [n for n, v in zip(self.NAMES, f[2:]) if v.lower().startswith("active")]
        return float(f[0]), float(f[1]), reasons

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self._sample_nvml() if self._nvml else self._sample_smi())
            except Exception:
                pass
            self._stop.wait(0.005 if self._nvml else 0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=5)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = sorted({r for s in self.samples for r in s[2]})
        return {"sm_mhz": statistics.median(s[0] for s in self.samples),
                "sm_max_mhz": max(s[1] for s in self.samples), "reasons": reasons, "samples": len(self.samples),
                "window": "the timed steps plus %.2f s of the same launches right after them" % CLOCK_TAIL_S}


def mask_rows_strided(oracle, family, pattern, S, stride, kw):
    """Rows 0, stride, 2*stride, ... of a pattern's mask, built from the oracle's predicates for those
    rows only, so that the S x S mask never exists."""
    import numpy as np
    return oracle.build_mask(family, pattern, S, rows=np.arange(0, S, stride), **kw)


class CpuSample:
    """A bounded sample of the workload for the CPU oracle: every `stride`-th query row of the first
    KV-head group (H/Hkv query heads, 1 KV head) of every call of the step, against all keys. The
    attended pairs of exactly those rows are counted from the mask, so the throughput is in the same
    effective-sparse-FLOP unit as the GPU's. It is a SAMPLE of the heads (one KV-head group of Hkv),
    not the per-group results summed."""

    def __init__(self, workload, threads, stride=1):
        import torch

        from oracle import intra_oracle as oracle
        self.oracle = oracle
        desc, B, S, H, Hkv, calls = WORKLOADS[workload]
        self.rep = H // Hkv
        self.calls = calls
        torch.set_num_threads(threads)
        self.q, self.k, self.v = oracle.make_inputs(1, S, self.rep, 1, seed=0)
        self.S, self.Hkv = S, Hkv
        self.set_stride(stride)

    def set_stride(self, stride):
        import torch
        self.stride = stride
        self.qs = self.q[:, ::stride].contiguous()
        self.ms = [torch.from_numpy(mask_rows_strided(self.oracle, f, p, self.S, stride, kw)) for f, p, kw in self.calls]
        self.flops = sum(4 * HEAD_DIM * self.rep * int(m.sum()) for m in self.ms)

    def run(self):
        t0 = time.perf_counter()
        for m in self.ms:
            self.oracle.masked_attention(self.qs, self.k, self.v, m)
        return time.perf_counter() - t0

    def describe(self):
        rows = "all query rows" if self.stride == 1 else f"every {self.stride}th query row"
        return (f"sampled: {rows} of {self.rep} query heads / 1 KV head (one KV-head group of {self.Hkv}) "
                f"of each call, all keys, B=1, S={self.S}")


MAX_SAMPLE_ROWS = 8192    # mask rows of a sample are R x S booleans: 512 MB at S = 65536


def fit_sample(sample, budget_s):
    """Grow the sample (halve the row thinning) while one pass is predicted to stay within budget_s.
    Starts from 512 rows; a pass costs a little more than twice the pass at half the rows."""
    stride = max(sample.S // 512, 1)
    sample.set_stride(stride)
    sample.run()                                           # warm-up (thread pool, allocator)
    dt = sample.run()
    while stride > 1 and sample.S // (stride // 2) <= MAX_SAMPLE_ROWS and 2.3 * dt <= budget_s:
        stride //= 2
        sample.set_stride(stride)
        dt = sample.run()
    return dt


def run_reference(args):
    """The reference's CPU implementation of the path (its fp32 dense-mask SDPA oracle, restated in
    oracle/) on the host cores; each step is a bounded sample of the workload, thinned so that the
    whole run stays within a couple of minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    desc = WORKLOADS[args.workload][0]
    sample = CpuSample(args.workload, threads, stride=max(WORKLOADS[args.workload][2] // 512, 1))
    fit_sample(sample, 60.0 / max(args.steps + args.warmup, 1))       # the whole run within about two minutes
    for _ in range(args.warmup):
        sample.run()
    total = sum(sample.run() for _ in range(args.steps))
    value = sample.flops * args.steps / total / 1e12
    line = {
        "impl": "reference", "metric": "effective sparse attention throughput (4*d*H*attended pairs / time)",
        "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "inputs": "seeded bf16 N(0,1), computed in fp32 on the CPU"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": sample.describe()},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def run_ours(args):
    import torch
    import torch.distributed as dist

    from intra_b200.interface import device_status
    from intra_b200.sharded import intra_image_attn_sharded, intra_llm_attn_sharded

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the attention path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    desc, B, S, H_total, Hkv_total, calls = WORKLOADS[args.workload]
    shard = world > 1 and not args.replicas
    if shard and Hkv_total % world:
        raise SystemExit(f"{Hkv_total} KV heads cannot be split over {world} ranks")
    # this rank's block of KV-head groups (the whole workload on one GPU or with --replicas)
    H, Hkv = (H_total // world, Hkv_total // world) if shard else (H_total, Hkv_total)
    g = torch.Generator(device="cpu").manual_seed(1000 + rank)
    hq = torch.randn(B, S, H, HEAD_DIM, generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    hk = torch.randn(B, S, Hkv, HEAD_DIM, generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    hv = torch.randn(B, S, Hkv, HEAD_DIM, generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    q, k, v = hq.to(dev), hk.to(dev), hv.to(dev)
    houts = [torch.empty_like(hq).pin_memory() for _ in calls]

    def run_call(c, q_, k_, v_, out=None, **extra):
        """One attention call through the head-sharded launcher, the API a multi-GPU caller uses (on one
        GPU, and without gather_output, it is the plain local call)."""
        family, pattern, kw = c
        fn = intra_llm_attn_sharded if family == "llm" else intra_image_attn_sharded
        return fn(q_, k_, v_, pattern, out=out, **kw, **extra)

    flops_calls = [call_flops(f, p, kw, S, H) for f, p, kw in calls]        # this rank's heads
    flops_step = sum(flops_calls)
    dom = max(range(len(calls)), key=lambda i: flops_calls[i])              # dominant launch

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    res = [torch.empty_like(q) for _ in calls]              # device-resident legs write here (out=)
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            for i, c in enumerate(calls):
                run_call(c, q, k, v, out=res[i])
        torch.cuda.synchronize()

        # ---- device-resident timed region: K steps, events around the region and around each launch
        evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in calls]
               for _ in range(args.steps)]
        t_beg, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with ClockSampler(local_rank) as clocks:
            t_beg.record(stream)
            for s in range(args.steps):
                for i, c in enumerate(calls):
                    evs[s][i][0].record(stream)
                    run_call(c, q, k, v, out=res[i])
                    evs[s][i][1].record(stream)
            t_end.record(stream)
            t_end.synchronize()
            # A short timed region sees few clock samples (an NVML query under load takes milliseconds),
            # so the same launches keep running (after the end event: untimed, uncounted) until the
            # sampler has watched this load for a quarter of a second in all.
            t_tail = time.perf_counter()
            while (t_beg.elapsed_time(t_end) < 1e3 * CLOCK_TAIL_S and time.perf_counter() - t_tail < CLOCK_TAIL_S):
                for i, c in enumerate(calls):
                    run_call(c, q, k, v, out=res[i])
                torch.cuda.synchronize()
            barrier()
        total_ms = t_beg.elapsed_time(t_end)
        launch_ms = [statistics.mean(evs[s][i][0].elapsed_time(evs[s][i][1]) for s in range(args.steps))
                     for i in range(len(calls))]

        # ---- optional: the same steps with every call's head-sharded output all-gathered over NCCL into
        # the full (B, S, H, 128) tensor on every rank, for callers that need it (reported beside the
        # headline, never part of it). The gather of call i runs on a side stream under call i+1.
        gather_ms = 0.0
        if args.gather_outputs and shard:
            def gathered_steps(n):
                pending = None
                for _ in range(n):
                    for i, c in enumerate(calls):
                        handle = run_call(c, q, k, v, out=res[i], gather_output=True, async_gather=True)
                        if pending is not None:
                            pending.wait()
                        pending = handle
                pending.wait()
            gathered_steps(3)
            g_beg, g_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            g_beg.record(stream)
            gathered_steps(args.steps)
            g_end.record(stream)
            barrier()
            gather_ms = g_beg.elapsed_time(g_end)

        # ---- on one GPU: the two calls of the S=16384 configuration (Gather-1 G=8, window 576), each
        # timed alone with CUDA events, for config.calls (not part of `value`)
        extra_calls = []
        if world == 1 and args.workload != "c2" and not args.no_extra:
            _, B2, S2, H2, Hkv2, calls2 = WORKLOADS["c2"]
            g2 = torch.Generator(device="cpu").manual_seed(2000)
            q2 = torch.randn(B2, S2, H2, HEAD_DIM, generator=g2, dtype=torch.float32).to(torch.bfloat16).to(dev)
            k2 = torch.randn(B2, S2, Hkv2, HEAD_DIM, generator=g2, dtype=torch.float32).to(torch.bfloat16).to(dev)
            v2 = torch.randn(B2, S2, Hkv2, HEAD_DIM, generator=g2, dtype=torch.float32).to(torch.bfloat16).to(dev)
            o2 = torch.empty_like(q2)
            n2 = 20
            for c in calls2:
                for _ in range(5):
                    run_call(c, q2, k2, v2, out=o2)
                # each call is timed as a short burst of its own after a pause, like the burst figure of the
                # measured peak it is compared with, not at the power cap the long timed region left behind
                torch.cuda.synchronize()
                time.sleep(0.5)
                pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n2)]
                for a_, b_ in pairs:
                    a_.record(stream)
                    run_call(c, q2, k2, v2, out=o2)
                    b_.record(stream)
                torch.cuda.synchronize()
                extra_calls.append((c, S2, call_flops(c[0], c[1], c[2], S2, H2),
                                    statistics.mean(a_.elapsed_time(b_) for a_, b_ in pairs), "intra_llm_attn"))
            # the Gather-1 call once more through the allocation-free C entry point (same kernel, scratch in
            # the library image), so that this entry point has a measured line of its own
            import ctypes

            from intra_b200._loader import lib as _lib, strides3 as _st
            c = calls2[0]
            args2 = (q2.data_ptr(), k2.data_ptr(), v2.data_ptr(), o2.data_ptr(), B2, S2, H2, Hkv2, _st(q2), _st(k2), _st(v2),
                     _st(o2), 1, c[2]["group_num"], 576, HEAD_DIM ** -0.5, local_rank, stream.cuda_stream, None)
            for _ in range(5):
                assert _lib.intra_b200_fwd_llm_noalloc(*args2) == 0
            torch.cuda.synchronize()
            time.sleep(0.5)
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n2)]
            for a_, b_ in pairs:
                a_.record(stream)
                _lib.intra_b200_fwd_llm_noalloc(*args2)
                b_.record(stream)
            torch.cuda.synchronize()
            prev = ctypes.c_int(-1)
            assert _lib.intra_b200_fwd_llm_noalloc(*args2[:-1], ctypes.byref(prev)) == 0 and prev.value == 0
            extra_calls.append((c, S2, call_flops(c[0], c[1], c[2], S2, H2),
                                statistics.mean(a_.elapsed_time(b_) for a_, b_ in pairs), "intra_b200_fwd_llm_noalloc (C ABI)"))
            del q2, k2, v2, o2

        # ---- end-to-end: pinned host buffers in, host buffers out, every step. Three streams pipeline
        # the steps: the copy-in of step i+1 and the copy-out of step i-1 run beside step i's kernels
        # (PCIe is full duplex), with device buffers double-buffered. Every step still copies its own
        # inputs in and its own outputs out.
        e_steps = 0 if args.no_e2e else max(3, min(args.steps, 20))
        s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        dbuf = [(torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)) for _ in range(2)]
        # outputs are double-buffered device tensors of the caller's too (out=): an allocation per call
        # on a side stream makes the caching allocator go back to cudaMalloc while copies are in flight
        obuf = [[torch.empty_like(q) for _ in calls] for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]      # inputs of the slot have landed
        ev_cmp = [torch.cuda.Event() for _ in range(2)]     # kernels of the slot are done (inputs reusable)
        ev_out = [torch.cuda.Event() for _ in range(2)]     # outputs of the slot are on the host

        def e2e_steps(n_steps):
            for st in range(n_steps):
                slot = st & 1
                with torch.cuda.stream(s_in):
                    if st >= 2:
                        s_in.wait_event(ev_cmp[slot])
                    dbuf[slot][0].copy_(hq, non_blocking=True)
                    dbuf[slot][1].copy_(hk, non_blocking=True)
                    dbuf[slot][2].copy_(hv, non_blocking=True)
                    ev_in[slot].record(s_in)
                with torch.cuda.stream(s_cmp):
                    s_cmp.wait_event(ev_in[slot])
                    if st >= 2:
                        s_cmp.wait_event(ev_out[slot])           # the slot's previous outputs are on the host
                    outs = [run_call(c, *dbuf[slot], out=obuf[slot][i]) for i, c in enumerate(calls)]
                    ev_cmp[slot].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[slot])
                    for i, o in enumerate(outs):
                        houts[i].copy_(o, non_blocking=True)
                    ev_out[slot].record(s_out)

        for st_ in (s_in, s_cmp, s_out):
            st_.wait_stream(stream)
        e2e_steps(min(2, e_steps))
        for st_ in (s_in, s_cmp, s_out):
            stream.wait_stream(st_)
        e_beg, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e_beg.record(stream)
        for st_ in (s_in, s_cmp, s_out):
            st_.wait_stream(stream)
        e2e_steps(e_steps)
        for st_ in (s_in, s_cmp, s_out):
            stream.wait_stream(st_)
        e_end.record(stream)
        barrier()
        e2e_ms = e_beg.elapsed_time(e_end)

    status = device_status(local_rank, reset=True)
    if status != 0:
        raise SystemExit(f"kernel status word {status}: a bounded wait gave up; numbers invalid")

    times = torch.tensor([total_ms, e2e_ms, gather_ms] + launch_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, gather_ms, *launch_ms = times.tolist()
    if rank == 0:
        peaks, peaks_kind = load_peaks()
        ms_per_step = total_ms / args.steps
        # flops_step is per rank; all ranks together did world * flops_step in the slowest rank's time
        value = world * flops_step / (ms_per_step * 1e-3) / 1e12
        e2e_value = world * flops_step / (e2e_ms / e_steps * 1e-3) / 1e12 if e_steps else None
        achieved = flops_calls[dom] / (launch_ms[dom] * 1e-3) / 1e12       # per GPU: one rank's launch
        peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        sustained = float(peaks.get("bf16_tflops_sustained", peak))

        def call_entry(c, S_, flops, ms, per, entry="intra_b200.sharded"):
            tf = flops / ms / 1e9
            return {"pattern": f"{c[0]}/{c[1]}", **c[2], "S": S_, "heads": per, "entry": entry, "ms": ms, "tflops": tf,
                    "frac_of_burst_peak": tf / peak, "frac_of_sustained_peak": tf / sustained}

        per_heads = f"{H}q/{Hkv}kv per GPU"
        call_list = [call_entry(c, S, flops_calls[i], launch_ms[i], per_heads) for i, c in enumerate(calls)]
        call_list += [call_entry(c, S2, fl, ms, "32q/8kv, 20 launches back to back after a 0.5 s pause, outside the timed region", ent)
                      for c, S2, fl, ms, ent in extra_calls]
        line = {
            "metric": "effective sparse attention throughput (4*d*H*attended pairs / time)",
            "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if shard or world == 1 else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": desc,
                       "per_rank": (f"KV-head groups sharded through intra_b200.sharded: {H} query / {Hkv} KV heads of "
                                    f"{H_total} / {Hkv_total} per rank, no data-path collective" if shard else
                                    ("the whole workload on one GPU" if world == 1 else
                                     "each rank runs the whole workload on its own seeded batch (--replicas)")),
                       "l2": "inputs+outputs per step and rank (%d MB) %s the 126 MB L2; no explicit flush" % (
                           (2 * q.numel() + k.numel() + v.numel()) * 2 // 2**20,
                           "exceed" if (2 * q.numel() + k.numel() + v.numel()) * 2 > 126 * 2**20 else "DO NOT exceed"),
                       "calls": call_list},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": world * (hq.numel() + hk.numel() + hv.numel()) * 2,
                    "d2h_bytes_per_step": world * sum(h.numel() for h in houts) * 2, "steps": e_steps,
                    "ms_per_step": e2e_ms / e_steps if e_steps else None},
            "gpu_launches": args.steps * len(calls),
            "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "kernel": "intra_fwd_dual_kernel (%s/%s launch)" % (calls[dom][0], calls[dom][1]),
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": peaks_kind + " bf16_tflops (burst)",
                         "frac_of_sustained": achieved / sustained,
                         "flops_per_launch": flops_calls[dom], "ms_per_launch": launch_ms[dom],
                         "traffic": NCU_TRAFFIC_BYTES.get(args.workload) if world == 1 else None},
        }
        if gather_ms > 0.0:
            line["gather"] = {"ms_per_step": gather_ms / args.steps,
                              "extra_ms_per_step": gather_ms / args.steps - ms_per_step,
                              "bytes_received_per_rank_per_step": len(calls) * (world - 1) * q.numel() * 2,
                              "what": "every call followed by an NCCL all-gather of its head-sharded output and the "
                                      "library's head-interleave kernel into the full (B, S, H, 128) tensor on every "
                                      "rank, on a side stream under the next call"}
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            sample = CpuSample(args.workload, threads, stride=max(S // 512, 1))
            fit_sample(sample, 5.0)                                     # about 5 s per pass of the sample
            dts = [sample.run() for _ in range(3)]
            line["cpu_baseline"] = {"value": sample.flops / statistics.median(dts) / 1e12, "unit": "TFLOP/s",
                                    "cores": threads, "kind": "port",
                                    "sample": sample.describe() + "; median of 3 passes"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the S=16384 calls timed for config.calls")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--gather-outputs", action="store_true",
                    help="on several GPUs: also time the steps with every output all-gathered")
    ap.add_argument("--replicas", action="store_true",
                    help="weak scaling: every rank runs the whole workload instead of its share of the KV-head groups")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "ours" and args.gpus != world:
        if args.gpus > 1 and world == 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
