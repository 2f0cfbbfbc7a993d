"""Latency table in the format of the reference's kernel benchmark (benchmarks/bench_kernel.py).

    python -m intra_b200.bench_kernel llm   [--seqlens 4096,...] [--groups 2,8] [--out file.json]
    python -m intra_b200.bench_kernel image [--out file.json]
    python -m intra_b200.bench_kernel stack [--seqlens 32768] [--layers 32] [--out file.json]

Same flags, same protocol (CUDA events around each call, 10 warm-ups, median of 50) and the same row
keys as the reference's benchmarks/results/*.json, so B200 rows can sit next to its A100 ones; each
sparse entry additionally gets `<key>_tflops`, the effective sparse TFLOP/s (4*128*H*attended pairs).
The dense baseline is torch SDPA with K/V expanded to the query heads, as in the reference; the
reference pins SDPA to its FlashAttention-2 backend (benchmarks/bench_kernel.py:37-42), here the backend
is pinned to the first of FLASH_ATTENTION, CUDNN_ATTENTION, EFFICIENT_ATTENTION that runs on the device,
and the file records which (`dense_backend`).

`--ref-ext PATH` loads the reference's own compiled extension (`intra_attn_cuda*.so`, the sm_100 build of
its mma.sync kernels) and times it with the same protocol on the same tensors in the same process: each
sparse entry then also gets `ref_<key>` (ms) and `ref_<key>_maxdiff` (max |ours - reference kernel| on
that call's output). Only run it at lengths that are multiples of 512: the reference's Gather-1 loader
reads past the sequence when S % 512 == 64.

`stack` runs the g2s4 layer schedule for real instead of extrapolating it from two timings as the
reference's table does (benchmarks/bench_kernel.py:67): `--layers` attention calls back to back, layer l
on its own seeded q/k/v (seed 1000 + l), Scatter G=2 on every eighth layer and window 576 on the others,
timed as one region with CUDA events, against the same number of dense causal SDPA calls on the same
tensors.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch
import torch.nn.functional as F

from . import intra_image_attn, intra_llm_attn

TEXT_LEN = 512


def median_ms(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


_dense_backend = None


def dense_backend():
    """The SDPA backend the dense baseline is pinned to: the first that runs a small causal bf16 call."""
    global _dense_backend
    if _dense_backend is None:
        from torch.nn.attention import SDPBackend, sdpa_kernel
        x = torch.zeros(1, 2, 128, 128, device="cuda", dtype=torch.bfloat16)
        for cand in (SDPBackend.FLASH_ATTENTION, SDPBackend.CUDNN_ATTENTION, SDPBackend.EFFICIENT_ATTENTION):
            try:
                with sdpa_kernel(cand):
                    F.scaled_dot_product_attention(x, x, x, is_causal=True)
                torch.cuda.synchronize()
                _dense_backend = cand
                break
            except RuntimeError:
                continue
        else:
            raise RuntimeError("no fused SDPA backend runs on this device")
    return _dense_backend


def dense_sdpa(q, k, v, causal):
    from torch.nn.attention import sdpa_kernel
    rep = q.shape[2] // k.shape[2]
    qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))
    if rep > 1:
        kt, vt = kt.repeat_interleave(rep, 1), vt.repeat_interleave(rep, 1)
    with sdpa_kernel(dense_backend()):
        return F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal)


class RefExt:
    """The reference's compiled extension, called the way its Python wrapper calls it
    (intra_attn/interface.py:43-45 and :64-66): contiguous (B, S, H, 128) tensors, pattern ids 0 / 1 / 4."""

    def __init__(self, path):
        import importlib.util
        spec = importlib.util.spec_from_file_location("intra_attn_cuda", path)
        self.mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(self.mod)

    def llm(self, q, k, v, pattern, group_num=8, window=576):
        if q.shape[1] % 512:
            raise ValueError("the reference extension is only run at lengths that are multiples of 512")
        pid = {"scatter": 0, "gather1": 1, "window": 4}[pattern]
        return self.mod.fwd_llm(q, k, v, None, None, 0.0, q.shape[-1] ** -0.5, True, -1, -1, 0.0, False, None,
                                pid, group_num, window)[0]

    def image(self, q, k, v, pattern, width):
        pid = {"scatter": 0, "gather0": 4}[pattern]
        return self.mod.fwd(q, k, v, None, None, 0.0, q.shape[-1] ** -0.5, False, -1, -1, 0.0, False, None,
                            pid, width, width)[0]


def time_ref(r, key, ref_fn, ours_fn, args):
    """Adds the reference extension's time for entry `key` and its largest difference from our output."""
    ours = ours_fn()
    theirs = ref_fn()
    torch.cuda.synchronize()
    r[f"ref_{key}_maxdiff"] = float((ours.float() - theirs.float()).abs().max())
    r[f"ref_{key}"] = median_ms(ref_fn, args.warmup, args.iters)


def llm_pairs(pattern, S, G=8, W=576):
    if pattern == "window":
        return sum((min(64 * b + 64, S) - 64 * b) * (64 * b - max(64 * b - (W - 64), 0))
                   + (min(64 * b + 64, S) - 64 * b) * (min(64 * b + 64, S) - 64 * b + 1) // 2
                   for b in range((S + 63) // 64))
    total = 0
    for g in range(G):
        if pattern == "scatter":
            n = S // G + (1 if g < S % G else 0)
        else:
            n = (S // (G * G)) * G + min(max(S % (G * G) - g * G, 0), G)
        total += n * (n + 1) // 2
    return total


def randn(*shape):
    return torch.randn(*shape, device="cuda", dtype=torch.bfloat16)


@torch.no_grad()
def bench_llm(args):
    rows = []
    for S in args.seqlens:
        q, k, v = randn(args.batch, S, args.heads, 128), randn(args.batch, S, args.kv_heads, 128), randn(args.batch, S, args.kv_heads, 128)
        flop = lambda pairs: 4 * 128 * args.heads * args.batch * pairs
        r = {"seqlen": S}
        try:
            r["dense"] = median_ms(lambda: dense_sdpa(q, k, v, True), args.warmup, args.iters)
        except RuntimeError:
            r["dense"] = None
        ref = args.ref
        for G in args.groups:
            ms = median_ms(lambda: intra_llm_attn(q, k, v, "scatter", group_num=G), args.warmup, args.iters)
            r[f"scatter_g{G}"] = ms
            r[f"scatter_g{G}_tflops"] = flop(llm_pairs("scatter", S, G)) / ms / 1e9
            if ref:
                time_ref(r, f"scatter_g{G}", lambda: ref.llm(q, k, v, "scatter", group_num=G),
                         lambda: intra_llm_attn(q, k, v, "scatter", group_num=G), args)
        if S % 64 == 0:
            ms = median_ms(lambda: intra_llm_attn(q, k, v, "gather1", group_num=8), args.warmup, args.iters)
            r["gather1_g8"] = ms
            r["gather1_g8_tflops"] = flop(llm_pairs("gather1", S, 8)) / ms / 1e9
            if ref:
                time_ref(r, "gather1_g8", lambda: ref.llm(q, k, v, "gather1", group_num=8),
                         lambda: intra_llm_attn(q, k, v, "gather1", group_num=8), args)
        ms = median_ms(lambda: intra_llm_attn(q, k, v, "window", window=576), args.warmup, args.iters)
        r["window576"] = ms
        r["window576_tflops"] = flop(llm_pairs("window", S, W=576)) / ms / 1e9
        if ref:
            time_ref(r, "window576", lambda: ref.llm(q, k, v, "window", window=576),
                     lambda: intra_llm_attn(q, k, v, "window", window=576), args)
        if "scatter_g2" in r:
            r["g2s4_32layer"] = 4 * r["scatter_g2"] + 28 * r["window576"]
            if r["dense"] is not None:
                r["dense_32layer"] = 32 * r["dense"]
        rows.append(r)
        print("  ".join(f"{a}={b:.3f}" if isinstance(b, float) else f"{a}={b}" for a, b in r.items()), flush=True)
    return rows


@torch.no_grad()
def bench_image(args):
    rows = []
    for width in (64, 128):
        S = TEXT_LEN + width * width
        q, k, v = (randn(args.batch, S, args.image_heads, 128) for _ in range(3))
        n_img = width * width // 8
        pairs = {"scatter": S * (TEXT_LEN + n_img), "gather0": TEXT_LEN * (TEXT_LEN + n_img) + width * width * 768}
        r = {"width": width, "seqlen": S}
        try:
            r["dense"] = median_ms(lambda: dense_sdpa(q, k, v, False), args.warmup, args.iters)
        except RuntimeError:
            r["dense"] = None
        for pattern in ("scatter", "gather0"):
            ms = median_ms(lambda: intra_image_attn(q, k, v, pattern, width), args.warmup, args.iters)
            r[pattern] = ms
            r[pattern + "_tflops"] = 4 * 128 * args.image_heads * args.batch * pairs[pattern] / ms / 1e9
            if args.ref:
                time_ref(r, pattern, lambda: args.ref.image(q, k, v, pattern, width),
                         lambda: intra_image_attn(q, k, v, pattern, width), args)
        r["interleaved_mean"] = (r["scatter"] + r["gather0"]) / 2
        rows.append(r)
        print("  ".join(f"{a}={b:.3f}" if isinstance(b, float) else f"{a}={b}" for a, b in r.items()), flush=True)
    return rows


def stack_pattern(layer):
    """g2s4: Scatter G=2 on layers 0, 8, 16, 24, window 576 on the other 28."""
    return ("scatter", {"group_num": 2}) if layer % 8 == 0 else ("window", {"window": 576})


@torch.no_grad()
def bench_stack(args):
    rows = []
    for S in args.seqlens:
        layers = []
        for layer in range(args.layers):
            g = torch.Generator(device="cuda").manual_seed(1000 + layer)
            mk = lambda h: torch.randn(args.batch, S, h, 128, device="cuda", dtype=torch.float32, generator=g).to(torch.bfloat16)
            layers.append((mk(args.heads), mk(args.kv_heads), mk(args.kv_heads)))
        out = torch.empty_like(layers[0][0])

        def sparse_pass():
            for layer, (q, k, v) in enumerate(layers):
                pattern, kw = stack_pattern(layer)
                intra_llm_attn(q, k, v, pattern, out=out, **kw)

        def dense_pass():
            for q, k, v in layers:
                dense_sdpa(q, k, v, True)

        r = {"seqlen": S, "layers": args.layers, "schedule": "g2s4",
             "intra_ms": median_ms(sparse_pass, 2, args.stack_iters)}
        flops = sum(4 * 128 * args.heads * args.batch *
                    (llm_pairs("scatter", S, 2) if layer % 8 == 0 else llm_pairs("window", S, W=576))
                    for layer in range(args.layers))
        r["intra_tflops"] = flops / r["intra_ms"] / 1e9
        try:
            r["dense_ms"] = median_ms(dense_pass, 1, args.stack_iters)
            r["speedup_vs_dense"] = r["dense_ms"] / r["intra_ms"]
        except RuntimeError:
            r["dense_ms"] = None
        rows.append(r)
        print("  ".join(f"{a}={b:.3f}" if isinstance(b, float) else f"{a}={b}" for a, b in r.items()), flush=True)
    return rows


def main():
    p = argparse.ArgumentParser()
    p.add_argument("mode", choices=["llm", "image", "stack"])
    p.add_argument("--layers", type=int, default=32)
    p.add_argument("--stack-iters", type=int, default=5)
    p.add_argument("--seqlens", default="4096,8192,16384,32768,65536")
    p.add_argument("--groups", default="2,8")
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--image-heads", type=int, default=24)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--iters", type=int, default=50)
    p.add_argument("--out", help="optional JSON output path")
    p.add_argument("--ref-ext", help="path of the reference's compiled extension to time beside this library")
    args = p.parse_args()
    args.ref = RefExt(args.ref_ext) if args.ref_ext else None
    args.seqlens = [int(x) for x in args.seqlens.split(",")]
    args.groups = [int(x) for x in args.groups.split(",")]
    print(f"device: {torch.cuda.get_device_name()}  torch {torch.__version__}")
    if args.mode == "stack" and args.seqlens == [4096, 8192, 16384, 32768, 65536]:
        args.seqlens = [32768]
    rows = {"llm": bench_llm, "image": bench_image, "stack": bench_stack}[args.mode](args)
    if args.out:
        with open(args.out, "w") as f:
            json.dump({"device": torch.cuda.get_device_name(), "torch": torch.__version__,
                       "dense_backend": str(_dense_backend) if _dense_backend is not None else None,
                       "args": {a: b for a, b in vars(args).items() if a not in ("out", "ref")}, "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()
