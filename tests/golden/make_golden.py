"""Regenerate the golden fixtures from the reference's own Python code.

    python tests/golden/make_golden.py /path/to/reference/checkout

Imports the reference's `intra_attn/reference.py` (pure PyTorch, runs on the CPU) and writes, next
to this script,

  masks.json      digests (sha256 of packed bits, pair count, row checksum) of the reference's
                  masks over the shape matrix of the reference's kernel test
                  (tests/test_kernel.py:33-51) plus small and ragged shapes;
  attention.npz   outputs of the reference's `masked_attention` on small seeded inputs, as bf16
                  bit patterns, with a digest of the inputs they were computed from.

The fixtures are what pins `oracle/intra_oracle.py` to the reference on machines where the
reference checkout is absent.
"""
import hashlib
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import intra_oracle as oracle  # noqa: E402  (input generator + digest helper only)

MASK_CASES = (
    [("llm", "scatter", S, dict(group_num=G)) for S in (32, 1000, 2048, 3000, 4096, 8192) for G in (2, 3, 8)]
    + [("llm", "scatter", 16384, dict(group_num=8))]
    + [("llm", "gather1", S, dict(group_num=8)) for S in (64, 2048, 4096, 8192, 16384)]
    + [("llm", "gather1", S, dict(group_num=G)) for S, G in ((32, 4), (1000, 8), (300, 3))]
    + [("llm", "window", S, dict(window=W)) for S in (200, 1000, 2048, 3000, 4096, 8192) for W in (576, 1000)]
    + [("llm", "window", 200, dict(window=96)), ("llm", "window", 16384, dict(window=576))]
    + [("image", p, 512 + w * w, dict(width=w)) for p in ("scatter", "gather0") for w in (16, 24, 32, 64, 128)]
)

ATTN_CASES = [
    # name, family, pattern, B, S, H, Hkv, kwargs, seed
    ("llm_scatter_g3", "llm", "scatter", 2, 333, 2, 1, dict(group_num=3), 11),
    ("llm_scatter_g8", "llm", "scatter", 1, 1000, 2, 1, dict(group_num=8), 12),
    ("llm_gather1_g8", "llm", "gather1", 1, 576, 2, 2, dict(group_num=8), 13),
    ("llm_window_160", "llm", "window", 2, 300, 2, 1, dict(window=160), 14),
    ("llm_window_576", "llm", "window", 1, 1000, 2, 1, dict(window=576), 15),
    ("img_scatter_w16", "image", "scatter", 2, 512 + 256, 1, 1, dict(width=16), 16),
    ("img_gather0_w16", "image", "gather0", 1, 512 + 256, 1, 1, dict(width=16), 17),
    ("img_scatter_w32", "image", "scatter", 1, 512 + 1024, 1, 1, dict(width=32), 18),
    ("img_gather0_w32", "image", "gather0", 1, 512 + 1024, 1, 1, dict(width=32), 19),
]


def load_reference(root):
    path = os.path.join(root, "intra_attn", "reference.py")
    spec = importlib.util.spec_from_file_location("intra_reference_spec", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def reference_mask(ref, family, pattern, S, kw):
    if family == "llm":
        if pattern == "scatter":
            return ref.llm_scatter_mask(S, kw["group_num"])
        if pattern == "gather1":
            return ref.llm_gather1_mask(S, kw["group_num"])
        return ref.llm_window_mask(S, kw["window"])
    if pattern == "scatter":
        return ref.image_scatter_mask(kw["width"])
    return ref.image_gather0_mask(kw["width"])


def bits(x):
    return x.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of the reference repository>")
    ref = load_reference(sys.argv[1])
    torch.set_num_threads(os.cpu_count())

    masks = []
    for family, pattern, S, kw in MASK_CASES:
        m = reference_mask(ref, family, pattern, S, kw).numpy()
        d = oracle.mask_digest(m)
        d.update(family=family, pattern=pattern, S=S, **kw)
        masks.append(d)
        print("mask", family, pattern, S, kw, d["pairs"], flush=True)
    with open(os.path.join(HERE, "masks.json"), "w") as f:
        json.dump(masks, f, indent=1)

    arrays, meta = {}, []
    for name, family, pattern, B, S, H, Hkv, kw, seed in ATTN_CASES:
        q, k, v = oracle.make_inputs(B, S, H, Hkv, seed=seed)
        mask = reference_mask(ref, family, pattern, S, kw)
        out = ref.masked_attention(q, k, v, mask)
        arrays[name] = bits(out)
        h = hashlib.sha256()
        for x in (q, k, v):
            h.update(bits(x).tobytes())
        meta.append(dict(name=name, family=family, pattern=pattern, B=B, S=S, H=H, Hkv=Hkv, seed=seed,
                         inputs_sha256=h.hexdigest(), **kw))
        print("attn", name, tuple(out.shape), flush=True)
    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **arrays)


if __name__ == "__main__":
    main()
