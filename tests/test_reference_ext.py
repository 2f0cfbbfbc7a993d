"""This library against the reference's own CUDA kernels on the same inputs, on the same GPU.

oracle/build_ref_ext.sh compiles the reference's extension for sm_100 from the reference checkout into
oracle/_ref/ (test infrastructure; git-ignored). Where that file is present, both implementations run
on seeded inputs at lengths the reference's own test uses (tests/test_kernel.py:33-51 of the reference)
and each output is held to the parity bar against the fp32 oracle; their mutual difference is reported.
The reference kernels run in a child process, so that a fault in them cannot take this process's CUDA
context with it. Skipped when the extension has not been built.
"""
import glob
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXT = sorted(glob.glob(os.path.join(ROOT, "oracle", "_ref", "intra_attn_cuda*.so")))

_SCRIPT = r"""
import sys, torch
sys.path.insert(0, sys.argv[1])
from intra_b200 import intra_image_attn, intra_llm_attn
from intra_b200.bench_kernel import RefExt
from oracle import intra_oracle as oracle
from tests import _util
ref = RefExt(sys.argv[2])
cases = [("llm", "scatter", 2048, 32, 8, {"group_num": 8}), ("llm", "scatter", 4096, 32, 8, {"group_num": 2}),
         ("llm", "gather1", 4096, 32, 8, {"group_num": 8}), ("llm", "window", 4096, 32, 8, {"window": 576}),
         ("image", "scatter", 512 + 64 * 64, 24, 24, {"width": 64}), ("image", "gather0", 512 + 64 * 64, 24, 24, {"width": 64})]
with torch.no_grad():
    for family, pattern, S, H, Hkv, kw in cases:
        q, k, v = oracle.make_inputs(1, S, H, Hkv, seed=0, device="cuda")
        if family == "llm":
            ours, theirs = intra_llm_attn(q, k, v, pattern, **kw), ref.llm(q, k, v, pattern, **kw)
        else:
            ours, theirs = intra_image_attn(q, k, v, pattern, **kw), ref.image(q, k, v, pattern, **kw)
        torch.cuda.synchronize()
        mask = oracle.build_mask(family, pattern, S, **kw)
        want = _util.oracle_attention(q, k, v, mask, on_device=True, fp32=True)
        e_ours = _util.check_against_oracle(ours, q, k, v, mask)
        e_ref = (theirs.float() - want.to(torch.bfloat16).float()).abs().max().item()
        diff = (ours.float() - theirs.float()).abs().max().item()
        print(f"PARITY {family}/{pattern} S={S}: ours {e_ours:.3e}  reference kernel {e_ref:.3e}  ours-vs-reference {diff:.3e}")
        assert e_ref <= 2e-2, "the reference's kernel misses its own test tolerance here"
        assert diff <= 2 * _util.ATOL
print("REFEXT-OK")
"""


@pytest.mark.skipif(not EXT, reason="oracle/_ref/intra_attn_cuda*.so has not been built (oracle/build_ref_ext.sh)")
def test_outputs_agree_with_the_reference_kernels():
    proc = subprocess.run([sys.executable, "-c", _SCRIPT, ROOT, EXT[-1]], capture_output=True, text=True,
                          timeout=900, cwd=ROOT)
    print(proc.stdout[-3000:])
    assert proc.returncode == 0 and "REFEXT-OK" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]
