"""The latency-table CLI (`python -m intra_b200.bench_kernel`) writes files in the format of the
reference's benchmarks/bench_kernel.py (its result files benchmarks/results/a100_llm.json and
a100_image.json): same top-level keys, same argument record, same row keys, plus this build's extras."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# keys of the reference's result files
REF_TOP = {"device", "args", "rows"}
REF_ARGS = {"mode", "seqlens", "groups", "batch", "heads", "kv_heads", "image_heads", "warmup", "iters"}
REF_LLM_ROW = ["seqlen", "dense", "scatter_g2", "scatter_g8", "gather1_g8", "window576", "g2s4_32layer", "dense_32layer"]
REF_IMAGE_ROW = ["width", "seqlen", "dense", "scatter", "gather0", "interleaved_mean"]


def _run(tmp_path, *argv):
    out = tmp_path / "rows.json"
    proc = subprocess.run([sys.executable, "-m", "intra_b200.bench_kernel", *argv, "--iters", "2", "--warmup", "1",
                           "--out", str(out)], capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    with open(out) as f:
        return json.load(f)


def _check(doc, row_keys, sparse_keys):
    assert REF_TOP <= set(doc) and REF_ARGS <= set(doc["args"])
    for row in doc["rows"]:
        assert [k for k in row if not k.endswith("_tflops")] == row_keys, "row keys or their order differ from the reference's"
        assert {k[:-7] for k in row if k.endswith("_tflops")} == set(sparse_keys)
        for k in sparse_keys:
            assert row[k] > 0 and row[k + "_tflops"] > 0


def test_llm_table_has_the_reference_format(tmp_path):
    doc = _run(tmp_path, "llm", "--seqlens", "1024,2048")
    assert [r["seqlen"] for r in doc["rows"]] == [1024, 2048] and doc["args"]["mode"] == "llm"
    _check(doc, REF_LLM_ROW, ["scatter_g2", "scatter_g8", "gather1_g8", "window576"])
    r = doc["rows"][0]
    assert abs(r["g2s4_32layer"] - (4 * r["scatter_g2"] + 28 * r["window576"])) < 1e-9
    assert doc["dense_backend"]


def test_image_table_has_the_reference_format(tmp_path):
    doc = _run(tmp_path, "image")
    assert [r["width"] for r in doc["rows"]] == [64, 128]
    _check(doc, REF_IMAGE_ROW, ["scatter", "gather0"])


def test_stack_mode_runs_the_layer_schedule(tmp_path):
    doc = _run(tmp_path, "stack", "--seqlens", "2048", "--layers", "8", "--stack-iters", "2")
    r = doc["rows"][0]
    assert r["layers"] == 8 and r["intra_ms"] > 0 and r["intra_tflops"] > 0
