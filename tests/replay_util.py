"""Drives bin/trace_run as a user would: a child process, JSON lines in, .f32 files out."""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(model_dir, dtype, steps, max_tokens, vocab, timeout=600, extra_args=()):
    """steps: list of {"entries": [{"id", "tokens", "want"}], "end": [...]}.
    Returns {step number: array [wanted, vocab]}.  `extra_args`: further options of trace_run."""
    out = tempfile.mkdtemp(prefix="mdma_trace_")
    lines = "".join(json.dumps({"step": i, **s}) + "\n" for i, s in enumerate(steps))
    res = subprocess.run([sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out,
                          "--max-tokens", str(max_tokens), *extra_args], input=lines, capture_output=True, text=True,
                         timeout=timeout)
    assert res.returncode == 0, f"trace_run failed:\n{res.stdout}\n{res.stderr}"
    done = [l for l in res.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(steps))], res.stdout
    logits = {}
    for i, s in enumerate(steps):
        n = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out, f"{i}.f32")
        if n:
            logits[i] = np.fromfile(path, dtype="<f4").reshape(n, vocab)
        else:
            assert not os.path.exists(path)
    return logits


def assert_close(got, ref, dtype, what=""):
    """Logits [rows, vocab] against the float64 oracle.  float32: 2e-5 absolute.  bfloat16: no logit off by
    more than 0.05, and no row whose root-mean-square error exceeds 2 % of the row's own deviation
    (measured on a B200 with the tests' weights: at most 0.033 and 1.4 %; one changed token among 97
    moves some later row by 0.3 and 12 % at least: tests/test_plain.py asserts that)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: logits that are not finite"
    err = np.abs(got - ref)
    if dtype == "float32":
        assert err.max() < TOL_F32, f"{what}: {err.max()}"
        return
    assert err.max() < TOL_BF16_ABS, f"{what}: {err.max()}"
    rel = np.sqrt((err ** 2).mean(axis=-1)) / ref.std(axis=-1)
    assert rel.max() < TOL_BF16_ROW, f"{what}: row error {rel.max()} of the row's deviation"


TOL_F32, TOL_BF16_ABS, TOL_BF16_ROW = 2e-5, 5e-2, 2e-2
