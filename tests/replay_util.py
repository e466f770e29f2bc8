"""Drives bin/trace_run as a user would: a child process, JSON lines in, .f32 files out."""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(model_dir, dtype, steps, max_tokens, vocab, timeout=600):
    """steps: list of {"entries": [{"id", "tokens", "want"}], "end": [...]}.
    Returns {step number: array [wanted, vocab]}."""
    out = tempfile.mkdtemp(prefix="mdma_trace_")
    lines = "".join(json.dumps({"step": i, **s}) + "\n" for i, s in enumerate(steps))
    res = subprocess.run([sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out,
                          "--max-tokens", str(max_tokens)], input=lines, capture_output=True, text=True,
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
