"""What bench.py answers without a GPU: more than one GPU, and the reference arm."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          cwd=ROOT, timeout=120)


def test_more_than_one_gpu_is_refused_in_one_line():
    r = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert r.returncode == 0
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_shapes_are_those_of_one_architecture():
    sys.path.insert(0, ROOT)
    import bench
    from mdma_b200.config import LlamaConfig
    assert set(bench.SHAPES) == {"llama-3.1-8b", "llama-2-7b", "llama-3.2-1b"}
    for name, (label, cfg) in bench.SHAPES.items():
        c = LlamaConfig.from_dict(cfg)            # every shape is a valid configuration of the architecture
        assert c.num_attention_heads % c.num_key_value_heads == 0 and label
    assert bench.SHAPES["llama-3.1-8b"][1]["num_hidden_layers"] == 32


def test_kernel_times_parses_its_options():
    r = subprocess.run([sys.executable, "-m", "mdma_b200.kernel_times", "--help"], capture_output=True, text=True,
                       cwd=ROOT, timeout=120)
    assert r.returncode == 0 and "--context" in r.stdout and "--copies" in r.stdout


import pytest  # noqa: E402


@pytest.mark.gpu
def test_kernel_times_runs_on_the_engines_own_parts():
    """The per-kernel timing tool still runs (it drives the engine's parts and decode session, so a change
    to them shows here), on a tiny shape, with and without the rotary encoding inside the attention kernel."""
    args = ["--hidden", "128", "--intermediate", "144", "--heads", "4", "--kv-heads", "2", "--head-dim", "32",
            "--vocab", "200", "--batch", "3", "--context", "100", "--copies", "2", "--repeat", "4"]
    for env in ({}, {"MDMA_FUSED_ROTARY": "0"}):
        r = subprocess.run([sys.executable, "-m", "mdma_b200.kernel_times", *args], capture_output=True, text=True,
                           cwd=ROOT, timeout=600, env=dict(os.environ, **env))
        assert r.returncode == 0, r.stderr
        for line in ("RMSNorm", "QKV product", "attention", "O product", "gate+up", "down product",
                     "the layer as the engine runs it", "final norm + LM head", "argmax", "sample"):
            assert any(l.startswith(line) or line in l for l in r.stdout.splitlines()), (line, r.stdout)
        assert ("(one kernel)" in r.stdout) == (not env)
