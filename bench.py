#!/usr/bin/env python3
"""Benchmark: decode tokens/s and prefill tokens/s at the Llama-3.1-8B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]
    python bench.py --shape llama-2-7b | llama-3.2-1b [--batch B] [--prompt-len P] [--prefill-tokens T]

Prints ONE JSON line.  The default run has the layer sizes of the
Llama-3.1-8B shape with random bfloat16 weights, a batch of 8 sequences
decoding after 512-token prompts in a cache sized for a context of 4096.  A
"step" is one decode step of the whole batch (forward, token selection,
feeding the tokens back).  `value` is timed on the device with CUDA events
around exactly K steps; `e2e` is the same through the Python entry point
(`Generator.generate`, host token lists in and out).  Decoding streams 15 GB
of weights per step, far more than the 126 MB L2, so nothing is flushed
between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_31_8B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=32, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
    rope_theta=500000.0, rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                           high_freq_factor=4.0, original_max_position_embeddings=8192),
    rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=131072)
# The other shapes that the baseline names (same architecture, other sizes): `--shape` picks one.
LLAMA_2_7B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=32, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=32, head_dim=128, intermediate_size=11008, vocab_size=32000,
    rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=4096)
LLAMA_32_1B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=16, hidden_size=2048,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256,
    rope_theta=500000.0, rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0,
                                           high_freq_factor=4.0, original_max_position_embeddings=8192),
    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)
SHAPES = {"llama-3.1-8b": ("Llama-3.1-8B shape", LLAMA_31_8B), "llama-2-7b": ("Llama-2-7B shape", LLAMA_2_7B),
          "llama-3.2-1b": ("Llama-3.2-1B shape", LLAMA_32_1B)}


def peaks():
    """Measured peaks if the driver wrote them, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src, sustained = 6650.0, 1590.0, "fallback", None
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            hbm = float(d.get("hbm_gbs", hbm))
            tf = float(d.get("bf16_tflops", tf))
            sustained = float(d["bf16_tflops_sustained"]) if d.get("bf16_tflops_sustained") else None
            src = "measured"
        except (ValueError, OSError):
            pass
    return hbm, tf, src, sustained


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(float(s[0])) for s in self.samples if s[0].replace(".", "").isdigit())
        mx = [int(float(s[1])) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[3:7]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def matmul_params(cfg, layers):
    E, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = E * (q + 2 * kv) + q * E + 3 * E * F
    return layers * per_layer, V * E


def prefill_flops(cfg, layers, T):
    body, head = matmul_params(cfg, layers)
    attn = layers * 2 * 2 * cfg["num_attention_heads"] * cfg["head_dim"] * (T * (T + 1) // 2)
    return 2 * T * body + 2 * head + attn          # the head runs on the last row only


def decode_bytes(cfg, layers, batch, context, elem_bytes=2):
    body, head = matmul_params(cfg, layers)
    kv_row = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * layers
    return (2 * (body + head) + batch * context * kv_row) * elem_bytes // 2


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--prompt-len-range", type=int, nargs=2, default=None, metavar=("LO", "HI"),
                    help="prompt lengths drawn uniformly from [LO, HI] instead of equal prompts (seeded)")
    ap.add_argument("--shape", default="llama-3.1-8b", choices=sorted(SHAPES), help="layer sizes (default: the headline shape)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in config)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill measurements")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end measurement (profiling runs)")
    ap.add_argument("--prefill-only", action="store_true", help="run only the 2,048-token prefill (profiling runs)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the true 32-bit engine (CUDA-core kernels), for the record; the headline is bfloat16")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "AliOsm/mdma is a Rust crate (Cargo.toml, no setup.py/pyproject.toml); pip cannot "
                          "install it and no cargo/rustc is in the image"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built in this library")
        return 2
    warmup = max(3, args.warmup)

    import torch
    from mdma_b200 import ops
    from mdma_b200.engine import Engine, StepEntry
    from mdma_b200.engine.generate import Generator
    from mdma_b200.sampling import SamplingParams

    shape_name, shape_cfg = SHAPES[args.shape]
    FULL_LAYERS = shape_cfg["num_hidden_layers"]
    if args.layers is None:
        args.layers = FULL_LAYERS
    cfg = dict(shape_cfg, num_hidden_layers=args.layers)
    hbm_gbs, bf16_tflops, peak_src, sustained = peaks()
    torch.cuda.set_device(0)
    max_batch = args.batch
    eng = Engine(config=cfg, seed=0, dtype=args.dtype, max_batch=max_batch,
                 max_context=max(args.context, args.prefill_tokens))
    sampler = eng.sampler
    gen = torch.Generator().manual_seed(0)

    def prompts(n, length):
        if args.prompt_len_range is not None and length == args.prompt_len:
            lo, hi = args.prompt_len_range
            lens = torch.randint(lo, hi + 1, (n,), generator=gen).tolist()
        else:
            lens = [length] * n
        return [torch.randint(0, cfg["vocab_size"], (m,), generator=gen).tolist() for m in lens]

    def time_decode(batch, steps):
        """Device time of `steps` decode steps of `batch` sequences after prompt_len-token prompts."""
        slots = [eng.acquire() for _ in range(batch)]
        ps = prompts(batch, args.prompt_len)
        logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, ps)])
        toks, _ = sampler.sample(logits, SamplingParams.greedy(), list(range(batch)), [0] * batch)
        sess = eng.decode_session()
        sess.start(slots, toks)
        for _ in range(warmup):
            sess.run(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        done = 0
        while done < steps:             # exactly `steps` steps, replayed in runs as generation does
            done += sess.run(min(sess.max_run, steps - done))
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        per_graph = sess.launches_per_step
        mean_prompt = sum(len(p) for p in ps) / batch
        for s in slots:
            eng.release(s)
        return ms / steps, per_graph * steps, mean_prompt

    def time_prefill(T=args.prefill_tokens):
        times = []
        for i in range(warmup + 5):
            s = eng.acquire()
            p = prompts(1, T)[0]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step([StepEntry(s, p, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            eng.release(s)
            if i >= warmup:
                times.append(e0.elapsed_time(e1))
        ms_p = sorted(times)[len(times) // 2]
        fl = prefill_flops(cfg, args.layers, T)
        out = {"value": round(T * 1000.0 / ms_p, 1), "tokens": T, "ms": round(ms_p, 3),
               "frac": round(fl / (ms_p * 1e-3) / (bf16_tflops * 1e12), 4), "frac_of": f"{peak_src} burst peak"}
        if sustained:          # the same against what the library GEMM holds over seconds under the power cap
            out["frac_sustained"] = round(fl / (ms_p * 1e-3) / (sustained * 1e12), 4)
        return out

    if args.prefill_only:
        print(json.dumps({"prefill": time_prefill(), "config": {"layers": args.layers, "layers_full": FULL_LAYERS}}))
        return 0

    clock = ClockSampler()          # samples until every measurement of this run is done
    clock.start()
    ms_step, launches, mean_prompt = time_decode(args.batch, args.steps)
    value = args.batch * 1000.0 / ms_step
    ctx_end = int(mean_prompt) + warmup + args.steps
    avg_ctx = mean_prompt + warmup + args.steps / 2
    bytes_step = decode_bytes(cfg, args.layers, args.batch, avg_ctx, 2 if args.dtype == "bfloat16" else 4)
    achieved = bytes_step / (ms_step * 1e-3) / 1e9

    # end to end: host token lists in, host token lists out, through Generator.generate
    e2e = None
    if not args.no_e2e:
        stamps = []
        g = Generator(eng)
        n_e2e = args.steps + warmup + 1
        g.generate(prompts(args.batch, args.prompt_len), max_tokens=2 * g.run_ahead + 2)        # warm the path
        up0, down0 = eng.h2d_bytes, eng.d2h_bytes + sampler.d2h_bytes
        t_start = time.perf_counter()
        g.generate(prompts(args.batch, args.prompt_len), max_tokens=n_e2e,
                   on_token=lambda r, t: stamps.append(time.perf_counter()) if r == args.batch - 1 else None)
        # Host token lists go in, host token lists come out.  The tokens of `run_ahead` replayed steps reach
        # the host in one copy, so the rate is taken over the whole call but for the prompt step: from the
        # moment the first tokens are on the host to the moment the last ones are.
        e2e_value = args.batch * (len(stamps) - 1) / (stamps[-1] - stamps[0])
        n_steps = len(stamps) - 1
        e2e = {"value": round(e2e_value, 2), "unit": "tokens/s",
               # counted from the tensors copied during the call (prompt ids and step metadata up from pinned
               # memory; tokens, flags and the kernels' status word down), divided by its decode steps
               "h2d_bytes_per_step": round((eng.h2d_bytes - up0) / n_steps, 1),
               "d2h_bytes_per_step": round((eng.d2h_bytes + sampler.d2h_bytes - down0) / n_steps, 1),
               "steps": n_steps, "run_ahead": g.run_ahead,
               "with_prompt_step": round(args.batch * len(stamps) / (stamps[-1] - t_start), 2)}

    out = {
        "metric": f"decode tokens/s ({shape_name}, batch {args.batch}, after " + (
            f"{args.prompt_len}-token prompts)" if args.prompt_len_range is None else
            f"prompts of {args.prompt_len_range[0]}-{args.prompt_len_range[1]} tokens)"),
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic (uniform random token ids, random N(0,0.02) weights)",
        "impl": "ours",
        "config": {"model": shape_name, "layers": args.layers, "layers_full": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": args.context, "prompt_len": args.prompt_len,
                   "context_at_end": ctx_end, "parallelism": "single GPU", "page_size": eng.page_size,
                   "cuda_graph": True,
                   "l2": f"inputs ({bytes_step / 1e9:.1f} GB of weights and cache per step) larger than L2, no flush",
                   "peaks": peak_src},
        "e2e": e2e, "gpu_launches": launches, "clocks": None,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
    }

    if not args.no_points:
        # the other batch sizes, each on an engine built for that many sequences (as a deployment for that
        # batch size would be: the kernels plan some choices for the most sequences an engine holds)
        out["prefill"] = time_prefill()
        points = {}
        for b in (1, 64):
            if b != eng.max_slots:
                eng.check_status()
                sampler = eng = None
                import gc
                gc.collect()
                torch.cuda.empty_cache()
                eng = Engine(config=cfg, seed=0, dtype=args.dtype, max_batch=b, max_context=max(args.context, args.prefill_tokens))
                sampler = eng.sampler
            ms_b, _, _ = time_decode(b, max(8, args.steps // 2))
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 2)
        out["points"] = points
    out["clocks"] = clock.stop()
    eng.check_status()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
