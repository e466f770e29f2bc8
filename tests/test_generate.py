"""Generation through the Python entry point and the command line."""
import json
import os
import subprocess
import sys

import pytest
import torch

from plain_llama import plain_forward, plain_generate, plain_sample
from tiny import SHARP, TINY_A, TINY_B, TINY_C, TINY_D, make_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def prompts_for(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]


def test_greedy_generation_matches_the_plain_implementation():
    """Tiny A, float32: prompts of 5, 11 and 17 tokens, 8 greedy tokens each."""
    import mdma_b200
    d, c, tensors = make_model(TINY_A, 0, torch.float32)
    prompts = prompts_for(TINY_A, (5, 11, 17), 0)
    outs = mdma_b200.generate(d, prompts, max_tokens=8, temperature=0.0, dtype="float32", max_batch=3)
    for p, o in zip(prompts, outs):
        assert o.tokens == plain_generate(c, tensors, p, 8)
        assert o.finish_reason == "length" and o.prompt_tokens == p


@pytest.mark.parametrize("page", [16, 32, 128])
def test_generation_with_other_page_sizes(page):
    """Cache pages of 16, 32 and 128 rows (the decode kernel's tile loads want multiples of 32, the rotary
    encoding inside it as well, the tcgen05 attention multiples of 64; what cannot be used gives way to another
    kernel): float32 tokens equal the plain implementation's, the bfloat16 engine's replayed decode equals its
    step-by-step loop, and graphs and eager steps agree across page boundaries."""
    from mdma_b200.engine import Engine
    d, c, tensors = make_model(TINY_B, 1, torch.bfloat16, std_scale=SHARP)
    prompts = prompts_for(TINY_B, (5, 70, 33, 127), 3)
    eng = Engine(d, dtype="float32", max_batch=4, max_context=256, page_size=page)
    outs = eng.generate(prompts, max_tokens=40)
    W = {k: v.float() for k, v in tensors.items()}
    for p, o in zip(prompts, outs):
        assert o.tokens == plain_generate(c, W, p, 40)
    del eng
    eng = Engine(d, dtype="bfloat16", max_batch=4, max_context=256, page_size=page)
    a = eng.generate(prompts, max_tokens=40)
    b = eng.generate(prompts, max_tokens=40, use_graphs=False)
    assert [o.tokens for o in a] == [o.tokens for o in b]
    eng.check_status()
    eng.cache.check()


def test_a_pass_size_smaller_than_the_batch():
    """An engine asked for passes of 16 tokens and 40 sequences: a decode step of 40 single tokens is one pass all
    the same (the pass size is raised to the number of slots), prompts still run in several passes."""
    from mdma_b200.engine import Engine
    d, c, tensors = make_model(TINY_A, 0, torch.float32, std_scale=SHARP)
    eng = Engine(d, dtype="float32", max_batch=40, max_context=64, chunk_tokens=16)
    assert eng.chunk_tokens == 40
    prompts = prompts_for(TINY_A, tuple(3 + i % 7 for i in range(40)), 9)
    outs = eng.generate(prompts, max_tokens=5)
    for p, o in zip(prompts[:6] + prompts[-3:], outs[:6] + outs[-3:]):
        assert o.tokens == plain_generate(c, tensors, p, 5)
    assert [o.tokens for o in outs] == [o.tokens for o in eng.generate(prompts, max_tokens=5, use_graphs=False)]
    eng.cache.check()


def test_batches_one_after_another_and_stop_tokens():
    import mdma_b200
    d, c, tensors = make_model(TINY_C, 2, torch.float32)
    prompts = prompts_for(TINY_C, (3, 40, 9, 1, 22), 5)
    free = [plain_generate(c, tensors, p, 6) for p in prompts]
    stop = [free[1][2], free[3][0]]                    # ends request 1 after two tokens, request 3 at once
    outs = mdma_b200.generate(d, prompts, max_tokens=6, dtype="float32", max_batch=2, stop_ids=stop)
    for p, o in zip(prompts, outs):
        want = plain_generate(c, tensors, p, 6, stop_ids=stop)
        assert o.tokens == want
        assert o.finish_reason == ("stop" if len(want) < 6 else "length")


def test_sampled_generation_is_seeded_and_independent_of_batch_mates():
    """Tiny B, bfloat16 weights: 4 prompts of 1, 7, 32 and 60 tokens, 16 tokens at temperature 0.8."""
    import mdma_b200
    d, c, tensors = make_model(TINY_B, 1, torch.bfloat16)
    prompts = prompts_for(TINY_B, (1, 7, 32, 60), 1)
    kw = dict(max_tokens=16, temperature=0.8, top_p=0.95, min_p=0.05, repetition_penalty=1.1, seed=11)
    for dtype in ("float32", "bfloat16"):
        a = mdma_b200.generate(d, prompts, dtype=dtype, max_batch=4, **kw)
        b = mdma_b200.generate(d, prompts, dtype=dtype, max_batch=4, **kw)
        assert [o.tokens for o in a] == [o.tokens for o in b]
        assert all(len(o.tokens) == 16 for o in a)
    other = mdma_b200.generate(d, prompts, dtype="float32", max_batch=4, **{**kw, "seed": 12})
    f32 = mdma_b200.generate(d, prompts, dtype="float32", max_batch=4, **kw)
    assert [o.tokens for o in other] != [o.tokens for o in f32]
    # the replayed decode loop keeps step counts, uniform numbers and histories on the device; the
    # step-by-step loop brings them from the host every step: the same tokens either way
    eager = mdma_b200.generate(d, prompts, dtype="float32", max_batch=4, use_graphs=False, **kw)
    assert [o.tokens for o in eager] == [o.tokens for o in f32]
    # request 2 alone, given its place in the list, draws the same tokens as inside the batch
    from mdma_b200.engine import Engine
    from mdma_b200.engine.generate import Generator
    from mdma_b200.sampling import SamplingParams, uniform
    # and the tokens follow the plain sampler on the plain model's logits
    params = SamplingParams(0.8, 0.95, 0.05, 1.1, 64, 11)
    W = {k: v.float() for k, v in tensors.items()}
    seq = list(prompts[2])
    for step in range(8):
        logits = plain_forward(c, W, seq, torch.float32)[-1]
        tok = plain_sample(logits.tolist(), seq, uniform(11, 2, step), 0.8, 0.95, 0.05, 1.1, 64)
        assert tok == f32[2].tokens[step], step
        seq.append(tok)


def test_repetition_window_longer_than_the_default_history():
    """A window of 100 tokens: the sampler's per-row history grows to hold it, in the replayed loop and in
    the step-by-step loop, and the tokens follow the plain sampler with that window."""
    import mdma_b200
    from mdma_b200.sampling import uniform
    d, c, tensors = make_model(TINY_B, 1, torch.bfloat16)
    prompts = prompts_for(TINY_B, (120, 90), 3)
    kw = dict(max_tokens=12, temperature=0.9, top_p=0.9, min_p=0.02, repetition_penalty=1.4, repetition_window=100, seed=5,
              dtype="float32", max_batch=2)
    got = mdma_b200.generate(d, prompts, **kw)
    eager = mdma_b200.generate(d, prompts, use_graphs=False, **kw)
    assert [o.tokens for o in got] == [o.tokens for o in eager]
    W = {k: v.float() for k, v in tensors.items()}
    seq = list(prompts[0])
    for step in range(6):
        logits = plain_forward(c, W, seq, torch.float32)[-1]
        tok = plain_sample(logits.tolist(), seq, uniform(5, 0, step), 0.9, 0.9, 0.02, 1.4, 100)
        assert tok == got[0].tokens[step], step
        seq.append(tok)


def test_command_line(tmp_path):
    d, c, tensors = make_model(TINY_A, 0, torch.float32, norm_jitter=0)     # as the seed alone gives it (--random-weights below)
    p = prompts_for(TINY_A, (6,), 3)[0]
    want = plain_generate(c, tensors, p, 5)
    env = dict(os.environ, PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mdma"), "run", d, ",".join(map(str, p)),
                          "--max-tokens", "5", "--dtype", "float32", "--json"], capture_output=True, text=True, env=env)
    assert res.returncode == 0, res.stderr
    out = json.loads(res.stdout.strip().splitlines()[-1])
    assert out["tokens"] == want and out["prompt_tokens"] == p and out["finish_reason"] == "length"
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mdma-run"), d, " ".join(map(str, p)), "5"],
                         capture_output=True, text=True, env=dict(env, MDMA_JSON="1"))
    assert res.returncode == 0, res.stderr
    assert json.loads(res.stdout.strip().splitlines()[-1])["tokens"][:5] == json.loads(
        subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mdma"), "run", d, ",".join(map(str, p)),
                        "--max-tokens", "5", "--json"], capture_output=True, text=True, env=env).stdout.strip().splitlines()[-1])["tokens"]
    # seeded random weights from the configuration alone: the same tokens as from the folder written with that seed
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mdma"), "run", os.path.join(d, "config.json"),
                          ",".join(map(str, p)), "--max-tokens", "5", "--dtype", "float32", "--json", "--random-weights", "0"],
                         capture_output=True, text=True, env=env)
    assert res.returncode == 0, res.stderr
    assert json.loads(res.stdout.strip().splitlines()[-1])["tokens"] == want
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mdma"), "plan", d, "--ctx", "64", "--json"],
                         capture_output=True, text=True, env=env)
    plan = json.loads(res.stdout)
    assert plan["total_bytes"] == sum(v for k, v in plan.items() if k.endswith("_bytes") and k != "total_bytes")


def test_engine_refuses_bad_steps_and_keeps_its_cache():
    from mdma_b200.engine import Engine, StepEntry, StepError
    d, c, tensors = make_model(TINY_A, 0, torch.float32)
    eng = Engine(d, dtype="float32", max_batch=2, max_context=64)
    s = eng.acquire()
    eng.step([StepEntry(s, [1, 2, 3], [2])])
    for bad in ([StepEntry(s, [999], [0])], [StepEntry(s, [], [])], [StepEntry(s, [1], [1])],
                [StepEntry(5, [1], [0])], [StepEntry(s, [1], [0]), StepEntry(s, [2], [0])],
                [StepEntry(s, [1] * 62, [0])], []):
        with pytest.raises(StepError):
            eng.step(bad)
        assert eng.cache.length(s) == 3
        eng.cache.check()
    ref = plain_forward(c, tensors, [1, 2, 3, 4], torch.float64)[-1]
    got = eng.step([StepEntry(s, [4], [0])])[0].double().cpu()
    assert (got - ref).abs().max() < 2e-5


def test_memory_plan_refuses_what_does_not_fit():
    from mdma_b200.engine import Engine, MemoryBudgetError
    d, _, _ = make_model(TINY_A, 0, torch.float32)
    with pytest.raises(MemoryBudgetError) as e:
        Engine(d, dtype="float32", max_batch=2, vram_bytes=1 << 20, reserve_mib=0)
    assert e.value.requested > e.value.available


def test_missing_library_fails_loudly(monkeypatch):
    from mdma_b200.csrc import build
    monkeypatch.setattr(build, "_loaded", {})
    monkeypatch.setattr(build, "library_path", lambda name: "/nonexistent/lib.so")
    monkeypatch.setattr(build, "find_nvcc", lambda: (_ for _ in ()).throw(build.BuildError("nvcc was not found")))
    from mdma_b200 import ops
    with pytest.raises(build.BuildError):
        ops.argmax(torch.zeros(1, 4, device="cuda:0"), torch.zeros(1, dtype=torch.int32, device="cuda:0"))


def test_plan_equals_what_is_held():
    """The memory plan, made from sizes alone, is what the engine then holds (the reference's rule:
    src/model/arch/llama/tests.rs:8-66, src/model/planning/tests.rs:6-30): every category, the total, and
    what the allocator says the process took; and generation takes nothing more, however long it runs."""
    import gc
    from mdma_b200.engine import Engine
    from mdma_b200.engine.step import plan_only
    for cfg, seed, wdtype, dtype in ((TINY_A, 0, torch.float32, "float32"), (TINY_B, 1, torch.bfloat16, "bfloat16"),
                                     (TINY_C, 2, torch.float32, "bfloat16")):
        d, _, _ = make_model(cfg, seed, wdtype)
        gc.collect()                    # engines of earlier tests give their memory back now, not in between
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        eng = Engine(d, dtype=dtype, max_batch=3, max_context=128)
        held = eng.held_bytes()
        assert eng.plan["total_bytes"] == held["total_bytes"] == sum(v for k, v in held.items() if k != "total_bytes")
        for key, value in held.items():
            assert eng.plan[key] == value, (key, eng.plan[key], value)
        taken = torch.cuda.memory_allocated() - before
        # one allocation; the allocator hands out segments of 2 MiB and counts a tail it cannot split off
        assert 0 <= taken - eng.plan["total_bytes"] < (2 << 20), (taken, eng.plan["total_bytes"])
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        alone = plan_only(d, dtype=dtype, max_batch=3, max_context=128, sms=sms)
        assert alone == eng.plan
        prompts = prompts_for(cfg, (5, 40, 17), seed)
        eng.generate(prompts, max_tokens=20)                    # warm: kernels loaded, graphs captured
        eng.generate(prompts, max_tokens=20, temperature=0.7, seed=3)
        torch.cuda.synchronize()
        warm = torch.cuda.memory_allocated()
        for seed2 in range(4):                                  # other options and seeds: the same graphs
            eng.generate(prompts, max_tokens=30, temperature=0.9, top_p=0.9, seed=seed2)
            eng.generate(prompts[::-1], max_tokens=30)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == warm
        assert len(eng.decode_session().graphs) <= 2 * 3        # (batch size 1..3) x (argmax, draw)
        del eng


def test_nothing_is_allocated_before_a_refusal(tmp_path):
    """A folder with a wrong tensor, a configuration no kernel takes and a plan beyond the budget are all
    refused before any device memory is taken (the reference counts its backend's allocations the same way:
    src/model/arch/llama/preflight/tests.rs:98-116)."""
    import json as _json
    from mdma_b200 import WeightsError
    from mdma_b200.engine import Engine, MemoryBudgetError
    from mdma_b200.weights import write_safetensors
    from mdma_b200.weights.safetensors_io import SafetensorsFile
    import gc
    gc.collect()
    torch.cuda.synchronize()

    def allocations():
        return torch.cuda.memory_stats()["allocation.all.allocated"]
    d, _, tensors = make_model(TINY_A, 0, torch.float32)
    # a folder whose head has one row too few, and a stray tensor
    bad = dict(tensors)
    bad["lm_head.weight"] = bad["lm_head.weight"][:-1].contiguous()
    bad["stray.bias"] = torch.zeros(3)
    write_safetensors(str(tmp_path / "model.safetensors"), bad)
    (tmp_path / "config.json").write_text(open(os.path.join(d, "config.json")).read())
    n0 = allocations()
    with pytest.raises(WeightsError):
        Engine(str(tmp_path), dtype="float32", max_batch=2)
    assert allocations() == n0
    # a head wider than any attention kernel takes
    wide = dict(TINY_A, head_dim=512)
    with pytest.raises(ValueError, match="head_dim 512"):
        Engine(config=wide, seed=0, dtype="float32", max_batch=2)
    assert allocations() == n0
    with pytest.raises(MemoryBudgetError):
        Engine(d, dtype="float32", max_batch=2, vram_bytes=1 << 20, reserve_mib=0)
    assert allocations() == n0


def test_graph_replay_equals_eager():
    """Decode steps replayed as CUDA graphs give the tokens of the eager path, greedy and sampled
    (the reference asks the same of its graph decoder: src/backend/test_support/graph.rs:16-75)."""
    import mdma_b200
    for cfg, seed, wdtype in ((TINY_A, 0, torch.float32), (TINY_B, 1, torch.bfloat16)):
        d, _, _ = make_model(cfg, seed, wdtype)
        prompts = prompts_for(cfg, (5, 11, 17, 3), 0)
        for dtype in ("float32", "bfloat16"):
            for kw in (dict(temperature=0.0), dict(temperature=0.8, top_p=0.9, repetition_penalty=1.1, seed=5)):
                a = mdma_b200.generate(d, prompts, max_tokens=12, dtype=dtype, max_batch=4, use_graphs=True, **kw)
                b = mdma_b200.generate(d, prompts, max_tokens=12, dtype=dtype, max_batch=4, use_graphs=False, **kw)
                assert [o.tokens for o in a] == [o.tokens for o in b], (dtype, kw)


def test_engine_generate_method():
    from mdma_b200.engine import Engine
    d, c, tensors = make_model(TINY_A, 0, torch.float32)
    eng = Engine(d, dtype="float32", max_batch=2, max_context=64)
    p = prompts_for(TINY_A, (6, 9), 3)
    outs = eng.generate(p, max_tokens=5)
    assert [o.tokens for o in outs] == [plain_generate(c, tensors, q, 5) for q in p]
    assert eng.generate(p, max_tokens=5)[0].tokens == outs[0].tokens       # slots were given back: it runs again


def test_generation_across_the_1024_bucket_and_run_ahead():
    """Prompts of 1,015 and 40 tokens, 30 tokens each: the longer sequence passes 1,024 positions, where
    the decode graphs of the next bucket are captured and the attention kernel changes its variant.
    Replayed in runs of eight steps, in runs of one, and step by step without graphs: the same tokens."""
    from mdma_b200.engine import Engine
    from mdma_b200.engine.generate import Generator
    from mdma_b200.sampling import SamplingParams
    d, c, tensors = make_model(TINY_D, 3, torch.bfloat16, std_scale=SHARP)
    prompts = prompts_for(TINY_D, (1015, 40, 300), 6)
    for dtype in ("float32", "bfloat16"):
        eng = Engine(d, dtype=dtype, max_batch=3, max_context=1100)
        for params in (SamplingParams.greedy(), SamplingParams(0.8, 0.95, 0.05, 1.2, 64, 9)):
            runs = Generator(eng, run_ahead=8).generate(prompts, 30, params)
            ones = Generator(eng, run_ahead=1).generate(prompts, 30, params)
            eager = Generator(eng, use_graphs=False).generate(prompts, 30, params)
            assert [o.tokens for o in runs] == [o.tokens for o in eager], (dtype, params)
            assert [o.tokens for o in ones] == [o.tokens for o in eager], (dtype, params)
            assert all(len(o.tokens) == 30 for o in runs)
        # a stop token inside a run: the sequence ends there, the others go on
        free = Generator(eng).generate(prompts, 30)
        stop = [free[1].tokens[11]]
        cut = Generator(eng, run_ahead=8).generate(prompts, 30, stop_ids=stop)
        step = Generator(eng, use_graphs=False).generate(prompts, 30, stop_ids=stop)
        assert [o.tokens for o in cut] == [o.tokens for o in step]
        assert cut[1].finish_reason == "stop" and len(cut[1].tokens) <= 11
        eng.cache.check()
        assert not eng.cache.lengths                           # every slot was given back
        del eng


def test_logits_of_the_replayed_decode_step_match_the_oracle():
    """The graph-replayed decode step lays out its own inputs; its logits (not only its tokens) are
    compared with the plain implementation, across 1,024 positions, in both dtypes."""
    from mdma_b200.engine import Engine, StepEntry
    from mdma_b200.sampling import SamplingParams
    from replay_util import assert_close
    d, c, tensors = make_model(TINY_D, 3, torch.bfloat16, std_scale=SHARP)
    W = {k: v.float() for k, v in tensors.items()}
    prompts = prompts_for(TINY_D, (1019, 37), 8)
    for dtype in ("float32", "bfloat16"):
        eng = Engine(d, dtype=dtype, max_batch=2, max_context=1100)
        slots = [eng.acquire() for _ in prompts]
        logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        tokens, _ = eng.sampler.sample(logits, SamplingParams.greedy(), [0, 1], [0, 0])
        seqs = [list(p) + [t] for p, t in zip(prompts, tokens)]
        sess = eng.decode_session()
        sess.start(slots, tokens)
        kept = []
        for _ in range(12):
            sess.run(1)
            toks, flags = sess.read()[-1]
            assert flags == [0, 0]
            kept.append(sess.logits[:2].double().cpu().numpy())
            for q, t in zip(seqs, toks):
                q.append(t)
        assert len(sess.graphs) == 2                            # one per bucket of 1,024 positions
        for i, q in enumerate(seqs):
            ref = plain_forward(c, W, q[:-1], torch.float64).numpy()
            for j in range(12):
                assert_close(kept[j][i], ref[len(prompts[i]) + j], dtype, f"replayed step {j}, sequence {i}")
        for s in slots:
            eng.release(s)
        del eng


def test_generation_reports_a_kernel_that_gave_up():
    """The status word that a bounded wait sets travels to the host with every step's tokens; generation
    raises instead of handing out tokens of a step that is not valid, gives its slots back, and the
    next call is clean."""
    from mdma_b200.engine import Engine
    from mdma_b200.engine.generate import Generator
    from mdma_b200.ops import KernelError
    d, c, tensors = make_model(TINY_B, 1, torch.bfloat16, std_scale=SHARP)
    eng = Engine(d, dtype="bfloat16", max_batch=2, max_context=128)
    p = prompts_for(TINY_B, (6, 9), 3)
    want = [o.tokens for o in eng.generate(p, max_tokens=12)]
    eng.rt.tc.status[0] = 3                         # as a block of a product kernel would
    with pytest.raises(KernelError, match="wait limit"):
        eng.generate(p, max_tokens=12)
    assert not eng.cache.lengths and int(eng.rt.tc.status[0]) == 0
    assert [o.tokens for o in eng.generate(p, max_tokens=12)] == want
    # during the replayed steps too: the word is read with each run's tokens
    calls = []

    def poison_once(request, token):
        calls.append(token)
        if len(calls) == 8:
            eng.rt.tc.status[0] = 1
    with pytest.raises(KernelError, match="wait limit"):
        Generator(eng).generate(p, 40, on_token=poison_once)
    assert not eng.cache.lengths
    assert [o.tokens for o in eng.generate(p, max_tokens=12)] == want


def test_an_engine_from_a_seed_holds_the_bits_of_the_folder_written_from_it():
    """Seeded random weights are a function of (seed, tensor name, element): the device fills its arena with
    the same bits that the folder writer produces on the host, so the same seed means the same model."""
    from mdma_b200.engine import Engine, StepEntry
    for cfg, seed, dtype in ((TINY_B, 5, "bfloat16"), (TINY_C, 6, "float32")):
        wd = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        d, c, tensors = make_model(cfg, seed, wd, std_scale=SHARP, norm_jitter=0)
        from_seed = Engine(config=cfg, seed=seed, dtype=dtype, max_batch=2, max_context=64, init_std=0.02 * SHARP)
        from_folder = Engine(d, dtype=dtype, max_batch=2, max_context=64)
        a = [t for p in from_seed.model.all_parts() for t in p.resident_tensors()]
        b = [t for p in from_folder.model.all_parts() for t in p.resident_tensors()]
        assert len(a) == len(b) and all(torch.equal(x, y) for x, y in zip(a, b))
        ids = prompts_for(cfg, (20,), 1)[0]
        la = from_seed.step([StepEntry(from_seed.acquire(), ids, [19])]).clone()
        lb = from_folder.step([StepEntry(from_folder.acquire(), ids, [19])])
        assert torch.equal(la, lb)


def test_graphs_survive_a_step_that_uses_the_large_scratch():
    """The kernels' scratch is taken once, for the largest step the engine can run, and never replaced:
    decode graphs captured after short prompts still hold valid addresses after a 300-token prompt has
    gone through the block-pair product (which keeps partial tiles in that scratch), in the same engine
    and in a second engine of the same process."""
    from mdma_b200.engine import Engine
    d, c, tensors = make_model(TINY_D, 3, torch.bfloat16, std_scale=SHARP)
    eng = Engine(d, dtype="bfloat16", max_batch=2, max_context=512)
    short = prompts_for(TINY_D, (5, 9), 21)
    long = prompts_for(TINY_D, (300, 140), 22)
    first = [o.tokens for o in eng.generate(short, max_tokens=16)]
    scratch = eng.rt.tc.scratch.data_ptr()
    eng.generate(long, max_tokens=4)
    other = Engine(d, dtype="bfloat16", max_batch=2, max_context=512)
    other.generate(long, max_tokens=4)
    assert eng.rt.tc.scratch.data_ptr() == scratch and other.rt.tc.scratch.data_ptr() != scratch
    assert [o.tokens for o in eng.generate(short, max_tokens=16)] == first          # replayed graphs
    assert [o.tokens for o in eng.generate(short, max_tokens=16, use_graphs=False)] == first


def test_loading_in_pieces_through_pinned_memory():
    """Tensors larger than the staging pieces (here 4 KiB) arrive whole, whatever their stored dtype."""
    from mdma_b200.config import load_config
    from mdma_b200.engine.model import DecoderModel
    from mdma_b200.weights import load_tensors, resident_dtype
    d, c, tensors = make_model(TINY_C, 2, torch.float32)
    arch, cfg = load_config(d)
    expected = DecoderModel(arch.describe(cfg)).expected_tensors()
    for compute in (torch.bfloat16, torch.float32):
        into = {n: torch.full(ts.shape, 7.0, dtype=resident_dtype(ts, torch.float32, compute), device="cuda:0")
                for n, ts in expected.items()}
        load_tensors(d, expected, compute, torch.device("cuda:0"), into=into, staging_bytes=4096)
        for n, t in tensors.items():
            assert torch.equal(into[n].cpu(), t.to(into[n].dtype)), n


@pytest.mark.parametrize("lengths", [(300, 70, 9), (150, 70, 9)])
def test_the_benchmark_layer_shape_in_bfloat16_against_true_32_bit(lengths):
    """Two layers of the Llama-3.1-8B shape (hidden 4096, 32/8 heads of 128, intermediate 14336, vocabulary
    128,256; random weights from a seed): prompts of 300, 70 and 9 tokens in one step (or 150, 70 and 9: a
    step of 129-256 tokens, whose O and down products run one block per tile with a K split left for the
    norms), then four steps of
    one token each, through the tensor-core kernels at their real sizes (block-pair products, the SwiGLU
    product's even split, K splits left for the norms, the head over 128k rows) against the same model in
    the float32 engine (CUDA-core kernels, no reduced precision anywhere).  The float32 engine keeps the
    seed's weights unrounded, so the difference includes rounding the weights to bfloat16 once:
    measured 0.11 at most on logits of deviation 1.28, 1.8 % of a row's deviation in the root mean square."""
    import numpy as np
    import bench
    from mdma_b200.engine import Engine, StepEntry
    cfg = dict(bench.LLAMA_31_8B, num_hidden_layers=2, max_position_embeddings=1024)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    res = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(config=cfg, seed=0, dtype=dtype, max_batch=3, max_context=512, logit_rows=16)
        slots = [eng.acquire() for _ in prompts]
        out = [eng.step([StepEntry(s, p, [0, len(p) // 2, len(p) - 1]) for s, p in zip(slots, prompts)]).cpu().numpy().copy()]
        for j in range(4):
            out.append(eng.step([StepEntry(s, [p[j]], [0]) for s, p in zip(slots, prompts)]).cpu().numpy().copy())
        eng.check_status()
        res[dtype] = np.concatenate(out).astype(np.float64)
        del eng
    a, b = res["float32"], res["bfloat16"]
    assert np.isfinite(b).all() and 1.0 < a.std() < 1.6
    err = np.abs(a - b)
    assert err.max() < 0.2, err.max()
    assert (np.sqrt((err ** 2).mean(1)) / a.std(1)).max() < 0.03


def test_long_prompts_at_the_benchmark_layer_shape_against_true_32_bit():
    """The same two layers with prompts of 2,500, 700 and 130 tokens: a first step of all but the last 64
    tokens as passes of 1,024 (the tcgen05 attention over dozens of key blocks, some of them cached by an
    earlier pass; block-pair products over many token tiles), a step of 56 tokens on that prefix, then eight
    steps of one token, the longest sequence beyond 2,048 positions (keys split over blocks).  Against the
    float32 engine, whose weights are not rounded: measured 0.116 at most on logits of deviation 1.28 and
    1.9 % of a row's deviation in the root mean square, the same on every row."""
    import numpy as np
    import bench
    from mdma_b200.engine import Engine, StepEntry
    cfg = dict(bench.LLAMA_31_8B, num_hidden_layers=2, max_position_embeddings=4096)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (2500, 700, 130)]
    res = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(config=cfg, seed=0, dtype=dtype, max_batch=3, max_context=2688, logit_rows=32, chunk_tokens=1024)
        slots = [eng.acquire() for _ in prompts]
        wants = lambda p: [0, len(p) // 3, len(p) // 2, len(p) - 2, len(p) - 1]
        out = [eng.step([StepEntry(s, p[:-64], wants(p[:-64])) for s, p in zip(slots, prompts)]).cpu().numpy().copy()]
        out.append(eng.step([StepEntry(s, p[-64:-8], [0, 55]) for s, p in zip(slots, prompts)]).cpu().numpy().copy())
        for j in range(8):
            out.append(eng.step([StepEntry(s, [p[len(p) - 8 + j]], [0]) for s, p in zip(slots, prompts)]).cpu().numpy().copy())
        eng.check_status()
        res[dtype] = np.concatenate(out).astype(np.float64)
        del eng
    a, b = res["float32"], res["bfloat16"]
    assert a.shape[0] == 45 and np.isfinite(b).all() and 1.0 < a.std() < 1.6
    err = np.abs(a - b)
    assert err.max() < 0.2, err.max()
    assert (np.sqrt((err ** 2).mean(1)) / a.std(1)).max() < 0.03


def test_random_traffic_replayed_runs_equal_the_step_by_step_loop():
    """Random batches (1-9 prompts of 1 to context-5 tokens, budgets of 1-40 tokens, greedy or sampled with
    random options, random stop tokens, runs of 1, 3 or 8 replayed steps): the same tokens and finish
    reasons as the loop that runs every step on its own, sequences ending inside runs and batches shrinking
    included, and no slot or page lost.  The kernels' choices depend on the engine's capacity, not on the
    live batch, within these sizes; that is what makes the two loops agree bit for bit."""
    import random
    from mdma_b200.engine import Engine
    from mdma_b200.engine.generate import Generator
    from mdma_b200.sampling import SamplingParams
    rnd = random.Random(0)
    for cfg, seed, wd, dtype in ((TINY_D, 3, torch.bfloat16, "bfloat16"), (TINY_B, 1, torch.bfloat16, "bfloat16"),
                                 (TINY_C, 2, torch.float32, "float32")):
        d, c, tensors = make_model(cfg, seed, wd, std_scale=SHARP)
        ctx = min(cfg["max_position_embeddings"], 700)
        eng = Engine(d, dtype=dtype, max_batch=6, max_context=ctx, max_tokens=6 * 64 * 4)
        g = torch.Generator().manual_seed(seed)
        for it in range(40):
            lens = [max(1, min(rnd.choice([1, 2, 5, 17, 63, 64, 65, 100, 130, ctx - 40, ctx - 5]), ctx - 1))
                    for _ in range(rnd.randint(1, 9))]
            prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
            max_tokens = rnd.choice([1, 2, 7, 8, 9, 20, 40])
            params = SamplingParams.greedy() if rnd.random() < 0.5 else SamplingParams(
                rnd.choice([0.5, 0.8, 1.2]), rnd.choice([1.0, 0.9]), rnd.choice([0.0, 0.05]), rnd.choice([1.0, 1.3]),
                rnd.choice([0, 16, 64, 200]), rnd.randint(0, 99))
            stop = [rnd.randrange(cfg["vocab_size"]) for _ in range(rnd.choice([0, 0, 3, 10]))]
            runs = Generator(eng, run_ahead=rnd.choice([1, 3, 8])).generate(prompts, max_tokens, params, stop)
            steps = Generator(eng, use_graphs=False).generate(prompts, max_tokens, params, stop)
            assert [(o.tokens, o.finish_reason) for o in runs] == [(o.tokens, o.finish_reason) for o in steps], (it, lens)
            eng.cache.check()
            assert not eng.cache.lengths
        eng.check_status()
        del eng
