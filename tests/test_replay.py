"""Trace replay against the plain implementation, in 32-bit and in bfloat16:
whole requests, the last 32 tokens one by one, batches of unequal lengths whose
slots are used again; and the schedules that only show in particular cuts: a
step run as several passes, a prompt fed in unequal pieces next to a batch
mate that decodes, decoding across the 1,024-position bucket of the decode
graphs, batches so large that the decode attention changes its variant, and
all of it with NaN in every cache row that belongs to nobody."""
import numpy as np
import pytest
import torch

from plain_llama import plain_forward
from replay_util import assert_close, replay
from tiny import SHARP, TINY_A, TINY_B, TINY_C, TINY_D, TINY_E, make_model

pytestmark = pytest.mark.gpu

CASES = [("a", TINY_A, 0, torch.float32), ("b", TINY_B, 1, torch.bfloat16), ("c", TINY_C, 2, torch.bfloat16)]
DTYPES = ["float32", "bfloat16"]


def requests_for(cfg, seed, lengths):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
            for i, n in enumerate(lengths)}


def oracle(c, tensors, ids, dtype="float32"):
    """float64 arithmetic on the weights the engine holds: the bfloat16 engine keeps matrices in
    bfloat16, so a folder stored in float32 is rounded once when it is loaded."""
    held = {k: (v.bfloat16().float() if dtype == "bfloat16" and v.dim() == 2 else v.float()) for k, v in tensors.items()}
    return plain_forward(c, held, ids, torch.float64).numpy()


def batched_trace(reqs, batches):
    """Way 3: every batch starts with a third of each prompt in one step, then one token per live
    request per step; shorter requests end earlier.  Returns (steps, [(request, place) per wanted row])."""
    steps, index = [], []
    for batch in batches:
        prompt = {rid: max(1, len(reqs[rid]) // 3) for rid in batch}
        steps.append({"entries": [{"id": rid, "tokens": reqs[rid][:prompt[rid]],
                                   "want": [0, prompt[rid] - 1] if prompt[rid] > 1 else [0]} for rid in batch], "end": []})
        index.append([(rid, p) for rid in batch for p in ((0, prompt[rid] - 1) if prompt[rid] > 1 else (0,))])
        pos = dict(prompt)
        live = [rid for rid in batch if pos[rid] < len(reqs[rid])]
        if len(live) < len(batch):
            steps[-1]["end"] = [rid for rid in batch if rid not in live]
        while live:
            entries = [{"id": rid, "tokens": [reqs[rid][pos[rid]]], "want": [0]} for rid in live]
            for rid in live:
                pos[rid] += 1
            ended = [rid for rid in live if pos[rid] == len(reqs[rid])]
            steps.append({"entries": entries, "end": ended})
            index.append([(rid, pos[rid] - 1) for rid in live])
            live = [rid for rid in live if rid not in ended]
    return steps, index


def check_rows(got, index, ref, dtype, what):
    for i, places in enumerate(index):
        want = np.stack([ref[rid][p] for rid, p in places])
        assert_close(got[i], want, dtype, f"{what}, step {i} {places[:3]}")


@pytest.mark.parametrize("name,cfg,seed,wdtype", CASES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_replay_three_ways(name, cfg, seed, wdtype, dtype):
    d, c, tensors = make_model(cfg, seed, wdtype, std_scale=SHARP)
    V = cfg["vocab_size"]
    lengths = [40, 97, 33, 70, 64, 128][: 6 if cfg["max_position_embeddings"] >= 128 else 4]
    reqs = requests_for(cfg, seed, lengths)
    ref = {rid: oracle(c, tensors, ids, dtype) for rid, ids in reqs.items()}

    # 1. each request alone and whole: one step, logits at every place
    steps = [{"entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
             for rid, ids in reqs.items()]
    got = replay(d, dtype, steps, max_tokens=128, vocab=V)
    whole = {}
    for i, rid in enumerate(reqs):
        whole[rid] = got[i]
        assert_close(got[i], ref[rid], dtype, f"whole {rid}")

    # 2. the last 32 tokens one by one
    steps, index = [], []
    for rid, ids in reqs.items():
        head = len(ids) - 32
        steps.append({"entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
        index.append((rid, 0, head))
        for j in range(head, len(ids)):
            steps.append({"entries": [{"id": rid, "tokens": [ids[j]], "want": [0]}],
                          "end": [rid] if j == len(ids) - 1 else []})
            index.append((rid, j, j + 1))
    got = replay(d, dtype, steps, max_tokens=128, vocab=V)
    for i, (rid, lo, hi) in enumerate(index):
        assert_close(got[i], ref[rid][lo:hi], dtype, f"one-by-one {rid} places {lo}..{hi}")
        if dtype == "float32":        # the same arithmetic whatever the cut
            assert np.abs(got[i] - whole[rid][lo:hi]).max() < 2e-6

    # 3. batches of unequal lengths; shorter requests end earlier; one batch after another
    rids = list(reqs)
    batches = (rids[:3], rids[3:], rids[:2][::-1])
    steps, index = batched_trace(reqs, batches)
    # the cache holds just the largest batch: slots and pages must be used again
    need = max(sum(-(-len(reqs[r]) // 64) * 64 for r in b) for b in batches)
    got = replay(d, dtype, steps, max_tokens=need, vocab=V)
    check_rows(got, index, ref, dtype, "batched")


@pytest.mark.parametrize("name,cfg,seed,wdtype", CASES + [("d", TINY_D, 3, torch.bfloat16)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_rows_that_belong_to_nobody_do_not_leak(name, cfg, seed, wdtype, dtype):
    """Way 3 again, with every cache row that no live request owns (free pages, rows beyond a request's
    length) filled with NaN before each step: a kernel that fetches whole tiles must not let them
    through.  The reference's rule is `written` against `len` (src/kv_cache.rs:246-268)."""
    d, c, tensors = make_model(cfg, seed, wdtype, std_scale=SHARP)
    V = cfg["vocab_size"]
    reqs = requests_for(cfg, seed + 10, [70, 33, 97, 5, 64, 41])
    ref = {rid: oracle(c, tensors, ids, dtype) for rid, ids in reqs.items()}
    rids = list(reqs)
    batches = (rids[:3], rids[3:], rids[1:3][::-1])
    steps, index = batched_trace(reqs, batches)
    need = max(sum(-(-len(reqs[r]) // 64) * 64 for r in b) for b in batches)
    got = replay(d, dtype, steps, max_tokens=need, vocab=V, extra_args=("--poison-unused",))
    check_rows(got, index, ref, dtype, "poisoned")
    # whole prompts too (the kernels of steps with many tokens), pages used again after a longer request
    steps = [{"entries": [{"id": rid, "tokens": reqs[rid], "want": [0, len(reqs[rid]) - 1]}], "end": [rid]}
             for rid in (rids[2], rids[1], rids[0])]
    got = replay(d, dtype, steps, max_tokens=128, vocab=V, extra_args=("--poison-unused",))
    for i, rid in enumerate((rids[2], rids[1], rids[0])):
        assert_close(got[i], ref[rid][[0, len(reqs[rid]) - 1]], dtype, f"poisoned whole {rid}")


@pytest.mark.parametrize("name,cfg,seed,wdtype", [CASES[0], CASES[2]])
@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_run_as_several_passes(name, cfg, seed, wdtype, dtype):
    """Three unequal prompts in ONE step on an engine that runs at most 48 tokens per pass: the step is
    cut into five passes (one prompt is cut twice, one shares a pass with the tail of another), wanted
    places lie on both sides of the cuts, and one list of places is out of order across a cut."""
    d, c, tensors = make_model(cfg, seed, wdtype, std_scale=SHARP)
    V = cfg["vocab_size"]
    reqs = requests_for(cfg, seed + 20, [100, 37, 75])
    ref = {rid: oracle(c, tensors, ids, dtype) for rid, ids in reqs.items()}
    wants = {"r0": [47, 48, 0, 99, 95, 96, 1], "r1": [36, 0, 10, 11], "r2": [74, 8, 9, 60]}
    steps = [{"entries": [{"id": rid, "tokens": reqs[rid], "want": wants[rid]} for rid in reqs], "end": []}]
    # then every request goes on by one token that repeats its last one: the cache the passes left is read
    steps.append({"entries": [{"id": rid, "tokens": [reqs[rid][-1]], "want": [0]} for rid in reqs], "end": list(reqs)})
    got = replay(d, dtype, steps, max_tokens=320, vocab=V, extra_args=("--chunk-tokens", "48"))
    want_rows = np.concatenate([ref[rid][wants[rid]] for rid in reqs])
    assert_close(got[0], want_rows, dtype, "several passes")
    longer = {rid: oracle(c, tensors, reqs[rid] + [reqs[rid][-1]], dtype)[-1] for rid in reqs}
    assert_close(got[1], np.stack([longer[rid] for rid in reqs]), dtype, "the token after several passes")
    if dtype == "float32":            # and the same bits as in one pass
        one = replay(d, dtype, steps, max_tokens=320, vocab=V)
        assert np.abs(one[0] - got[0]).max() < 2e-6


@pytest.mark.parametrize("name,cfg,seed,wdtype", [CASES[1], CASES[2]])
@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_in_unequal_pieces_beside_a_decoding_batch_mate(name, cfg, seed, wdtype, dtype):
    """One request is fed as 70 + 20 + 1 + 37 tokens onto its growing cached prefix while its batch mate,
    after a 30-token prompt, decodes one token per step (the reference's resumed prefill:
    src/model/compat_tests.rs:321-338)."""
    d, c, tensors = make_model(cfg, seed, wdtype, std_scale=SHARP)
    V = cfg["vocab_size"]
    reqs = requests_for(cfg, seed + 30, [128, 33])
    ref = {rid: oracle(c, tensors, ids, dtype) for rid, ids in reqs.items()}
    cuts_x, cuts_y = [0, 70, 90, 91, 128], [0, 30, 31, 32, 33]
    steps, index = [], []
    for k in range(4):
        x0, x1, y0, y1 = cuts_x[k], cuts_x[k + 1], cuts_y[k], cuts_y[k + 1]
        wx = sorted({0, (x1 - x0) // 2, x1 - x0 - 1})
        steps.append({"entries": [{"id": "r0", "tokens": reqs["r0"][x0:x1], "want": wx},
                                  {"id": "r1", "tokens": reqs["r1"][y0:y1], "want": [y1 - y0 - 1]}],
                      "end": ["r0", "r1"] if k == 3 else []})
        index.append([("r0", x0 + w) for w in wx] + [("r1", y1 - 1)])
    got = replay(d, dtype, steps, max_tokens=192, vocab=V)
    check_rows(got, index, ref, dtype, "pieces")


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_across_the_1024_bucket(dtype):
    """A request of 1,100 tokens whose prompt ends at 1,000 decodes its next 100 tokens one by one: the
    decode attention goes from one block per (sequence, kv head) to keys split over blocks with a merge
    at 1,024 positions.  A short batch mate keeps the batch unequal."""
    cfg = TINY_D
    d, c, tensors = make_model(cfg, 3, torch.bfloat16, std_scale=SHARP)
    V = cfg["vocab_size"]
    reqs = requests_for(cfg, 40, [1100, 120])
    ref = {rid: oracle(c, tensors, ids, dtype) for rid, ids in reqs.items()}
    head = {"r0": 1000, "r1": 20}
    steps = [{"entries": [{"id": rid, "tokens": reqs[rid][:head[rid]], "want": [0, head[rid] - 1]} for rid in reqs], "end": []}]
    index = [[(rid, p) for rid in reqs for p in (0, head[rid] - 1)]]
    for j in range(100):
        steps.append({"entries": [{"id": rid, "tokens": [reqs[rid][head[rid] + j]], "want": [0]} for rid in reqs],
                      "end": list(reqs) if j == 99 else []})
        index.append([(rid, head[rid] + j) for rid in reqs])
    got = replay(d, dtype, steps, max_tokens=1152 + 128, vocab=V, extra_args=("--poison-unused",))
    check_rows(got, index, ref, dtype, "across 1,024")


@pytest.mark.parametrize("n_requests", [48, 100, 140])
@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_of_many_sequences(dtype, n_requests):
    """48, 100 and 140 short requests with 8 kv heads: sequences x kv heads = 384 is at least twice the number of
    multiprocessors, where the decode attention takes blocks of fewer warps without a split; 800 is more than five
    times (blocks of one warp); with 140 the step has more than 128 tokens (other kernels for the products)."""
    cfg = TINY_D
    d, c, tensors = make_model(cfg, 3, torch.bfloat16, std_scale=SHARP)
    V = cfg["vocab_size"]
    g = torch.Generator().manual_seed(50)
    lengths = torch.randint(8, 70, (n_requests,), generator=g).tolist()
    reqs = requests_for(cfg, 51, lengths)
    ref = {rid: oracle(c, tensors, ids, dtype) for rid, ids in reqs.items()}
    steps = [{"entries": [{"id": rid, "tokens": ids[:-6], "want": [len(ids) - 7]} for rid, ids in reqs.items()], "end": []}]
    index = [[(rid, len(ids) - 7) for rid, ids in reqs.items()]]
    for j in range(6, 0, -1):
        steps.append({"entries": [{"id": rid, "tokens": [ids[-j]], "want": [0]} for rid, ids in reqs.items()],
                      "end": list(reqs) if j == 1 else []})
        index.append([(rid, len(ids) - j) for rid, ids in reqs.items()])
    got = replay(d, dtype, steps, max_tokens=n_requests * 128, vocab=V, extra_args=("--poison-unused",))
    check_rows(got, index, ref, dtype, f"{n_requests} sequences")


def test_first_tokens_and_long_decoding():
    """One token prompts, then every token decoded; 250 steps deep."""
    d, c, tensors = make_model(TINY_B, 5, torch.float32, std_scale=SHARP)
    V = TINY_B["vocab_size"]
    reqs = requests_for(TINY_B, 9, [250, 1, 2])
    steps, index = [], []
    live = list(reqs)
    pos = {rid: 0 for rid in reqs}
    while live:
        steps.append({"entries": [{"id": rid, "tokens": [reqs[rid][pos[rid]]], "want": [0]} for rid in live],
                      "end": [rid for rid in live if pos[rid] + 1 == len(reqs[rid])]})
        index.append([(rid, pos[rid]) for rid in live])
        for rid in live:
            pos[rid] += 1
        live = [rid for rid in live if pos[rid] < len(reqs[rid])]
    for dtype in DTYPES:
        ref = {rid: oracle(c, tensors, ids, dtype) for rid, ids in reqs.items()}
        got = replay(d, dtype, steps, max_tokens=384, vocab=V)
        check_rows(got, index, ref, dtype, "long decoding")


def test_padding_and_batch_mates_change_nothing():
    """A request's float32 logits are the same alone and next to longer and shorter ones."""
    d, c, tensors = make_model(TINY_C, 3, torch.float32, std_scale=SHARP)
    V = TINY_C["vocab_size"]
    reqs = requests_for(TINY_C, 4, [50, 3, 111])
    alone = replay(d, "float32", [{"entries": [{"id": "x", "tokens": reqs["r0"], "want": [49]}], "end": ["x"]}],
                   max_tokens=64, vocab=V)[0]
    together = replay(d, "float32", [{"entries": [{"id": rid, "tokens": ids, "want": [len(ids) - 1]}
                                                   for rid, ids in reqs.items()], "end": list(reqs)}],
                      max_tokens=256, vocab=V)[0]
    assert np.abs(alone[0] - together[0]).max() < 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_heads_wider_than_the_fast_attention_takes(dtype):
    """head_dim 160 (a multiple of 16 beyond the tensor-core attention's 128): the engine takes the plain
    attention kernel for it, in bfloat16 too; whole prompts, then tokens one by one, two unequal requests."""
    d, c, tensors = make_model(TINY_E, 6, torch.bfloat16, std_scale=SHARP)
    V = TINY_E["vocab_size"]
    reqs = requests_for(TINY_E, 60, [90, 41])
    ref = {rid: oracle(c, tensors, ids, dtype) for rid, ids in reqs.items()}
    head = {"r0": 70, "r1": 21}
    steps = [{"entries": [{"id": rid, "tokens": reqs[rid][:head[rid]], "want": list(range(head[rid]))} for rid in reqs], "end": []}]
    index = [[(rid, p) for rid in reqs for p in range(head[rid])]]
    for j in range(20):
        steps.append({"entries": [{"id": rid, "tokens": [reqs[rid][head[rid] + j]], "want": [0]} for rid in reqs],
                      "end": list(reqs) if j == 19 else []})
        index.append([(rid, head[rid] + j) for rid in reqs])
    got = replay(d, dtype, steps, max_tokens=256, vocab=V, extra_args=("--poison-unused",))
    check_rows(got, index, ref, dtype, "wide heads")
