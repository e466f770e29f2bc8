"""Trace replay against the plain implementation: whole requests, the last 32
tokens one by one, and batches of unequal lengths whose slots are used again;
in 32-bit and in bfloat16."""
import numpy as np
import pytest
import torch

from plain_llama import plain_forward
from replay_util import replay
from tiny import TINY_A, TINY_B, TINY_C, make_model

pytestmark = pytest.mark.gpu

# (absolute tolerance on logits, per engine dtype); logits are O(1)
TOL = {"float32": 2e-5, "bfloat16": 4e-2}
CASES = [("a", TINY_A, 0, torch.float32), ("b", TINY_B, 1, torch.bfloat16), ("c", TINY_C, 2, torch.bfloat16)]


def requests_for(cfg, seed, lengths):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
            for i, n in enumerate(lengths)}


def oracle(c, tensors, ids):
    return plain_forward(c, {k: v.float() for k, v in tensors.items()}, ids, torch.float64).numpy()


@pytest.mark.parametrize("name,cfg,seed,wdtype", CASES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_three_ways(name, cfg, seed, wdtype, dtype):
    d, c, tensors = make_model(cfg, seed, wdtype)
    V = cfg["vocab_size"]
    lengths = [40, 97, 33, 70, 64, 128][: 6 if cfg["max_position_embeddings"] >= 128 else 4]
    reqs = requests_for(cfg, seed, lengths)
    ref = {rid: oracle(c, tensors, ids) for rid, ids in reqs.items()}
    tol = TOL[dtype]

    # 1. each request alone and whole: one step, logits at every place
    steps = [{"entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
             for rid, ids in reqs.items()]
    got = replay(d, dtype, steps, max_tokens=128, vocab=V)
    whole = {}
    for i, rid in enumerate(reqs):
        whole[rid] = got[i]
        err = np.abs(got[i] - ref[rid]).max()
        assert err < tol, f"whole {rid}: {err}"

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
        err = np.abs(got[i] - ref[rid][lo:hi]).max()
        assert err < tol, f"one-by-one {rid} places {lo}..{hi}: {err}"
        if dtype == "float32":        # the same arithmetic whatever the cut
            assert np.abs(got[i] - whole[rid][lo:hi]).max() < 2e-6

    # 3. batches of unequal lengths; shorter requests end earlier; one batch after another
    rids = list(reqs)
    steps, index = [], []
    for batch in (rids[:3], rids[3:], rids[:2][::-1]):
        prompt = {rid: max(1, len(reqs[rid]) // 3) for rid in batch}
        steps.append({"entries": [{"id": rid, "tokens": reqs[rid][:prompt[rid]],
                                   "want": [0, prompt[rid] - 1]} for rid in batch], "end": []})
        index.append([(rid, p) for rid in batch for p in (0, prompt[rid] - 1)])
        pos = dict(prompt)
        live = list(batch)
        while live:
            entries = [{"id": rid, "tokens": [reqs[rid][pos[rid]]], "want": [0]} for rid in live]
            for rid in live:
                pos[rid] += 1
            ended = [rid for rid in live if pos[rid] == len(reqs[rid])]
            steps.append({"entries": entries, "end": ended})
            index.append([(rid, pos[rid] - 1) for rid in live])
            live = [rid for rid in live if rid not in ended]
    # the cache holds just the largest batch: slots and pages must be used again
    need = max(sum(-(-len(reqs[r]) // 64) * 64 for r in b) for b in (rids[:3], rids[3:], rids[:2]))
    got = replay(d, dtype, steps, max_tokens=need, vocab=V)
    for i, places in enumerate(index):
        for row, (rid, p) in enumerate(places):
            err = np.abs(got[i][row] - ref[rid][p]).max()
            assert err < tol, f"batched {rid} place {p} (step {i}): {err}"


def test_first_tokens_and_long_decoding():
    """One token prompts, then every token decoded; 250 steps deep."""
    d, c, tensors = make_model(TINY_B, 5, torch.float32)
    V = TINY_B["vocab_size"]
    reqs = requests_for(TINY_B, 9, [250, 1, 2])
    ref = {rid: oracle(c, tensors, ids) for rid, ids in reqs.items()}
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
    for dtype in ("float32", "bfloat16"):
        got = replay(d, dtype, steps, max_tokens=384, vocab=V)
        for i, places in enumerate(index):
            for row, (rid, p) in enumerate(places):
                assert np.abs(got[i][row] - ref[rid][p]).max() < TOL[dtype], (dtype, rid, p)


def test_padding_and_batch_mates_change_nothing():
    """A request's float32 logits are the same alone and next to longer and shorter ones."""
    d, c, tensors = make_model(TINY_C, 3, torch.float32)
    V = TINY_C["vocab_size"]
    reqs = requests_for(TINY_C, 4, [50, 3, 111])
    alone = replay(d, "float32", [{"entries": [{"id": "x", "tokens": reqs["r0"], "want": [49]}], "end": ["x"]}],
                   max_tokens=64, vocab=V)[0]
    together = replay(d, "float32", [{"entries": [{"id": rid, "tokens": ids, "want": [len(ids) - 1]}
                                                   for rid, ids in reqs.items()], "end": list(reqs)}],
                      max_tokens=256, vocab=V)[0]
    assert np.abs(alone[0] - together[0]).max() < 2e-6
