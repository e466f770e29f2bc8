"""The plain implementation itself, and the stored outputs that pin it (no GPU)."""
import json
import math
import os

import pytest
import torch

from plain_llama import (plain_argmax, plain_attention, plain_forward, plain_generate, plain_inv_freq,
                         plain_rmsnorm, plain_rope, plain_sample, plain_swiglu)
from tiny import TINY_A, TINY_B, make_model

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "plain_tiny.json")


def test_rmsnorm_formula():
    x = torch.tensor([[3.0, 4.0]])
    y = plain_rmsnorm(x, torch.tensor([2.0, 0.5]), 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]]))


def test_rope_layouts_agree_up_to_a_permutation():
    torch.manual_seed(0)
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    f = plain_inv_freq(8, 10000.0, None)
    pos = torch.tensor([0, 1, 7, 30, 100])
    inter = plain_rope(x, pos, f, "interleaved")
    perm = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7])               # interleaved -> split-half order
    split = plain_rope(x[..., perm], pos, f, "split_half")
    assert torch.allclose(inter[..., perm], split)
    assert torch.allclose(plain_rope(x, torch.zeros(5, dtype=torch.long), f, "split_half"), x)   # position 0
    assert torch.allclose(inter.norm(dim=-1), x.norm(dim=-1))   # a rotation


def test_llama3_frequency_bands():
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=64)
    base = plain_inv_freq(32, 500000.0, None).double()
    scaled = plain_inv_freq(32, 500000.0, sc).double()
    wl = 2 * math.pi / base
    assert torch.allclose(scaled[wl < 16], base[wl < 16])                    # short waves kept
    assert torch.allclose(scaled[wl > 64], base[wl > 64] / 8.0, rtol=1e-6)   # long waves slowed
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and torch.all(scaled[mid] <= base[mid]) and torch.all(scaled[mid] >= base[mid] / 8.0)


def test_attention_is_causal_and_windowed():
    torch.manual_seed(1)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    full = plain_attention(q, k, v, 0.35)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0                                   # the future must not matter
    assert torch.allclose(plain_attention(q, k2, v2, 0.35)[:4], full[:4])
    assert torch.allclose(full[0].reshape(4, 8), v[0].repeat_interleave(2, dim=0))   # one key: its value
    win = plain_attention(q, k, v, 0.35, window=2)
    k3, v3 = k.clone(), v.clone()
    k3[:3], v3[:3] = 5.0, 5.0                                    # outside the window of query 5
    assert torch.allclose(plain_attention(q, k3, v3, 0.35, window=2)[5], win[5])


def test_swiglu_formula():
    g, u = torch.tensor([0.0, 2.0]), torch.tensor([3.0, 3.0])
    assert torch.allclose(plain_swiglu(g, u), torch.tensor([0.0, 2.0 / (1 + math.exp(-2.0)) * 3.0]))


def test_sampler_rules():
    logits = [0.0, 3.0, 3.0, -1.0]
    assert plain_argmax(logits) == 1                             # ties: the lowest index
    assert plain_sample(logits, [], 0.3, temperature=0.0) == 1
    assert plain_sample(logits, [1], 0.3, temperature=0.0, repetition_penalty=2.0) == 2   # penalty flips greedy
    assert plain_sample([-2.0, -1.0], [1], 0.3, 0.0, repetition_penalty=3.0) == 0          # negative: multiplied
    # min-p and top-p collapse to the best token
    assert plain_sample([5.0, 1.0, 0.0], [], 0.99, temperature=1.0, min_p=0.5) == 0
    assert plain_sample([5.0, 1.0, 0.0], [], 0.99, temperature=1.0, top_p=0.5) == 0
    # categorical over the descending order: u picks by cumulative mass
    p = torch.softmax(torch.tensor([1.0, 2.0, 0.5]), 0)
    assert plain_sample([1.0, 2.0, 0.5], [], float(p[1]) * 0.5, 1.0) == 1
    assert plain_sample([1.0, 2.0, 0.5], [], float(p[1]) + 1e-3, 1.0) == 0
    assert plain_sample([1.0, 2.0, 0.5], [], 0.9999, 1.0) == 2


def test_golden_outputs_still_hold():
    gold = json.load(open(GOLDEN))
    for name, cfg, seed in (("tiny_a", TINY_A, 0), ("tiny_b", TINY_B, 1)):
        _, c, tensors = make_model(cfg, seed, torch.float32)
        ids = gold[name]["ids"]
        logits = plain_forward(c, tensors, ids, torch.float64)
        want = torch.tensor(gold[name]["last_logits_first8"], dtype=torch.float64)
        assert torch.allclose(logits[-1, :8], want, atol=1e-9), name
        assert plain_generate(c, tensors, ids, 6) == gold[name]["greedy6"]


def test_float32_and_float64_agree():
    _, c, tensors = make_model(TINY_B, 1, torch.float32)
    ids = list(range(3, 40))
    a = plain_forward(c, tensors, ids, torch.float32).double()
    b = plain_forward(c, tensors, ids, torch.float64)
    assert (a - b).abs().max() < 2e-5


def test_the_two_plain_implementations_agree():
    """tests/plain_llama.py (PyTorch) and tests/plain_ref.cpp (C++ scalar loops, rotation as a complex
    product, llama3 scaling stated on frequencies) were written separately from the formulas; they must
    give the same logits at every place, for every shape and option of the tiny configurations."""
    from plain_llama import plain_inv_freq
    from plain_ref import ref_forward, ref_inv_freq
    from tiny import SHARP, TINY_C, TINY_D
    for cfg, seed in ((TINY_A, 0), (TINY_B, 1), (TINY_C, 2), (TINY_D, 3), (dict(TINY_A, rope_layout="split_half"), 4),
                      (dict(TINY_B, rope_layout="interleaved", tie_word_embeddings=False), 5)):
        _, c, tensors = make_model(cfg, seed, torch.float32, std_scale=SHARP)
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, cfg["vocab_size"], (61,), generator=g).tolist()
        a = plain_forward(c, tensors, ids, torch.float64)
        b = ref_forward(c, tensors, ids)
        assert (a - b).abs().max() < 1e-12, cfg
        D = c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"]
        fa = plain_inv_freq(D, c.get("rope_theta", 10000.0), c.get("rope_scaling"))
        fb = ref_inv_freq(D, c.get("rope_theta", 10000.0), c.get("rope_scaling"))
        assert torch.equal(fa.double(), fb)


def test_llama3_table_by_hand():
    """The scaled table at values worked out by hand: theta 16, head 8, L = 64, factor 8, low 1, high 4.
    f = 1, 1/2, 1/4, 1/8; wavelengths 6.28, 12.6, 25.1, 50.3.  L/high = 16, L/low = 64: the first two
    stay, the last two lie in the band: smooth = (64/25.13 - 1)/3 = 0.5155 and (64/50.27 - 1)/3 = 0.0911."""
    from plain_llama import plain_inv_freq
    f = plain_inv_freq(8, 16.0, dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                     original_max_position_embeddings=64)).double()
    two_pi = 2 * math.pi
    s2, s3 = (64 / (two_pi * 4) - 1) / 3, (64 / (two_pi * 8) - 1) / 3
    want = [1.0, 0.5, (1 - s2) * 0.25 / 8 + s2 * 0.25, (1 - s3) * 0.125 / 8 + s3 * 0.125]
    assert torch.allclose(f, torch.tensor(want, dtype=torch.float64), rtol=1e-6)
    # beyond the band everything is divided by the factor
    f = plain_inv_freq(8, 16.0, dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                     original_max_position_embeddings=4)).double()
    assert torch.allclose(f, torch.tensor([1.0, 0.5, 0.25, 0.125], dtype=torch.float64) / 8, rtol=1e-6)


def test_the_oracle_tells_a_wrong_cache_row_from_rounding():
    """With the tests' weights, changing ONE token anywhere among the first 96 of 97 moves some later
    row of logits by far more than the bfloat16 tolerances of tests/replay_util.py (0.05 absolute, 2 % of
    a row's deviation): at least 5 times for the least influential token of any shape, and 10 times for
    the median token.  So a stale, missing or misplaced cache row cannot hide under the tolerance."""
    from replay_util import TOL_BF16_ABS, TOL_BF16_ROW
    from tiny import SHARP, TINY_C, TINY_D
    for cfg, seed, wd in ((TINY_A, 0, torch.float32), (TINY_B, 1, torch.bfloat16), (TINY_C, 2, torch.bfloat16),
                          (TINY_D, 3, torch.bfloat16)):
        _, c, tensors = make_model(cfg, seed, wd, std_scale=SHARP)
        W = {k: v.float() for k, v in tensors.items()}
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, cfg["vocab_size"], (97,), generator=g).tolist()
        base = plain_forward(c, W, ids, torch.float64)
        moved_abs, moved_row = [], []
        for j in range(0, 96, 5):
            other = list(ids)
            other[j] = (other[j] + 1) % cfg["vocab_size"]
            delta = plain_forward(c, W, other, torch.float64)[j + 1:] - base[j + 1:]
            moved_abs.append(delta.abs().max().item())
            moved_row.append((delta.pow(2).mean(1).sqrt() / base[j + 1:].std(1)).max().item())
        assert min(moved_abs) >= 5 * TOL_BF16_ABS and min(moved_row) >= 5 * TOL_BF16_ROW, (cfg, min(moved_abs), min(moved_row))
        assert sorted(moved_abs)[len(moved_abs) // 2] >= 10 * TOL_BF16_ABS
