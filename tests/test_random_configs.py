"""Random tiny configurations of the architecture through the engine against the plain implementation: head sizes
16 to 128 in steps of 16, 1 to 5 kv heads, groups of 1 to 8, widths and vocabularies that are no power of two,
1 to 3 layers, both rotary layouts, with and without llama3 scaling and tied embeddings, whole prompts (in passes of
64 for some) and then single tokens, NaN in the cache rows nobody owns.  Ninety such configurations were run once by
hand (largest bfloat16 error 0.028 and 1.1 % of a row's deviation, float32 5e-6); this is the short form."""
import random

import numpy as np
import pytest
import torch

from plain_llama import plain_forward
from replay_util import assert_close
from tiny import SHARP, make_model

pytestmark = pytest.mark.gpu


def random_config(rnd):
    kv = rnd.choice([1, 2, 3, 4, 5])
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=rnd.choice([1, 2, 3]),
               hidden_size=rnd.choice([40, 72, 96, 100, 136, 200, 264]), num_attention_heads=kv * rnd.choice([1, 2, 3, 4, 5, 8]),
               num_key_value_heads=kv, head_dim=rnd.choice([16, 32, 48, 64, 80, 96, 112, 128]),
               intermediate_size=rnd.choice([56, 104, 176, 200, 330]), vocab_size=rnd.randint(90, 700),
               rope_theta=rnd.choice([10000.0, 500000.0]), rms_norm_eps=rnd.choice([1e-5, 1e-6, 3e-6]),
               tie_word_embeddings=rnd.random() < 0.5, max_position_embeddings=256,
               rope_layout=rnd.choice(["interleaved", "split_half"]))
    cfg["rope_scaling"] = (dict(rope_type="llama3", factor=rnd.choice([2.0, 8.0]), low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=64) if rnd.random() < 0.5 else None)
    return cfg


@pytest.mark.parametrize("seed", range(100, 112))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration(seed, dtype):
    from mdma_b200.engine import Engine, StepEntry
    rnd = random.Random(seed)
    cfg = random_config(rnd)
    # wide models get smaller weights, so that logits stay of the size the tolerances were measured at
    scale = SHARP * min(1.0, (96.0 / cfg["hidden_size"]) ** 0.5)
    d, c, tensors = make_model(cfg, seed, torch.bfloat16 if dtype == "bfloat16" else torch.float32, std_scale=scale)
    held = {k: v.float() for k, v in tensors.items()}
    eng = Engine(d, dtype=dtype, max_batch=3, max_context=256, logit_rows=64, chunk_tokens=rnd.choice([8192, 64]))
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randint(0, cfg["vocab_size"], (rnd.randint(8, 150),), generator=g).tolist() for _ in range(rnd.randint(1, 3))]
    ref = [plain_forward(c, held, s, torch.float64).numpy() for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    cut = [len(s) - 6 for s in seqs]
    what = {k: cfg[k] for k in ("head_dim", "num_key_value_heads", "num_attention_heads", "hidden_size", "intermediate_size")}
    eng.cache.poison_unused()
    wants = [sorted({0, n // 2, n - 1}) for n in cut]
    out = eng.step([StepEntry(sl, s[:n], w) for sl, s, n, w in zip(slots, seqs, cut, wants)]).double().cpu().numpy()
    assert_close(out, np.stack([ref[i][p] for i, w in enumerate(wants) for p in w]), dtype, f"prompts, {what}")
    for step in range(6):
        eng.cache.poison_unused()
        out = eng.step([StepEntry(sl, [s[n + step]], [0]) for sl, s, n in zip(slots, seqs, cut)]).double().cpu().numpy()
        assert_close(out, np.stack([ref[i][n + step] for i, n in enumerate(cut)]), dtype, f"token {step}, {what}")
    eng.check_status()
    eng.cache.check()
