"""Random schedules through `Engine.step` against the plain implementation: unequal batches, prompts whole or
cut in random pieces on their cached prefix, single tokens, requests that end earlier, slots and pages used
again, wanted places in any order, passes of 48 or 100 tokens, cache pages of 16 to 128 rows, NaN in the cache rows
that belong to nobody.
A longer run of the same generator (13,000 steps) was made once by hand; this is its short form."""
import random

import numpy as np
import pytest
import torch

from plain_llama import plain_forward
from replay_util import assert_close
from tiny import SHARP, TINY_A, TINY_B, TINY_C, TINY_D, make_model

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,cfg,seed,wdtype", [("d", TINY_D, 3, torch.bfloat16), ("b", TINY_B, 1, torch.bfloat16),
                                                  ("c", TINY_C, 2, torch.bfloat16), ("a", TINY_A, 0, torch.float32)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_schedules(name, cfg, seed, wdtype, dtype):
    from mdma_b200.engine import Engine, StepEntry
    rnd = random.Random(seed * 7 + len(dtype))
    d, c, tensors = make_model(cfg, seed, wdtype, std_scale=SHARP)
    held = {k: (v.bfloat16().float() if dtype == "bfloat16" and v.dim() == 2 else v.float()) for k, v in tensors.items()}
    ctx = min(cfg["max_position_embeddings"], 260)
    for trial in range(3):
        chunk = (8192, 48, 100)[(trial + seed) % 3]
        # pages of 64 rows as everywhere, and once of 16, 32 or 128 (other tile loads, other kernels for some steps)
        page = 64 if trial < 2 else (16, 32, 128, 32)[seed % 4]
        eng = Engine(d, dtype=dtype, max_batch=5, max_context=ctx, max_tokens=5 * 384, chunk_tokens=chunk, logit_rows=64,
                     page_size=page)
        g = torch.Generator().manual_seed(rnd.randrange(10 ** 6))
        for _batch in range(3):
            n = rnd.randint(1, 5)
            seqs = [torch.randint(0, cfg["vocab_size"], (rnd.choice([1, 3, 33, 64, 65, 97, 130, ctx - 1, ctx]),),
                                  generator=g).tolist()[:ctx] for _ in range(n)]
            ref = [plain_forward(c, held, s, torch.float64).numpy() for s in seqs]
            slots = [eng.acquire() for _ in seqs]
            pos, live = [0] * n, list(range(n))
            while live:
                mode = rnd.random()          # whole prompts, single tokens, or pieces of random length
                entries, places = [], []
                for i in live:
                    left = len(seqs[i]) - pos[i]
                    take = left if (pos[i] == 0 and mode < 0.3) else (1 if mode < 0.7 else rnd.randint(1, left))
                    want = rnd.sample(range(take), min(take, rnd.choice([0, 1, 1, 2, 3])))
                    entries.append(StepEntry(slots[i], seqs[i][pos[i]:pos[i] + take], want))
                    places += [(i, pos[i] + w) for w in want]
                    pos[i] += take
                if rnd.random() < 0.5:
                    eng.cache.poison_unused()
                out = eng.step(entries).double().cpu().numpy()
                if places:
                    assert_close(out, np.stack([ref[i][p] for i, p in places]), dtype, f"pass size {chunk}, places {places[:4]}")
                for i in list(live):
                    if pos[i] == len(seqs[i]):
                        eng.release(slots[i])
                        live.remove(i)
            eng.cache.check()
            assert not eng.cache.lengths
        eng.check_status()
        del eng
