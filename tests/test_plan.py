"""The product planner (host code of the tensor-core library, callable without a GPU): whatever it chooses for a
step of up to `chunk` tokens fits the scratch an engine reserves for that chunk size from sizes alone, at the
benchmark's layer shapes, a small model's and odd ones; and a few of the choices that the measurements in
`profiles/` rest on."""
import pytest

from mdma_b200 import ops_tensor

STORE, ACCUMULATE, GATED = 0, 1, 2
SHAPES = {          # name -> [(mode, features, K)]
    "8b": [(STORE, 6144, 4096), (ACCUMULATE, 4096, 4096), (GATED, 14336, 4096), (ACCUMULATE, 4096, 14336), (STORE, 128256, 4096)],
    "7b": [(STORE, 12288, 4096), (ACCUMULATE, 4096, 4096), (GATED, 11008, 4096), (ACCUMULATE, 4096, 11008), (STORE, 32000, 4096)],
    "1b": [(STORE, 3072, 2048), (ACCUMULATE, 2048, 2048), (GATED, 8192, 2048), (ACCUMULATE, 2048, 8192), (STORE, 128256, 2048)],
    "odd": [(STORE, 520, 264), (ACCUMULATE, 136, 2048), (GATED, 331, 640), (ACCUMULATE, 5000, 72), (STORE, 97, 8)],
}


@pytest.mark.parametrize("sms", [148, 132, 78])
@pytest.mark.parametrize("name", sorted(SHAPES))
def test_every_plan_fits_the_scratch_reserved_for_its_chunk_size(name, sms):
    tokens = list(range(1, 300)) + list(range(300, 1200, 7)) + [2048, 4096, 8191, 8192]
    for m in tokens:
        bound = ops_tensor.scratch_floats_bound(sms, m, 1, ())
        for mode, n, k in SHAPES[name]:
            bn, splits = ops_tensor.gemm_plan(mode, m, n, k, sms)
            assert bn in (16, 32, 64, 128, 256, 512) and (splits >= 1 or splits in (-2, -3, -4)), (m, mode, n, k, bn, splits)
            if bn != 512:
                assert bn >= min(m, 256) or m > 128, (m, bn)          # a token tile covers the step, or the step is tiled
            need = ops_tensor.gemm_scratch_floats(bn, splits, m, n, sms)
            assert need <= bound, f"{name}: {m} tokens, mode {mode}, {n} x {k}: plan ({bn}, {splits}) needs {need} floats, {bound} reserved"


def test_choices_that_the_measurements_rest_on():
    plan = lambda mode, m, n, k: ops_tensor.gemm_plan(mode, m, n, k, 148)
    assert plan(STORE, 8, 6144, 4096) == (16, 4)             # QKV at batch 8: four splits (the next kernel adds them up itself)
    assert plan(ACCUMULATE, 8, 4096, 4096) == (16, 9)        # O: two blocks per SM
    assert plan(GATED, 8, 14336, 4096) == (16, -2)           # gate+up: K split inside a cluster of two
    assert plan(GATED, 64, 14336, 4096) == (64, 1)
    assert plan(GATED, 128, 14336, 4096)[0] == 512           # block pairs from 97 tokens
    assert plan(ACCUMULATE, 256, 4096, 14336) == (256, 4)    # down of 256 tokens: one wide token tile, four splits
    assert plan(STORE, 256, 6144, 4096) == (128, 1)          # QKV stays unsplit there (its partial sums cost the rotary kernel more)
    assert plan(GATED, 2048, 14336, 4096) == (512, 1) and plan(STORE, 2048, 6144, 4096) == (512, 1)
    assert plan(STORE, 8, 128256, 4096) == (16, 1)           # the head: more tiles than SMs, no split


@pytest.mark.parametrize("sms", [148, 78])
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(32, 8, 128), (32, 32, 128), (32, 8, 64), (16, 8, 16), (6, 3, 48), (64, 1, 32), (40, 2, 64)])
def test_every_choice_of_key_splits_fits_the_scratch_reserved_for_attention(heads, kv_heads, head_dim, sms):
    """The attention kernels keep tokens x heads x splits x (head_dim + 2) floats when they split the keys; the
    engine reserves a bound computed from sizes alone.  Every (sequences, tokens per sequence, context, capacity)
    the step function can see must stay below it."""
    reserved = (ops_tensor.scratch_floats_bound(sms, 8192, 1, [(heads, kv_heads, head_dim)])
                - ops_tensor.scratch_floats_bound(sms, 8192, 1, ()))
    worst = 0
    for n_seqs in list(range(1, 40)) + [48, 64, 100, 148, 200, 300, 600]:
        for max_new in (1, 2, 5, 16, 17, 64, 129, 700):
            if n_seqs * max_new > 8192:
                continue
            for max_len in (1, 64, 580, 1024, 1025, 4096, 40000):
                if max_len < max_new:
                    continue
                for most in (None, n_seqs, max(n_seqs, 64)):
                    splits = ops_tensor.attention_splits(n_seqs, max_new, max_len, heads, kv_heads, sms, most)
                    assert 1 <= splits <= 32
                    need = n_seqs * max_new * heads * splits * (head_dim + 2) if splits > 1 else 0
                    worst = max(worst, need)
                    assert need <= reserved, (n_seqs, max_new, max_len, most, splits, need, reserved)
    assert worst > 0          # the sweep did reach split cases
