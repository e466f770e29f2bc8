"""Each part alone, built from a PartSpec and fed through a hand-made step context."""
import math

import pytest
import torch

from plain_llama import plain_attention, plain_inv_freq, plain_rmsnorm, plain_rope, plain_swiglu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Ctx:
    """A step context by hand: one or more sequences starting at position 0 in slots 0.."""

    def __init__(self, rt, seq_lens, widths, chunk=256):
        from mdma_b200.engine.step import StepContext
        ws = {n: torch.empty(chunk, c, dtype=torch.float32 if k == "f32" else rt.dtype, device=DEV)
              for n, (c, k) in widths.items()}
        self.ctx = StepContext(rt, ws)
        tok_seq = [s for s, n in enumerate(seq_lens) for _ in range(n)]
        tok_pos = [p for n in seq_lens for p in range(n)]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        c = self.ctx
        c.n_tokens, c.n_seqs = len(tok_seq), len(seq_lens)
        c.tok_seq, c.tok_pos, c.seq_slot = i32(tok_seq), i32(tok_pos), i32(list(range(len(seq_lens))))
        c.max_new, c.max_len = max(seq_lens), max(seq_lens)
        c.host_seq_new, c.host_seq_pos0 = list(seq_lens), [0] * len(seq_lens)
        starts = [0]
        for n in seq_lens:
            starts.append(starts[-1] + n)
        c.seq_start, c.seq_pos0 = i32(starts), i32([0] * len(seq_lens))


def runtime(dtype, kernels="plain"):
    from mdma_b200.parts.base import Runtime
    return Runtime(dtype, torch.device(DEV), gemm="tensor" if kernels == "tensor" else "simt",
                   attention="fast" if kernels == "tensor" else "simple")


def near(got, want, dtype):
    """Error against the output's own scale: float32 to 2e-5 of it, bfloat16 (8-bit
    mantissa, several roundings on the way) to 1.5e-2 of it."""
    got, want = got.double().cpu(), want.double().cpu()
    rel = 2e-5 if dtype == torch.float32 else 1.5e-2
    err = (got - want).abs().max().item()
    assert err <= rel * want.abs().max().item(), f"max err {err:.3g} at output scale {want.abs().max().item():.3g}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from mdma_b200.registry import NORMS
    from mdma_b200.spec import PartSpec
    part = NORMS.get("rmsnorm")(PartSpec("rmsnorm", dict(width=200, eps=2e-5), prefix="n."))
    assert {k: v.shape for k, v in part.tensor_specs().items()} == {"weight": (200,)}
    w = torch.rand(200, device=DEV) + 0.5
    rt = runtime(dtype)
    part.bind({"weight": w}, rt)
    c = Ctx(rt, [7], {})
    x = torch.randn(7, 200, device=DEV)
    out = torch.empty(7, 200, device=DEV, dtype=dtype)
    part.forward(c.ctx, x, out)
    near(out, plain_rmsnorm(x.double().cpu(), w.double().cpu(), 2e-5), dtype)


@pytest.mark.parametrize("dtype,kernels", [(torch.float32, "plain"), (torch.bfloat16, "plain"), (torch.bfloat16, "tensor")])
def test_gated_mlp_part(dtype, kernels):
    from mdma_b200.registry import FEED_FORWARDS
    from mdma_b200.spec import PartSpec
    E, F = 72, 200
    part = FEED_FORWARDS.get("gated_mlp")(PartSpec("gated_mlp", dict(hidden_size=E, intermediate_size=F), prefix="m."))
    assert {k: v.shape for k, v in part.tensor_specs().items()} == {
        "gate_proj.weight": (F, E), "up_proj.weight": (F, E), "down_proj.weight": (E, F)}
    torch.manual_seed(0)
    t = {k: (torch.randn(v.shape, device=DEV) * 0.1).to(dtype) for k, v in part.tensor_specs().items()}
    rt = runtime(dtype, kernels)
    part.bind(t, rt)
    c = Ctx(rt, [5, 3], part.workspace())
    h = torch.randn(8, E, device=DEV).to(dtype)
    x = torch.randn(8, E, device=DEV)
    x0 = x.clone()
    part.forward(c.ctx, h, x)
    hd = h.double().cpu()
    W = {k: v.double().cpu() for k, v in t.items()}
    want = x0.double().cpu() + plain_swiglu(hd @ W["gate_proj.weight"].t(), hd @ W["up_proj.weight"].t()) @ W["down_proj.weight"].t()
    near(x, want, dtype)


@pytest.mark.parametrize("dtype,kernels", [(torch.float32, "plain"), (torch.bfloat16, "plain"), (torch.bfloat16, "tensor")])
@pytest.mark.parametrize("H,K,hd,window,layout", [(6, 2, 48, 0, "split_half"), (4, 1, 32, 9, "interleaved")])
def test_attention_part(dtype, kernels, H, K, hd, window, layout):
    """Two sequences of unequal length in one step, through the part's own cache view."""
    from mdma_b200.cache import SequenceCache
    from mdma_b200.registry import MIXERS
    from mdma_b200.spec import PartSpec
    E = 88
    pos = PartSpec("rotary", dict(head_dim=hd, rotary_dim=hd, theta=30000.0, layout=layout, scaling=None))
    scale = 0.9 / math.sqrt(hd)
    part = MIXERS.get("attention")(PartSpec("attention", dict(hidden_size=E, num_heads=H, num_kv_heads=K,
                                                               head_dim=hd, scale=scale, window=window,
                                                               position=pos), prefix="a."))
    torch.manual_seed(1)
    t = {k: (torch.randn(v.shape, device=DEV) * 0.15).to(dtype) for k, v in part.tensor_specs().items()}
    rt = runtime(dtype, kernels)
    part.bind(t, rt)
    lens = [37, 12]
    cache = SequenceCache([part.kv_need()], [part.state_need()], 64 * 4, 2, 128, dtype, torch.device(DEV), 64)
    slots = [cache.acquire(), cache.acquire()]
    cache.extend(dict(zip(slots, lens)))
    c = Ctx(rt, lens, part.workspace())
    h = torch.randn(sum(lens), E, device=DEV).to(dtype)
    x = torch.zeros(sum(lens), E, device=DEV)
    part.forward(c.ctx, h, x, cache.view(0), True)
    W = {k: v.double().cpu() for k, v in t.items()}
    inv = plain_inv_freq(hd, 30000.0, None)
    off = 0
    for n in lens:
        hs = h[off:off + n].double().cpu()
        q = plain_rope((hs @ W["q_proj.weight"].t()).reshape(n, H, hd), torch.arange(n), inv, layout)
        k = plain_rope((hs @ W["k_proj.weight"].t()).reshape(n, K, hd), torch.arange(n), inv, layout)
        v = (hs @ W["v_proj.weight"].t()).reshape(n, K, hd)
        want = plain_attention(q, k, v, scale, window) @ W["o_proj.weight"].t()
        near(x[off:off + n], want, dtype)
        off += n


def test_rotary_part_table():
    from mdma_b200.config.llama import RopeScaling
    from mdma_b200.parts.rotary import inverse_frequencies
    sc = RopeScaling("llama3", 8.0, 1.0, 4.0, 64)
    got = inverse_frequencies(32, 500000.0, sc)
    want = plain_inv_freq(32, 500000.0, dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                             high_freq_factor=4.0, original_max_position_embeddings=64))
    assert torch.equal(got, want)
    assert torch.equal(inverse_frequencies(48, 1e4, None), plain_inv_freq(48, 1e4, None))


def test_embedding_and_head_parts():
    from mdma_b200.registry import EMBEDDINGS, HEADS
    from mdma_b200.spec import PartSpec
    V, E = 331, 40
    emb = EMBEDDINGS.get("embedding")(PartSpec("embedding", dict(vocab_size=V, width=E), prefix="e."))
    head = HEADS.get("lm_head")(PartSpec("lm_head", dict(vocab_size=V, width=E), prefix="h."))
    w = torch.randn(V, E, device=DEV)
    rt = runtime(torch.float32)
    emb.bind({"weight": w}, rt)
    head.bind({"weight": w}, rt)
    c = Ctx(rt, [4], {})
    ids = torch.tensor([3, 330, 0, 3], dtype=torch.int32, device=DEV)
    x = torch.empty(4, E, device=DEV)
    emb.forward(c.ctx, ids, x)
    assert torch.equal(x, w[ids.long()])
    logits = torch.empty(4, V, device=DEV)
    head.forward(c.ctx, x, logits, 4)
    assert torch.allclose(logits.double().cpu(), (x.double() @ w.double().t()).cpu(), atol=1e-4)
