"""Generality of the parts: a toy mixer with state of its own, a toy
architecture that mixes it with attention layers, runs one layer twice and lets
one layer read another's cache — all defined here, registered, built from a
model folder and stepped, without touching the framework's files."""
import json
import math
import os

import numpy as np
import pytest
import torch

from plain_llama import plain_attention, plain_inv_freq, plain_rmsnorm, plain_rope, plain_swiglu
from tiny import jitter_norm_weights

pytestmark = pytest.mark.gpu

E, H, K, D, F, V = 48, 4, 2, 16, 72, 97


def register_toy():
    from mdma_b200.cache import StateNeed
    from mdma_b200.config import Architecture
    from mdma_b200.parts.base import Part
    from mdma_b200.registry import ARCHITECTURES, MIXERS
    from mdma_b200.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

    class DecayMixer(Part):
        """s <- decay * s + W_in h_t;  x_t += W_out s.  The state s is per sequence, fixed size."""

        def __init__(self, spec):
            super().__init__(spec)
            self.width, self.inner, self.decay = spec.params["width"], spec.params["inner"], spec.params["decay"]

        def tensor_specs(self):
            return {"in.weight": TensorSpec((self.inner, self.width)), "out.weight": TensorSpec((self.width, self.inner))}

        def kv_need(self):
            return None

        def state_need(self):
            return StateNeed((self.inner,), torch.float32)

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.w_in, self.w_out = tensors["in.weight"].float(), tensors["out.weight"].float()

        def forward(self, ctx, h, x, view, owns_cache=True):
            u = h[:ctx.n_tokens].float() @ self.w_in.t()
            row = 0
            for slot, n in zip(ctx.host_seq_slot, ctx.host_seq_new):
                s = view.state[slot]
                for t in range(row, row + n):
                    s.mul_(self.decay).add_(u[t])
                    x[t] += self.w_out @ s
                row += n

    MIXERS.register("toy_decay", DecayMixer, replace=True)

    def config_from_dict(d):
        return dict(d)

    def describe(c):
        def norm(prefix):
            return PartSpec("rmsnorm", dict(width=E, eps=c["eps"]), prefix=prefix)

        def ffn(prefix):
            return PartSpec("gated_mlp", dict(hidden_size=E, intermediate_size=F), prefix=prefix)
        pos = PartSpec("rotary", dict(head_dim=D, rotary_dim=D, theta=c["theta"], layout="split_half", scaling=None))

        def attn(prefix, shared):
            return PartSpec("attention", dict(hidden_size=E, num_heads=H, num_kv_heads=K, head_dim=D,
                                              scale=D ** -0.5, window=0, position=pos, shared_cache=shared), prefix=prefix)
        layers = [
            LayerSpec("prenorm", norm("l0.n1."), attn("l0.attn.", False), norm("l0.n2."), ffn("l0.mlp.")),
            LayerSpec("prenorm", norm("l1.n1."), PartSpec("toy_decay", dict(width=E, inner=24, decay=c["decay"]),
                                                           prefix="l1.mix."), norm("l1.n2."), ffn("l1.mlp.")),
            LayerSpec("prenorm", norm("l2.n1."), attn("l2.attn.", True), norm("l2.n2."), ffn("l2.mlp.")),
        ]
        # layer 1 runs twice (two states); layer 2 reads the cache that entry 0 wrote
        schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, cache=0), ScheduleEntry(1)]
        return ModelSpec(hidden_size=E, vocab_size=V, max_positions=256,
                         embedding=PartSpec("embedding", dict(vocab_size=V, width=E), prefix="emb."),
                         layers=layers, schedule=schedule, final_norm=norm("final."),
                         lm_head=PartSpec("lm_head", dict(vocab_size=V, width=E), prefix="head."))

    ARCHITECTURES.register("ToyMixedLM", Architecture("ToyMixedLM", config_from_dict, describe), replace=True)


def plain_toy(c, W, ids):
    """The same toy model, whole sequence, float64, written out by hand."""
    W = {k: v.double() for k, v in W.items()}
    T = len(ids)
    x = W["emb.weight"][torch.tensor(ids)]
    inv = plain_inv_freq(D, c["theta"], None)
    pos = torch.arange(T)
    kv = {}

    def mlp(x, p):
        h = plain_rmsnorm(x, W[p + "n2.weight"], c["eps"])
        return x + plain_swiglu(h @ W[p + "mlp.gate_proj.weight"].t(), h @ W[p + "mlp.up_proj.weight"].t()) @ W[p + "mlp.down_proj.weight"].t()

    def attn(x, p, shared):
        h = plain_rmsnorm(x, W[p + "n1.weight"], c["eps"])
        q = plain_rope((h @ W[p + "attn.q_proj.weight"].t()).reshape(T, H, D), pos, inv, "split_half")
        if not shared:
            kv["k"] = plain_rope((h @ W[p + "attn.k_proj.weight"].t()).reshape(T, K, D), pos, inv, "split_half")
            kv["v"] = (h @ W[p + "attn.v_proj.weight"].t()).reshape(T, K, D)
        return x + plain_attention(q, kv["k"], kv["v"], D ** -0.5) @ W[p + "attn.o_proj.weight"].t()

    def decay(x, p):
        h = plain_rmsnorm(x, W[p + "n1.weight"], c["eps"])
        u = h @ W[p + "mix.in.weight"].t()
        s = torch.zeros(24, dtype=torch.float64)
        out = x.clone()
        for t in range(T):
            s = c["decay"] * s + u[t]
            out[t] = x[t] + W[p + "mix.out.weight"] @ s
        return out

    x = mlp(attn(x, "l0.", False), "l0.")
    x = mlp(decay(x, "l1."), "l1.")
    x = mlp(attn(x, "l2.", True), "l2.")
    x = mlp(decay(x, "l1."), "l1.")
    return plain_rmsnorm(x, W["final.weight"], c["eps"]) @ W["head.weight"].t()


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 6e-2)])
def test_toy_architecture_builds_and_steps(tmp_path, dtype, tol):
    register_toy()
    from mdma_b200.engine import Engine, StepEntry
    from mdma_b200.weights import write_random_model
    from mdma_b200.weights.safetensors_io import SafetensorsFile
    cfg = dict(architectures=["ToyMixedLM"], eps=1e-5, theta=5000.0, decay=0.8)
    d = write_random_model(str(tmp_path / "toy"), cfg, 7, torch.float32)
    jitter_norm_weights(d, 7)          # norm weights that differ in every vector
    sf = SafetensorsFile(os.path.join(d, "model.safetensors"))
    W = {n: sf.tensor(n).clone() for n in sf.entries}
    assert "l2.attn.k_proj.weight" not in W and "l1.mix.in.weight" in W     # the sharing layer owns no k/v
    eng = Engine(d, dtype=dtype, max_batch=3, max_context=128, logit_rows=128)
    assert len(eng.cache.groups) == 1 and eng.cache.groups[0].sites == [0]  # one cache site, read twice
    assert sorted(eng.cache.states) == [1, 3]                               # two runs, two states
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (33, 9, 70)]
    ref = [plain_toy(cfg, W, s).numpy() for s in seqs]
    # whole prompts of unequal length in one step
    slots = [eng.acquire() for _ in seqs]
    out = eng.step([StepEntry(sl, s, list(range(len(s)))) for sl, s in zip(slots, seqs)]).cpu().numpy()
    off = 0
    for s, r in zip(seqs, ref):
        assert np.abs(out[off:off + len(s)] - r).max() < tol
        off += len(s)
    for sl in slots:
        eng.release(sl)
    # a prompt, then one token each; the second batch reuses the slots (state must start from zero)
    slots = [eng.acquire() for _ in seqs]
    cut = [len(s) // 2 for s in seqs]
    eng.step([StepEntry(sl, s[:c], []) for sl, s, c in zip(slots, seqs, cut)])
    pos = list(cut)
    live = list(range(len(seqs)))
    while live:
        out = eng.step([StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu().numpy()
        for row, i in enumerate(live):
            assert np.abs(out[row] - ref[i][pos[i]]).max() < tol, (i, pos[i])
            pos[i] += 1
        for i in [i for i in live if pos[i] == len(seqs[i])]:
            eng.release(slots[i])
        live = [i for i in live if pos[i] < len(seqs[i])]
    eng.cache.check()


# ---------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, both defined here.

def register_toy_routed():
    from mdma_b200 import ops
    from mdma_b200.config import Architecture
    from mdma_b200.parts.base import Part
    from mdma_b200.registry import ARCHITECTURES, FEED_FORWARDS, POSITIONS
    from mdma_b200.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

    class RoutedMLP(Part):
        """Top-1 of n experts: router logits in float32, the chosen expert's SwiGLU, weighted by
        its softmax probability; x += p * expert(h)."""

        def __init__(self, spec):
            super().__init__(spec)
            self.width, self.inner, self.n = spec.params["width"], spec.params["inner"], spec.params["experts"]

        def tensor_specs(self):
            t = {"router.weight": TensorSpec((self.n, self.width))}
            for e in range(self.n):
                t[f"experts.{e}.gate.weight"] = TensorSpec((self.inner, self.width))
                t[f"experts.{e}.up.weight"] = TensorSpec((self.inner, self.width))
                t[f"experts.{e}.down.weight"] = TensorSpec((self.width, self.inner))
            return t

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.t = {k: v.float() for k, v in tensors.items()}

        def forward(self, ctx, h, x):
            hf = h[:ctx.n_tokens].float()
            probs = torch.softmax(hf @ self.t["router.weight"].t(), dim=-1)      # router in float32
            top = probs.argmax(dim=-1)
            for e in range(self.n):
                rows = (top == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                he = hf[rows]
                g = he @ self.t[f"experts.{e}.gate.weight"].t()
                act = g / (1 + torch.exp(-g)) * (he @ self.t[f"experts.{e}.up.weight"].t())
                x[rows] += probs[rows, e:e + 1] * (act @ self.t[f"experts.{e}.down.weight"].t())

    class LearnedOffsets(Part):
        """A position encoding that is no rotation: q and k get a learned vector per position added
        (a table in the checkpoint), then k and v go to the cache."""

        def __init__(self, spec):
            super().__init__(spec)
            self.head_dim, self.max_pos = spec.params["head_dim"], spec.params["max_positions"]

        def tensor_specs(self):
            return {"table": TensorSpec((self.max_pos, self.head_dim))}

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.table = tensors["table"]
            self.zero_freq = torch.zeros(self.head_dim // 2, dtype=torch.float32, device=rt.device)

        def encode_and_store(self, ctx, qkv, n_heads, n_kv_heads, head_dim, view, write_kv):
            n = ctx.n_tokens
            add = self.table[ctx.tok_pos.long()].to(qkv.dtype)                    # [n, head_dim]
            heads = n_heads + (n_kv_heads if write_kv else 0)                     # q and k, not v
            rows = qkv[:n, :heads * head_dim].reshape(n, heads, head_dim)
            rows += add[:, None, :]
            # angle 0 everywhere: the library's cache-write kernel then only stores k and v
            ops.rope_cache_write(qkv, n, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, self.zero_freq,
                                 view.k if write_kv else None, view.v if write_kv else None,
                                 view.page_table if write_kv else None, view.max_pages, view.page_size,
                                 n_heads, n_kv_heads, head_dim, head_dim, False, write_kv)

    FEED_FORWARDS.register("toy_routed", RoutedMLP, replace=True)
    POSITIONS.register("toy_learned", LearnedOffsets, replace=True)

    def describe(c):
        norm = lambda p: PartSpec("rmsnorm", dict(width=E, eps=c["eps"]), prefix=p)
        pos = PartSpec("toy_learned", dict(head_dim=D, max_positions=64), prefix="pos.")
        attn = lambda p: PartSpec("attention", dict(hidden_size=E, num_heads=H, num_kv_heads=K, head_dim=D,
                                                    scale=D ** -0.5, window=0, position=pos), prefix=p)
        layers = [
            LayerSpec("prenorm", norm("l0.n1."), attn("l0.attn."), norm("l0.n2."),
                      PartSpec("toy_routed", dict(width=E, inner=40, experts=3), prefix="l0.moe.")),
            LayerSpec("prenorm", norm("l1.n1."), attn("l1.attn."), norm("l1.n2."),
                      PartSpec("gated_mlp", dict(hidden_size=E, intermediate_size=F), prefix="l1.mlp.")),
        ]
        return ModelSpec(hidden_size=E, vocab_size=V, max_positions=64,
                         embedding=PartSpec("embedding", dict(vocab_size=V, width=E), prefix="emb."),
                         layers=layers, schedule=[ScheduleEntry(0), ScheduleEntry(1)], final_norm=norm("final."),
                         lm_head=PartSpec("lm_head", dict(vocab_size=V, width=E), prefix="head."))

    ARCHITECTURES.register("ToyRoutedLM", Architecture("ToyRoutedLM", dict, describe), replace=True)


def plain_toy_routed(c, W, ids):
    W = {k: v.double() for k, v in W.items()}
    T = len(ids)
    x = W["emb.weight"][torch.tensor(ids)]
    add = W["pos.table"][:T]

    def attn(x, p):
        h = plain_rmsnorm(x, W[p + "n1.weight"], c["eps"])
        q = (h @ W[p + "attn.q_proj.weight"].t()).reshape(T, H, D) + add[:, None, :]
        k = (h @ W[p + "attn.k_proj.weight"].t()).reshape(T, K, D) + add[:, None, :]
        v = (h @ W[p + "attn.v_proj.weight"].t()).reshape(T, K, D)
        return x + plain_attention(q, k, v, D ** -0.5) @ W[p + "attn.o_proj.weight"].t()

    x = attn(x, "l0.")
    h = plain_rmsnorm(x, W["l0.n2.weight"], c["eps"])
    probs = torch.softmax(h @ W["l0.moe.router.weight"].t(), dim=-1)
    top = probs.argmax(-1)
    out = x.clone()
    for t in range(T):
        e = int(top[t])
        g = h[t] @ W[f"l0.moe.experts.{e}.gate.weight"].t()
        act = plain_swiglu(g, h[t] @ W[f"l0.moe.experts.{e}.up.weight"].t())
        out[t] = x[t] + probs[t, e] * (act @ W[f"l0.moe.experts.{e}.down.weight"].t())
    x = attn(out, "l1.")
    h = plain_rmsnorm(x, W["l1.n2.weight"], c["eps"])
    x = x + plain_swiglu(h @ W["l1.mlp.gate_proj.weight"].t(), h @ W["l1.mlp.up_proj.weight"].t()) @ W["l1.mlp.down_proj.weight"].t()
    return plain_rmsnorm(x, W["final.weight"], c["eps"]) @ W["head.weight"].t()


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    """One model with a routed and a dense feed-forward in different layers and a position encoding that
    is not rotary, registered from here; float32 so that every token takes the same expert in both."""
    register_toy_routed()
    from mdma_b200.engine import Engine, StepEntry
    from mdma_b200.weights import write_random_model, write_safetensors
    from mdma_b200.weights.safetensors_io import SafetensorsFile
    cfg = dict(architectures=["ToyRoutedLM"], eps=1e-5)
    d = write_random_model(str(tmp_path / "toy2"), cfg, 3, torch.float32)
    jitter_norm_weights(d, 3)          # norm weights that differ in every vector
    sf = SafetensorsFile(os.path.join(d, "model.safetensors"))
    W = {n: sf.tensor(n).clone() for n in sf.entries}
    W["l0.moe.router.weight"] = W["l0.moe.router.weight"] * 40      # decisive routing, all experts used
    W["pos.table"] = W["pos.table"] * 10
    write_safetensors(os.path.join(d, "model.safetensors"), W)
    eng = Engine(d, dtype="float32", max_batch=2, max_context=64, logit_rows=64)
    g = torch.Generator().manual_seed(1)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (40, 13)]
    ref = [plain_toy_routed(cfg, W, s).numpy() for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    cut = [25, 5]
    out = eng.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    off = 0
    for s, r, c in zip(seqs, ref, cut):
        assert np.abs(out[off:off + c] - r[:c]).max() < 5e-5
        off += c
    for step in range(8):
        out = eng.step([StepEntry(sl, [s[c + step]], [0]) for sl, s, c in zip(slots, seqs, cut)]).cpu().numpy()
        for row, (r, c) in enumerate(zip(ref, cut)):
            assert np.abs(out[row] - r[c + step]).max() < 5e-5


# ---- a block arrangement of its own, with more parts than the four of a layer ------------------------------
def register_toy_sandwich():
    """x += post_norm(mixer(pre_norm(x))) and the same around the feed-forward: two norms per layer that the
    built-in arrangement does not have, found in `LayerSpec.extras`; the arrangement asks for a workspace
    buffer of its own.  Registered from here."""
    from mdma_b200.config import Architecture
    from mdma_b200.registry import ARCHITECTURES, BLOCKS, FEED_FORWARDS, MIXERS, NORMS
    from mdma_b200.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    class SandwichBlock:
        def __init__(self, spec):
            self.spec = spec
            make = lambda reg, ps: reg.get(ps.kind)(ps)
            self.mixer_norm, self.mixer = make(NORMS, spec.mixer_norm), make(MIXERS, spec.mixer)
            self.ffn_norm, self.ffn = make(NORMS, spec.ffn_norm), make(FEED_FORWARDS, spec.ffn)
            self.post_mixer, self.post_ffn = make(NORMS, spec.extras["post_mixer_norm"]), make(NORMS, spec.extras["post_ffn_norm"])

        def parts(self):
            return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.post_mixer, self.post_ffn]

        def workspace(self):
            return {"normed": (E, "act"), "branch": (E, "f32"), "branch_normed": (E, "act")}

        def forward(self, ctx, x, view, owns_cache=True):
            n = ctx.n_tokens
            h, y, yn = ctx.buf("normed", E), ctx.buf("branch", E, torch.float32), ctx.buf("branch_normed", E)
            for pre, part, post in ((self.mixer_norm, self.mixer, self.post_mixer), (self.ffn_norm, self.ffn, self.post_ffn)):
                pre.forward(ctx, x, h)
                y[:n].zero_()
                if part is self.mixer:
                    part.forward(ctx, h, y, view, owns_cache)
                else:
                    part.forward(ctx, h, y)
                post.forward(ctx, y, yn)              # adds up what a K-split product left for y, then norms it
                x[:n] += yn[:n].float()

    BLOCKS.register("toy_sandwich", SandwichBlock, replace=True)

    def describe(c):
        norm = lambda prefix: PartSpec("rmsnorm", dict(width=E, eps=c["eps"]), prefix=prefix)
        pos = PartSpec("rotary", dict(head_dim=D, rotary_dim=D, theta=c["theta"], layout="interleaved", scaling=None))
        layers = []
        for i in range(2):
            p = f"l{i}."
            layers.append(LayerSpec(
                "toy_sandwich" if i == 0 else "prenorm", norm(p + "n1."),
                PartSpec("attention", dict(hidden_size=E, num_heads=H, num_kv_heads=K, head_dim=D, scale=D ** -0.5,
                                           window=0, position=pos), prefix=p + "attn."),
                norm(p + "n2."), PartSpec("gated_mlp", dict(hidden_size=E, intermediate_size=F), prefix=p + "mlp."),
                extras={"post_mixer_norm": norm(p + "n3."), "post_ffn_norm": norm(p + "n4.")} if i == 0 else {}))
        return ModelSpec(hidden_size=E, vocab_size=V, max_positions=256,
                         embedding=PartSpec("embedding", dict(vocab_size=V, width=E), prefix="emb."),
                         layers=layers, schedule=[ScheduleEntry(0), ScheduleEntry(1)], final_norm=norm("final."),
                         lm_head=PartSpec("lm_head", dict(vocab_size=V, width=E), prefix="head."))

    ARCHITECTURES.register("ToySandwichLM", Architecture("ToySandwichLM", lambda d: dict(d), describe), replace=True)


def plain_toy_sandwich(c, W, ids):
    W = {k: v.double() for k, v in W.items()}
    T = len(ids)
    x = W["emb.weight"][torch.tensor(ids)]
    inv = plain_inv_freq(D, c["theta"], None)
    pos = torch.arange(T)

    def attn(h, p):
        q = plain_rope((h @ W[p + "attn.q_proj.weight"].t()).reshape(T, H, D), pos, inv, "interleaved")
        k = plain_rope((h @ W[p + "attn.k_proj.weight"].t()).reshape(T, K, D), pos, inv, "interleaved")
        v = (h @ W[p + "attn.v_proj.weight"].t()).reshape(T, K, D)
        return plain_attention(q, k, v, D ** -0.5) @ W[p + "attn.o_proj.weight"].t()

    def mlp(h, p):
        return plain_swiglu(h @ W[p + "mlp.gate_proj.weight"].t(), h @ W[p + "mlp.up_proj.weight"].t()) @ W[p + "mlp.down_proj.weight"].t()
    n = lambda v, name: plain_rmsnorm(v, W[name], c["eps"])
    x = x + n(attn(n(x, "l0.n1.weight"), "l0."), "l0.n3.weight")
    x = x + n(mlp(n(x, "l0.n2.weight"), "l0."), "l0.n4.weight")
    x = x + attn(n(x, "l1.n1.weight"), "l1.")
    x = x + mlp(n(x, "l1.n2.weight"), "l1.")
    return n(x, "final.weight") @ W["head.weight"].t()


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 8e-2)])
def test_a_block_arrangement_with_parts_of_its_own(tmp_path, dtype, tol):
    """A layer arranged differently (norms after the mixer and after the feed-forward, taken from
    `LayerSpec.extras`, with workspace the arrangement asks for itself) next to an ordinary layer; in
    bfloat16 the products leave K-split partial sums that only the built-in arrangement knows of: the model
    completes the residual stream before it hands it to the foreign one."""
    register_toy_sandwich()
    from mdma_b200.engine import Engine, StepEntry
    from mdma_b200.weights import write_random_model
    from mdma_b200.weights.safetensors_io import SafetensorsFile
    cfg = dict(architectures=["ToySandwichLM"], eps=1e-5, theta=10000.0)
    d = write_random_model(str(tmp_path / "toy3"), cfg, 4, torch.bfloat16 if dtype == "bfloat16" else torch.float32, std=0.08)
    jitter_norm_weights(d, 4)          # norm weights that differ in every vector
    sf = SafetensorsFile(os.path.join(d, "model.safetensors"))
    W = {n: sf.tensor(n).clone().float() for n in sf.entries}
    assert "l0.n3.weight" in W and "l1.n3.weight" not in W          # the loader learnt the extra tensors from the parts
    eng = Engine(d, dtype=dtype, max_batch=2, max_context=128, logit_rows=128)
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (70, 9)]
    ref = [plain_toy_sandwich(cfg, W, s).numpy() for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    cut = [50, 3]
    out = eng.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    off = 0
    for r, c in zip(ref, cut):
        assert np.abs(out[off:off + c] - r[:c]).max() < tol
        off += c
    for step in range(6):
        out = eng.step([StepEntry(sl, [s[c + step]], [0]) for sl, s, c in zip(slots, seqs, cut)]).cpu().numpy()
        for row, (r, c) in enumerate(zip(ref, cut)):
            assert np.abs(out[row] - r[c + step]).max() < tol
    eng.check_status()


# ---- the built-in parts with options that Llama does not use: biases after every product, a GELU gate ----------
def register_toy_biased():
    """Two ordinary layers whose attention has a bias vector after each of its four products and whose
    feed-forward is gated by GELU (tanh form) with biases after its three: options of the parts, chosen by
    an architecture that is registered from here."""
    from mdma_b200.config import Architecture
    from mdma_b200.registry import ARCHITECTURES
    from mdma_b200.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    def describe(c):
        norm = lambda prefix: PartSpec("rmsnorm", dict(width=E, eps=c["eps"]), prefix=prefix)
        pos = PartSpec("rotary", dict(head_dim=D, rotary_dim=D, theta=c["theta"], layout="split_half", scaling=None))
        layers = []
        for i in range(2):
            p = f"l{i}."
            layers.append(LayerSpec(
                "prenorm", norm(p + "n1."),
                PartSpec("attention", dict(hidden_size=E, num_heads=H, num_kv_heads=K, head_dim=D, scale=D ** -0.5,
                                           window=0, position=pos, bias=True), prefix=p + "attn."),
                norm(p + "n2."),
                PartSpec("gated_mlp", dict(hidden_size=E, intermediate_size=F, bias=True,
                                           activation="gelu_tanh" if i == 0 else "silu"), prefix=p + "mlp.")))
        return ModelSpec(hidden_size=E, vocab_size=V, max_positions=256,
                         embedding=PartSpec("embedding", dict(vocab_size=V, width=E), prefix="emb."),
                         layers=layers, schedule=[ScheduleEntry(0), ScheduleEntry(1)], final_norm=norm("final."),
                         lm_head=PartSpec("lm_head", dict(vocab_size=V, width=E), prefix="head."))

    ARCHITECTURES.register("ToyBiasedLM", Architecture("ToyBiasedLM", lambda d: dict(d), describe), replace=True)


def plain_toy_biased(c, W, ids):
    W = {k: v.double() for k, v in W.items()}
    T = len(ids)
    x = W["emb.weight"][torch.tensor(ids)]
    inv = plain_inv_freq(D, c["theta"], None)
    pos = torch.arange(T)
    lin = lambda h, name: h @ W[name + ".weight"].t() + W[name + ".bias"]
    for i in range(2):
        p = f"l{i}."
        h = plain_rmsnorm(x, W[p + "n1.weight"], c["eps"])
        q = plain_rope(lin(h, p + "attn.q_proj").reshape(T, H, D), pos, inv, "split_half")
        k = plain_rope(lin(h, p + "attn.k_proj").reshape(T, K, D), pos, inv, "split_half")
        v = lin(h, p + "attn.v_proj").reshape(T, K, D)
        x = x + lin(plain_attention(q, k, v, D ** -0.5), p + "attn.o_proj")
        h = plain_rmsnorm(x, W[p + "n2.weight"], c["eps"])
        g, u = lin(h, p + "mlp.gate_proj"), lin(h, p + "mlp.up_proj")
        if i == 0:
            act = 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3))) * u
        else:
            act = plain_swiglu(g, u)
        x = x + lin(act, p + "mlp.down_proj")
    return plain_rmsnorm(x, W["final.weight"], c["eps"]) @ W["head.weight"].t()


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 8e-2)])
def test_biases_and_another_gate_activation_are_options_of_the_parts(tmp_path, dtype, tol):
    """The bias vectors are seeded like matrices (so that a missing one shows), laid out with q, k and v as one
    vector beside the one matrix, added once however the product is split over K, and reach the attention
    kernel that does the rotary encoding itself (single tokens) through the first partial sum."""
    register_toy_biased()
    from mdma_b200.engine import Engine, StepEntry
    from mdma_b200.weights import write_random_model
    from mdma_b200.weights.safetensors_io import SafetensorsFile
    cfg = dict(architectures=["ToyBiasedLM"], eps=1e-5, theta=10000.0)
    d = write_random_model(str(tmp_path / "toy4"), cfg, 5, torch.bfloat16 if dtype == "bfloat16" else torch.float32, std=0.08)
    jitter_norm_weights(d, 5)          # norm weights that differ in every vector
    sf = SafetensorsFile(os.path.join(d, "model.safetensors"))
    W = {n: sf.tensor(n).clone().float() for n in sf.entries}
    assert W["l0.attn.q_proj.bias"].shape == (H * D,) and float(W["l1.mlp.down_proj.bias"].abs().max()) > 0.05
    eng = Engine(d, dtype=dtype, max_batch=2, max_context=128, logit_rows=128)
    held = eng.held_bytes()
    assert all(eng.memory_plan()[k] == v for k, v in held.items())         # the bias vectors are in the plan
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (70, 9)]
    ref = [plain_toy_biased(cfg, W, s).numpy() for s in seqs]
    # the biases matter: without them the logits differ by far more than the tolerance
    W0 = {n: (torch.zeros_like(t) if n.endswith(".bias") else t) for n, t in W.items()}
    assert np.abs(plain_toy_biased(cfg, W0, seqs[0]).numpy() - ref[0]).max() > 10 * tol
    slots = [eng.acquire() for _ in seqs]
    cut = [50, 3]
    out = eng.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    off = 0
    for r, c in zip(ref, cut):
        assert np.abs(out[off:off + c] - r[:c]).max() < tol
        off += c
    for step in range(6):
        out = eng.step([StepEntry(sl, [s[c + step]], [0]) for sl, s, c in zip(slots, seqs, cut)]).cpu().numpy()
        for row, (r, c) in enumerate(zip(ref, cut)):
            assert np.abs(out[row] - r[c + step]).max() < tol
    eng.check_status()


# ---- layers with different cache needs in one model: all keys, and windows of two widths ------------------------
WINDOWS = (0, 40, 100)
GEOMETRY = ((H, K, D), (H, K, D), (2, 1, 32))        # heads, kv heads, head size of each layer: the last differs too


def register_toy_windowed():
    """Three attention layers: the first reads every key, the others only the last 40 and the last 100, and the
    last has other heads (2 of 32 over 1 kv head).  Their caches are three groups with storage of their own; the windowed groups give pages back while a sequence
    grows.  An architecture registered from here, out of the built-in parts."""
    from mdma_b200.config import Architecture
    from mdma_b200.registry import ARCHITECTURES
    from mdma_b200.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    def describe(c):
        norm = lambda prefix: PartSpec("rmsnorm", dict(width=E, eps=c["eps"]), prefix=prefix)
        layers = []
        for i, (window, (h, k, d)) in enumerate(zip(WINDOWS, GEOMETRY)):
            p = f"l{i}."
            pos = PartSpec("rotary", dict(head_dim=d, rotary_dim=d, theta=c["theta"], layout="split_half", scaling=None))
            layers.append(LayerSpec(
                "prenorm", norm(p + "n1."),
                PartSpec("attention", dict(hidden_size=E, num_heads=h, num_kv_heads=k, head_dim=d, scale=d ** -0.5,
                                           window=window, position=pos), prefix=p + "attn."),
                norm(p + "n2."), PartSpec("gated_mlp", dict(hidden_size=E, intermediate_size=F), prefix=p + "mlp.")))
        return ModelSpec(hidden_size=E, vocab_size=V, max_positions=512,
                         embedding=PartSpec("embedding", dict(vocab_size=V, width=E), prefix="emb."),
                         layers=layers, schedule=[ScheduleEntry(i) for i in range(len(WINDOWS))], final_norm=norm("final."),
                         lm_head=PartSpec("lm_head", dict(vocab_size=V, width=E), prefix="head."))

    ARCHITECTURES.register("ToyWindowedLM", Architecture("ToyWindowedLM", lambda d: dict(d), describe), replace=True)


def plain_toy_windowed(c, W, ids):
    W = {k: v.double() for k, v in W.items()}
    T = len(ids)
    x = W["emb.weight"][torch.tensor(ids)]
    pos = torch.arange(T)
    for i, (window, (nh, nk, hd)) in enumerate(zip(WINDOWS, GEOMETRY)):
        p = f"l{i}."
        inv = plain_inv_freq(hd, c["theta"], None)
        h = plain_rmsnorm(x, W[p + "n1.weight"], c["eps"])
        q = plain_rope((h @ W[p + "attn.q_proj.weight"].t()).reshape(T, nh, hd), pos, inv, "split_half")
        k = plain_rope((h @ W[p + "attn.k_proj.weight"].t()).reshape(T, nk, hd), pos, inv, "split_half")
        v = (h @ W[p + "attn.v_proj.weight"].t()).reshape(T, nk, hd)
        x = x + plain_attention(q, k, v, hd ** -0.5, window) @ W[p + "attn.o_proj.weight"].t()
        h = plain_rmsnorm(x, W[p + "n2.weight"], c["eps"])
        x = x + plain_swiglu(h @ W[p + "mlp.gate_proj.weight"].t(), h @ W[p + "mlp.up_proj.weight"].t()) @ W[p + "mlp.down_proj.weight"].t()
    return plain_rmsnorm(x, W["final.weight"], c["eps"]) @ W["head.weight"].t()


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 8e-2)])
def test_layers_with_all_keys_and_with_windows_in_one_model(tmp_path, dtype, tol):
    """Prompts of 330 and 75 tokens in pieces (200 + 66 + single tokens; 70 + single tokens), NaN in every cache row
    nobody owns: logits against the plain implementation with the same windows; the windowed groups hold
    only the pages their windows reach (and gave the others back while the sequence grew), the group of all keys
    holds them all."""
    register_toy_windowed()
    from mdma_b200.engine import Engine, StepEntry
    from mdma_b200.weights import write_random_model
    cfg = dict(architectures=["ToyWindowedLM"], eps=1e-5, theta=10000.0)
    d = write_random_model(str(tmp_path / "toy5"), cfg, 6, torch.bfloat16 if dtype == "bfloat16" else torch.float32, std=0.08)
    W = {n: t.float() for n, t in jitter_norm_weights(d, 6).items()}
    eng = Engine(d, dtype=dtype, max_batch=2, max_context=384, logit_rows=256)
    groups = {g.need.window: g for g in eng.cache.groups}
    assert sorted(groups) == [0, 40, 100] and all(len(g.sites) == 1 for g in groups.values())
    gen = torch.Generator().manual_seed(4)
    seqs = [torch.randint(0, V, (n,), generator=gen).tolist() for n in (330, 75)]
    ref = [plain_toy_windowed(cfg, W, s).numpy() for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    pos = [0, 0]
    plan = [[200, 66] + [1] * 64, [70] + [1] * 5]            # tokens each request brings, step by step
    for step in range(max(len(p) for p in plan)):
        entries, places = [], []
        for i in range(2):
            if step < len(plan[i]):
                n = plan[i][step]
                want = sorted({0, n // 2, n - 1})
                entries.append(StepEntry(slots[i], seqs[i][pos[i]:pos[i] + n], want))
                places += [(i, pos[i] + w) for w in want]
                pos[i] += n
        eng.cache.poison_unused()
        out = eng.step(entries).cpu().numpy()
        want_rows = np.stack([ref[i][p] for i, p in places])
        assert np.abs(out - want_rows).max() < tol, (step, np.abs(out - want_rows).max())
    assert pos == [330, 75]
    page = eng.cache.page_size
    held = lambda window, slot: sorted(groups[window].seq_pages[slot])
    assert held(0, slots[0]) == list(range(-(-330 // page)))
    for window in (40, 100):
        first = max(0, 330 - window) // page                 # the page of the earliest key the next token would read
        assert held(window, slots[0]) == list(range(first, -(-330 // page))), (window, held(window, slots[0]))
    eng.cache.check()
    for s in slots:
        eng.release(s)
    eng.cache.check()
    assert all(g.pages.free_count == g.n_pages for g in groups.values())
    # and through the generation loop: replayed decode steps (graphs) equal the step-by-step loop while the
    # windows move over page boundaries and pages are given back between runs
    prompts = [s[:130] for s in seqs[:1]] + [seqs[1][:20]]
    a = eng.generate(prompts, max_tokens=70)
    b = eng.generate(prompts, max_tokens=70, use_graphs=False)
    assert [o.tokens for o in a] == [o.tokens for o in b] and all(len(o.tokens) == 70 for o in a)
    eng.cache.check()
    eng.check_status()
