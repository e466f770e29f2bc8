"""Times of the decode step's kernels one by one, at the sizes of a configuration.

    python -m mdma_b200.kernel_times [--batch 8] [--context 580] [--hidden 4096] [--intermediate 14336]
                                     [--heads 32] [--kv-heads 8] [--head-dim 128] [--vocab 128256]
                                     [--bn 128 --splits 2]      (the products with another tile and split)

An engine with `--copies` layers of these sizes is built with seeded random weights, its cache is filled
to `--context` positions, and each kernel of a layer is called through the engine's own parts with the
step context of the engine's own decode session (nothing here lays out step metadata of its own).  Every
kernel is captured `--repeat` times in a CUDA graph, going through the layers in turn so that the 126 MB
L2 does not serve weights or cache, and timed with CUDA events around two replays.  The sizes default to
the Llama-3.1-8B layer.  The numbers under `profiles/` that name this module were made with it.
"""
from __future__ import annotations

import argparse

import torch


def _timeit(name: str, fn, repeat: int, nbytes: int = 0) -> float:
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(repeat):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000 / (2 * repeat)
    print(f"{name:44s} {us:9.2f} us" + (f"  {nbytes / us / 1e3:7.0f} GB/s" if nbytes else ""), flush=True)
    return us


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=580)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=14336)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--copies", type=int, default=6, help="layers (copies of weights and cache) that take turns")
    ap.add_argument("--repeat", type=int, default=48)
    ap.add_argument("--bn", type=int, default=None,
                    help="token tile of the four products instead of the plan's: 16...256 one block per tile, 512 block pairs")
    ap.add_argument("--splits", type=int, default=None,
                    help="K splits of the QKV, O and down products instead of the plan's (with --bn below 512)")
    a = ap.parse_args(argv)

    from . import ops
    from .engine import Engine
    from .sampling import SamplingParams
    torch.cuda.set_device(0)
    B, C = a.batch, a.copies
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=C, hidden_size=a.hidden,
               num_attention_heads=a.heads, num_key_value_heads=a.kv_heads, head_dim=a.head_dim,
               intermediate_size=a.intermediate, vocab_size=a.vocab, rope_theta=500000.0, rms_norm_eps=1e-5,
               tie_word_embeddings=False, max_position_embeddings=a.context + 64)
    eng = Engine(config=cfg, seed=0, dtype="bfloat16", max_batch=B, max_context=a.context + 64)
    # B sequences of `context` positions: pages are reserved and counted as written (their rows hold zeros)
    slots = [eng.acquire() for _ in range(B)]
    ext = {s: a.context - 1 for s in slots}
    eng.cache.extend(ext)
    eng.cache.commit(ext)
    sess = eng.decode_session()
    sess.start(slots, [1] * B)
    eng.cache.extend({s: 1 for s in slots})          # room for the token of this step
    sess._bucket = -(-a.context // 1024) * 1024
    ctx = sess.set_context(B)
    blocks = eng.model.blocks
    x = ctx.buf("x", a.hidden, torch.float32)
    h = ctx.buf("normed", a.hidden)
    eng.model.embedding.forward(ctx, ctx.ids, x)
    view = lambda i: eng.cache.view(i % C)
    tc = eng.rt.tc
    from . import ops_tensor

    def settle():
        ops_tensor.flush_pending(eng.device, tc)

    forced = dict(bn=a.bn, splits=a.splits if a.splits is not None else 1) if a.bn is not None else None

    def product(lin, src, dst, mode):
        # the part's own call, or (--bn/--splits) the same product with a tile and a split that the plan would not take
        if forced is None:
            lin._run(mode, src, dst, B, defer=True)
        else:
            kw = dict(forced, splits=1) if mode == ops.GEMM_SWIGLU else forced
            ops_tensor.gemm(src, lin.w, dst, mode, lin.w2, B, defer=True, st=tc, **kw)
        tc.pending = None                              # the partial sums stay where they are; nobody adds them here

    def qkv_only(i):
        m = blocks[i % C].mixer
        product(m.qkv_proj, h, ctx.buf("qkv", m.row_width), ops.GEMM_STORE)

    def attention_only(i):
        m = blocks[i % C].mixer
        qkv, out = ctx.buf("qkv", m.row_width), ctx.buf("attn_out", m.q_width)
        if m._fusable(ctx, view(i)):
            inv_freq, rot, inter = m.position.rotary_table()
            ops_tensor.attention_decode_rotary(ctx, qkv, view(i), out, m.n_heads, m.n_kv_heads, m.head_dim, m.window,
                                               m.scale, inv_freq, rot, inter, st=tc)
        else:
            m.position.encode_and_store(ctx, qkv, m.n_heads, m.n_kv_heads, m.head_dim, view(i), True)
            ops_tensor.attention(ctx, qkv, view(i), out, m.n_heads, m.n_kv_heads, m.head_dim, m.window, m.scale, st=tc)

    def o_only(i):
        m = blocks[i % C].mixer
        product(m.o_proj, ctx.buf("attn_out", m.q_width), x, ops.GEMM_ACCUMULATE)

    def gate_up_only(i):
        f = blocks[i % C].ffn
        product(f.gate_up, h, ctx.buf("act", f.inner), ops.GEMM_SWIGLU)

    def down_only(i):
        f = blocks[i % C].ffn
        product(f.down, ctx.buf("act", f.inner), x, ops.GEMM_ACCUMULATE)

    n = a.repeat
    E, F, H, K, D, V = a.hidden, a.intermediate, a.heads, a.kv_heads, a.head_dim, a.vocab
    fused = blocks[0].mixer._fusable(ctx, view(0))
    total = 0.0
    total += 2 * _timeit("RMSNorm", lambda i: blocks[i % C].mixer_norm.forward(ctx, x, h), n)
    total += _timeit("QKV product (partial sums left)", qkv_only, n, (H + 2 * K) * D * E * 2)
    total += _timeit("rotary + cache write + attention" + (" (one kernel)" if fused else ""), attention_only, n,
                     B * a.context * K * D * 2 * 2)
    total += _timeit("O product (partial sums left)", o_only, n, H * D * E * 2)
    total += _timeit("gate+up with SwiGLU", gate_up_only, n, 2 * F * E * 2)
    total += _timeit("down product (partial sums left)", down_only, n, F * E * 2)
    layer_bytes = ((H + 2 * K) * D * E + H * D * E + 3 * F * E) * 2
    print(f"sum of the kernels of a layer: {total:.1f} us; its weights: {layer_bytes / 1e6:.0f} MB")
    settle()
    _timeit("the layer as the engine runs it", lambda i: blocks[i % C].forward(ctx, x, view(i), True), max(8, n // 2),
            layer_bytes + B * a.context * K * D * 4)
    settle()

    # once per step: LM head, token selection
    logits = eng.logits[:B]
    hr = ctx.buf("h_rows", E)
    _timeit("final norm + LM head", lambda i: eng.model.logits_of(ctx, ctx.want_rows, B, logits), 8, V * E * 2)
    _timeit("argmax", lambda i: eng.sampler.argmax(logits, B), 16)
    eng.sampler.load_state(SamplingParams(), list(range(B)), [0] * B, None)
    logits.copy_(torch.randn(B, V, device=eng.device) * 3)
    _timeit("sample (default options)", lambda i: eng.sampler.sample_resident(logits), 10)
    eng.check_status()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
