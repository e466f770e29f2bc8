"""Times of the decode step's kernels one by one, at the sizes of a configuration.

    python -m mdma_b200.kernel_times [--batch 8] [--context 580] [--hidden 4096] [--intermediate 14336]
                                     [--heads 32] [--kv-heads 8] [--head-dim 128] [--vocab 128256]

Every kernel is captured `--repeat` times in a CUDA graph and timed with CUDA events around two replays
(steady state, no launch gaps from the host).  Weights and caches rotate through several copies so that
the 126 MB L2 does not serve them.  The sizes default to the Llama-3.1-8B layer.  The numbers under
`profiles/` that name this module were made with it.
"""
from __future__ import annotations

import argparse

import torch

from . import ops, ops_tensor


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
    print(f"{name:34s} {us:9.2f} us" + (f"  {nbytes / us / 1e3:7.0f} GB/s" if nbytes else ""), flush=True)
    return us


class _Meta:
    """What the attention and rotary kernels read of a decode step: one new token per sequence."""

    def __init__(self, batch: int, context: int, dev):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        self.n_seqs = self.n_tokens = batch
        self.max_new, self.max_len = 1, context
        self.seq_start = i32(list(range(batch + 1)))
        self.seq_pos0 = i32([context - 1] * batch)
        self.seq_slot = i32(list(range(batch)))
        self.tok_seq = i32(list(range(batch)))
        self.tok_pos = i32([context - 1] * batch)


class _View:
    pass


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=580)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=14336)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--copies", type=int, default=6, help="copies of weights and cache that take turns")
    ap.add_argument("--repeat", type=int, default=48)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    B, E, F, H, K, D, V, C = a.batch, a.hidden, a.intermediate, a.heads, a.kv_heads, a.head_dim, a.vocab, a.copies
    qkv_w = (H + 2 * K) * D

    def weights(n, k):
        return [(torch.randn(n, k, device=dev) * 0.02).bfloat16() for _ in range(C)]
    w_qkv, w_o, w_gate, w_up, w_down = weights(qkv_w, E), weights(E, H * D), weights(F, E), weights(F, E), weights(E, F)
    h = torch.randn(B, E, device=dev).bfloat16()
    x = torch.randn(B, E, device=dev)
    qkv = torch.zeros(B, qkv_w, device=dev, dtype=torch.bfloat16)
    attn_out = torch.zeros(B, H * D, device=dev, dtype=torch.bfloat16)
    act = torch.zeros(B, F, device=dev, dtype=torch.bfloat16)
    norm_w = torch.ones(E, device=dev, dtype=torch.bfloat16)
    page = 64
    n_pages = -(-(a.context + 64) // page)
    k_cache = torch.randn(C, B * n_pages, page, K, D, device=dev).bfloat16()
    v_cache = torch.randn_like(k_cache)
    table = torch.arange(B * n_pages, dtype=torch.int32, device=dev).reshape(B, n_pages)
    meta = _Meta(B, a.context, dev)
    inv_freq = torch.ones(D // 2, device=dev)

    def view(i):
        v = _View()
        v.k, v.v, v.page_table, v.max_pages, v.page_size = k_cache[i], v_cache[i], table, n_pages, page
        return v

    def pending(t, mode):
        return ops_tensor.take_pending(t, mode, B) or (None, 0, 0)

    def rope(i, part):
        ops.rope_cache_write(qkv, B, meta.tok_seq, meta.tok_pos, meta.seq_slot, inv_freq, k_cache[i], v_cache[i],
                             table, n_pages, page, H, K, D, D, False, True, part[0], part[1], part[2])

    scale = 1.0 / D ** 0.5
    n = a.repeat
    total = 0.0
    total += _timeit("QKV product (partials deferred)", lambda i: (ops_tensor.gemm(h, w_qkv[i % C], qkv, 0, None, B, defer=True), pending(qkv, 0)), n, w_qkv[0].numel() * 2)
    total += _timeit("rotary + cache write", lambda i: rope(i % C, (None, 0, 0)), n)
    total += _timeit("attention", lambda i: ops_tensor.attention(meta, qkv, view(i % C), attn_out, H, K, D, 0, scale), n, B * a.context * K * D * 2 * 2)
    total += _timeit("O product (partials deferred)", lambda i: (ops_tensor.gemm(attn_out, w_o[i % C], x, 1, None, B, defer=True), pending(x, 1)), n, w_o[0].numel() * 2)
    total += 2 * _timeit("RMSNorm", lambda i: ops.rmsnorm(x, norm_w, 1e-5, h, None, B), n)
    total += _timeit("gate+up with SwiGLU", lambda i: ops_tensor.gemm(h, w_gate[i % C], act, 2, w_up[i % C], B), n, 2 * w_gate[0].numel() * 2)
    total += _timeit("down product (partials deferred)", lambda i: (ops_tensor.gemm(act, w_down[i % C], x, 1, None, B, defer=True), pending(x, 1)), n, w_down[0].numel() * 2)
    layer_bytes = (w_qkv[0].numel() + w_o[0].numel() + 3 * w_gate[0].numel()) * 2
    print(f"sum of the kernels of a layer: {total:.1f} us; its weights: {layer_bytes / 1e6:.0f} MB")

    def layer(i):
        j = i % C
        ops.rmsnorm(x, norm_w, 1e-5, h, None, B)
        ops_tensor.gemm(h, w_qkv[j], qkv, 0, None, B, defer=True)
        rope(j, pending(qkv, 0))
        ops_tensor.attention(meta, qkv, view(j), attn_out, H, K, D, 0, scale)
        ops_tensor.gemm(attn_out, w_o[j], x, 1, None, B, defer=True)
        part = pending(x, 1)
        ops.rmsnorm(x, norm_w, 1e-5, h, None, B, part[0], part[1], part[2])
        ops_tensor.gemm(h, w_gate[j], act, 2, w_up[j], B)
        ops_tensor.gemm(act, w_down[j], x, 1, None, B, defer=True)
        part = pending(x, 1)
        ops.rmsnorm(x, norm_w, 1e-5, h, None, B, part[0], part[1], part[2])
    _timeit("the kernels of a layer as a chain", layer, max(8, n // 2))

    # once per step: LM head, token selection
    logits = torch.zeros(B, V, device=dev)
    tokens = torch.zeros(B, dtype=torch.int32, device=dev)
    flags = torch.zeros_like(tokens)
    w_head = [(torch.randn(V, E, device=dev) * 0.02).bfloat16() for _ in range(2)]
    _timeit("LM head", lambda i: ops_tensor.gemm(h, w_head[i % 2], logits, 0, None, B), 8, V * E * 2)
    _timeit("argmax", lambda i: ops.argmax(logits, tokens, flags, B), 16)
    peaked = torch.randn(B, V, device=dev) * 3
    uniforms = torch.rand(B, device=dev)
    scratch = torch.empty(ops.sample_scratch_words(B, V), device=dev)
    history = torch.randint(0, V, (B, 64), dtype=torch.int32, device=dev)
    history_len = torch.full((B,), 64, dtype=torch.int32, device=dev)
    for name, rows, (temp, top_p, min_p, pen) in (
            ("sample, defaults, peaked logits", peaked, (0.8, 0.95, 0.05, 1.1)),
            ("sample, temperature only", peaked, (0.8, 1.0, 0.0, 1.0)),
            ("sample, top-p 0.9 only", peaked, (0.8, 0.9, 0.0, 1.0)),
            ("sample, defaults, flat logits", peaked * (0.05 / 3), (0.8, 0.95, 0.05, 1.1))):
        _timeit(name, lambda i: ops.sample(rows, uniforms, tokens, scratch, temp, top_p, min_p, pen, 64, history,
                                           history_len, flags), 10)
    ops_tensor.check_status(dev)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
