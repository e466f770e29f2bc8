"""Python faces of the CUDA kernels.

Each function checks what the kernel cannot check (devices, dtypes,
contiguity, sizes), passes raw pointers and the current stream to the C entry
point and raises `KernelError` with the library's message on failure.  There
is no fallback: without the compiled library, or off the GPU, these raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
GEMM_STORE, GEMM_ACCUMULATE, GEMM_SWIGLU = 0, 1, 2


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream of the current device, as the launches take it (the stream object
    of torch costs several microseconds to make, and a step makes hundreds of launches)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch._C._cuda_getDevice()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


LAUNCHES = 0      # kernel launches made through this module (a claim bench.py reports)


def _call(libname: str, fn: str, *args, launches: int = 1):
    global LAUNCHES
    LAUNCHES += launches
    lib = _build._loaded.get(libname) or _build.load(libname)
    rc = getattr(lib, fn)(*args)
    if rc != 0:
        raise KernelError(lib.mdma_last_error().decode(errors="replace"))


_i = ctypes.c_int
_f = ctypes.c_float


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(table, ids, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous()
    n = ids.numel()
    assert out.shape[0] >= n and out.shape[1] == table.shape[1] and out.is_contiguous()
    _call("core", "mdma_embed_rows", _ptr(table), _i(dtype_code(table.dtype)), _ptr(ids), _ptr(out),
          _i(n), _i(table.shape[1]), _i(table.shape[0]), _stream())


def fill_normal(out: torch.Tensor, key: int, table: torch.Tensor, std: float) -> None:
    """out.flat[i] = std * (a normal quantile picked by a hash of (key, i)); the host side of the same
    arithmetic is `weights.random_init.normal_values`.  `table`: 65,537 float quantiles on the device."""
    _need_cuda(out, table)
    assert out.is_contiguous() and table.dtype == torch.float32 and table.numel() == 65537
    _call("core", "mdma_fill_normal", _ptr(out), _i(dtype_code(out.dtype)), ctypes.c_long(out.numel()),
          ctypes.c_ulonglong(key & ((1 << 64) - 1)), _ptr(table), _f(std), _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
            partial: Optional[torch.Tensor] = None, splits: int = 0, split_stride: int = 0) -> None:
    """out[i] = rmsnorm(x[rows[i]] or x[i]) * w; x is the float residual stream.  With
    `partial` [splits, rows, width] the rows of x are first completed: x += sum of the partials."""
    _need_cuda(x, w, out, rows)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    width = x.shape[-1]
    assert w.numel() == width and out.shape[-1] == width
    n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert out.shape[0] >= n
    if rows is not None:
        assert rows.dtype == torch.int32
    _call("core", "mdma_rmsnorm", _ptr(x), _ptr(w), _i(dtype_code(w.dtype)), _ptr(rows), _ptr(out),
          _i(dtype_code(out.dtype)), _i(n), _i(width), _f(eps), _ptr(partial), _i(splits if partial is not None else 0),
          ctypes.c_long(split_stride), _stream())


ACT_SILU, ACT_GELU_TANH = 0, 1
ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH}


def ending_args(n_features: int, bias: Optional[torch.Tensor], bias2: Optional[torch.Tensor], act: int):
    """The four arguments by which the product kernels take their bias vectors and the gate's activation."""
    for b in (bias, bias2):
        if b is not None:
            assert b.is_cuda and b.is_contiguous() and b.shape == (n_features,)
            assert bias.dtype == b.dtype and b.dtype in (torch.float32, torch.bfloat16)
    assert bias2 is None or bias is not None
    return _ptr(bias), _ptr(bias2), _i(dtype_code(bias.dtype) if bias is not None else F32), _i(act)


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = GEMM_STORE,
              w2: Optional[torch.Tensor] = None, m: Optional[int] = None, bias: Optional[torch.Tensor] = None,
              bias2: Optional[torch.Tensor] = None, act: int = ACT_SILU) -> None:
    """out[:m] (=, +=) a[:m] @ w.T (+ bias) on the CUDA cores; the gated mode takes gate=w, up=w2 and
    gives act(gate) * up."""
    _need_cuda(a, w, out, w2)
    assert a.dim() == 2 and w.dim() == 2 and out.dim() == 2
    assert a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
    M = a.shape[0] if m is None else m
    N, K = w.shape
    assert a.shape[1] == K and out.shape[1] == N and out.shape[0] >= M and a.shape[0] >= M
    if w2 is not None:
        assert w2.shape == w.shape and w2.dtype == w.dtype and w2.is_contiguous()
    _call("core", "mdma_gemm_simt", _i(mode), _ptr(a), _i(dtype_code(a.dtype)), _i(a.stride(0)),
          _ptr(w), _ptr(w2), _i(dtype_code(w.dtype)), _ptr(out), _i(dtype_code(out.dtype)),
          _i(out.stride(0)), _i(M), _i(N), _i(K), *ending_args(N, bias, bias2, act), _stream())


def rope_cache_write(qkv: torch.Tensor, n_tokens: int, tok_seq, tok_pos, seq_slot, inv_freq,
                     k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                     page_table: Optional[torch.Tensor], max_pages: int, page_size: int,
                     n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                     interleaved: bool, write_kv: bool, partial: Optional[torch.Tensor] = None,
                     splits: int = 0, split_stride: int = 0) -> None:
    """Rotate q (in place) and k, write k and v to the cache.  With `partial`
    [splits, tokens, row width] floats the projection row is their sum instead of qkv's content."""
    _need_cuda(qkv, tok_seq, tok_pos, seq_slot, inv_freq, k_cache, v_cache, page_table)
    assert qkv.stride(1) == 1 and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2
    if write_kv:
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
        assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    _call("core", "mdma_rope_cache_write", _ptr(qkv), _i(dtype_code(qkv.dtype)), _i(qkv.stride(0)),
          _ptr(partial), _i(splits if partial is not None else 0), ctypes.c_long(split_stride),
          _i(qkv.shape[1]), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot), _ptr(inv_freq), _ptr(k_cache), _ptr(v_cache),
          _ptr(page_table), _i(max_pages), _i(page_size),
          _i(n_tokens), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(rotary_dim), _i(int(interleaved)),
          _i(int(write_kv)), _stream())


def attention_simple(q: torch.Tensor, n_tokens: int, k_cache, v_cache, tok_seq, tok_pos, seq_slot,
                     page_table: torch.Tensor, max_pages: int, page_size: int,
                     out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                     window: int, scale: float) -> None:
    """q: rows of the fused projection (first n_heads*head_dim columns are the queries)."""
    _need_cuda(q, k_cache, v_cache, tok_seq, tok_pos, seq_slot, out, page_table)
    assert q.stride(1) == 1 and out.is_contiguous() and out.dtype == q.dtype == k_cache.dtype
    assert out.shape[1] == n_heads * head_dim and out.shape[0] >= n_tokens
    _call("core", "mdma_attention_simple", _ptr(q), _i(dtype_code(q.dtype)), _i(q.stride(0)),
          _ptr(k_cache), _ptr(v_cache), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_slot),
          _ptr(page_table), _i(max_pages), _i(page_size), _ptr(out),
          _i(n_tokens), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(window),
          _f(scale), _stream())


_argmax_scratch: dict = {}


def argmax_scratch_words(n_rows: int, vocab: int) -> int:
    return 3 * max(n_rows, 1) * (-(-vocab // 4096))


def argmax(logits: torch.Tensor, tokens: torch.Tensor, flags: Optional[torch.Tensor] = None,
           n_rows: Optional[int] = None, scratch: Optional[torch.Tensor] = None) -> None:
    """tokens[r] = index of the largest logit of row r (the lowest index among equals);
    flags[r] = 1 if the row holds a value that is not finite.  `scratch`: floats for the first
    stage's partial results (`argmax_scratch_words`); without it a buffer of this module is used."""
    _need_cuda(logits, tokens, flags, scratch)
    assert logits.dtype == torch.float32 and logits.is_contiguous() and tokens.dtype == torch.int32
    n = logits.shape[0] if n_rows is None else n_rows
    need = argmax_scratch_words(n, logits.shape[1])
    if scratch is not None:
        if scratch.numel() < need:
            raise KernelError(f"argmax needs {need} words of scratch, {scratch.numel()} given")
    else:
        scratch = _argmax_scratch.get(logits.device.index)
    if scratch is None or scratch.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("argmax scratch cannot grow during graph capture")
        scratch = _argmax_scratch[logits.device.index] = torch.empty(max(need, 1 << 16), dtype=torch.float32,
                                                                     device=logits.device)
    _call("core", "mdma_argmax", _ptr(logits), _i(n), _i(logits.shape[1]), _ptr(tokens), _ptr(flags),
          _ptr(scratch), ctypes.c_long(scratch.numel()), _stream(), launches=2)


def sample_scratch_words(n_rows: int, vocab: int) -> int:
    """Floats of scratch `sample` needs: exponentials, candidate probabilities and candidate ids of every row."""
    return 3 * n_rows * vocab


def sample(logits: torch.Tensor, uniforms: Optional[torch.Tensor], tokens: torch.Tensor, probs_scratch: torch.Tensor,
           temperature: float, top_p: float, min_p: float, penalty: float, penalty_window: int,
           history: Optional[torch.Tensor] = None, history_len: Optional[torch.Tensor] = None,
           flags: Optional[torch.Tensor] = None, n_rows: Optional[int] = None, impl: int = 0,
           requests: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None, seed: int = 0,
           advance: bool = False, dev_params: Optional[torch.Tensor] = None) -> None:
    """One token per row of `logits`.  The uniform number of a row is `uniforms[r]`, or, without
    `uniforms`, made on the device from (seed, requests[r], steps[r]).  `history` [rows, cap] is a ring of
    recent token ids per row and `history_len` the count of tokens ever added to it.  `advance`: the
    kernel appends the selected token to the ring and adds one to `steps`.
    `impl`: 0 picks (a cluster of eight blocks per row when the row fits), 1 one block per row, 2 the cluster.
    `dev_params` (eight 32-bit words on the device: temperature, top_p, min_p, penalty as floats, the
    window, an unused word, the seed's low and high halves) replaces the options given by value, so that
    a captured launch serves whatever the host writes there before a replay."""
    _need_cuda(logits, uniforms, tokens, probs_scratch, history, history_len, flags, requests, steps, dev_params)
    assert dev_params is None or (dev_params.dtype == torch.int32 and dev_params.numel() >= 8)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert tokens.dtype == torch.int32 and (uniforms is None or uniforms.dtype == torch.float32)
    assert uniforms is not None or (requests is not None and steps is not None)
    assert requests is None or (requests.dtype == torch.int32 and steps.dtype == torch.int32)
    n = logits.shape[0] if n_rows is None else n_rows
    assert probs_scratch.dtype == torch.float32 and probs_scratch.numel() >= sample_scratch_words(n, logits.shape[1])
    hstride = 0
    if history is not None:
        assert history.dtype == torch.int32 and history_len.dtype == torch.int32 and history.is_contiguous()
        hstride = history.shape[1]
    _call("core", "mdma_sample", _ptr(logits), _i(n), _i(logits.shape[1]), _ptr(history),
          _ptr(history_len), _i(hstride), _ptr(uniforms), _ptr(requests), _ptr(steps),
          ctypes.c_ulonglong(seed & ((1 << 64) - 1)), _i(int(advance)), _f(temperature), _f(top_p), _f(min_p),
          _f(penalty), _i(penalty_window), _ptr(probs_scratch), ctypes.c_long(probs_scratch.numel()), _ptr(tokens),
          _ptr(flags), _i(impl), _ptr(dev_params), _stream())


def advance_decode(tokens: torch.Tensor, ids: torch.Tensor, tok_pos: torch.Tensor, seq_pos0: torch.Tensor,
                   n: int, ring: Optional[torch.Tensor] = None, counter: Optional[torch.Tensor] = None) -> None:
    """ids <- tokens, positions += 1: what a decode step leaves for the next one.  With `ring`
    [rows, words] the first `words` integers at `tokens` (tokens, flags and what lies behind them in
    the same buffer) are also kept in row counter % rows, and the counter moves on."""
    _need_cuda(tokens, ids, tok_pos, seq_pos0, ring, counter)
    words, rows = (ring.shape[1], ring.shape[0]) if ring is not None else (0, 0)
    assert ring is None or (ring.dtype == torch.int32 and ring.is_contiguous() and counter.dtype == torch.int32)
    _call("core", "mdma_advance_decode", _ptr(tokens), _ptr(ids), _ptr(tok_pos), _ptr(seq_pos0), _i(n),
          _i(words), _ptr(ring), _i(rows), _ptr(counter), _stream())
