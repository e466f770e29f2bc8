"""Python faces of the tensor-core kernels (bfloat16 only): the tcgen05 matrix
product and the fast attention kernels.  As in `ops`, nothing here falls back:
a shape the kernels refuse raises `KernelError`."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import ops
from .csrc import build as _build
from .ops import KernelError, _call, _f, _i, _need_cuda, _ptr, _stream

# MDMA_EVEN_SPLIT=0: the block-pair GEMM gives every pair whole tiles only (for comparisons).
EVEN_SPLIT = os.environ.get("MDMA_EVEN_SPLIT", "1") != "0"

FORCED_ATTENTION = os.environ.get("MDMA_ATTN")        # "tc" or "mma": one attention kernel for every step (comparisons)

PAIR_TOKENS = 96         # steps of more tokens than this may run a product on the block-pair kernel (the gated one from 97)


def pair_scratch_floats(sms: int) -> int:
    """Partial tiles of the block-pair kernel's even K-block split: one per block, two accumulators."""
    return sms * 2 * 256 * 128


def scratch_floats_bound(sms: int, max_tokens: int, max_seqs: int, attention_shapes=()) -> int:
    """An upper bound of the scratch any step of up to `max_tokens` tokens in up to `max_seqs`
    sequences needs, from sizes alone (an engine reserves this much once and never grows it).
    K-split products keep splits x tokens x features floats with splits x tiles <= 2 x SMs, tiles of
    128 features x up to 64 tokens (one per SM for 128 tokens); attention keeps tokens x heads x
    splits x (head_dim + 2) floats.  `attention_shapes`: (heads, kv heads, head_dim) of each mixer."""
    del max_seqs          # the bounds below hold for any number of sequences
    need = 2 * sms * 128 * 64
    if max_tokens > PAIR_TOKENS:
        need = max(need, pair_scratch_floats(sms))
    products, need = need, 0          # a projection's partial sums and the attention's can be alive together
    for heads, kv_heads, head_dim in attention_shapes:
        group = max(1, heads // max(kv_heads, 1))
        # Keys are split only while the grid is short of blocks (see `attention_splits`): decode has
        # sequences x kv heads blocks < 2 x SMs and splits <= 3 x SMs / blocks + 1, so tokens x splits
        # < 5 x SMs / kv heads; other steps have tokens <= blocks x tile tokens / kv heads and
        # splits <= 2 x SMs / blocks + 1, so tokens x splits < 4 x SMs x tile tokens / kv heads.
        tile_tokens = max(1, 64 // group)
        need = max(need, 5 * sms * group * (head_dim + 2), 4 * sms * tile_tokens * group * (head_dim + 2))
    return products + need + 64


class TensorState:
    """What the tensor-core kernels share between launches on one device: a status word their
    bounded waits set, the flags of the block-pair kernel's even split, scratch for partial sums,
    and the record of a K-split product whose partial sums still wait to be added up.  An engine
    owns one, carved from its arena and never reallocated (captured graphs hold its addresses);
    kernels called without one (tests, tools) share a per-device default that may grow."""

    def __init__(self, device: torch.device, scratch_floats: int, sms: Optional[int] = None,
                 status: Optional[torch.Tensor] = None, sk_flags: Optional[torch.Tensor] = None,
                 scratch: Optional[torch.Tensor] = None, growable: bool = False):
        self.device = device
        self.sms = sms if sms is not None else torch.cuda.get_device_properties(device).multi_processor_count
        zeros = lambda n, dtype: torch.zeros(n, dtype=dtype, device=device)
        self.status = status if status is not None else zeros(4, torch.int32)
        self.sk_flags = sk_flags if sk_flags is not None else zeros(max(512, 4 * self.sms), torch.int32)
        self.scratch = scratch if scratch is not None else zeros(max(scratch_floats, 1), torch.float32)
        self.pending: Optional[Pending] = None
        self.growable = growable

    def need(self, floats: int, what: str) -> None:
        if floats <= self.scratch.numel():
            return
        if not self.growable:
            raise KernelError(f"{what} needs {floats} floats of scratch, the engine reserved {self.scratch.numel()}")
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"{what}: scratch is too small and cannot grow during graph capture")
        self.scratch = torch.empty(floats, dtype=torch.float32, device=self.device)

    def clear(self) -> None:
        """After a wait ran out: reset the status word and the flags a block pair may have left standing."""
        self.status.zero_()
        self.sk_flags.zero_()
        self.pending = None


_default: dict = {}


def _device_state(device: torch.device) -> TensorState:
    st = _default.get(device.index)
    if st is None:
        st = _default[device.index] = TensorState(device, 1 << 20, growable=True)
    return st


def check_status(device: torch.device, st: Optional[TensorState] = None) -> None:
    """Raise if a tensor-core kernel gave up on a wait since the last check (synchronises)."""
    st = st or _default.get(device.index)
    if st is not None and int(st.status[0].item()) != 0:
        st.clear()
        raise KernelError("a tensor-core kernel ran into its wait limit; its output is not valid")


def gemm_supported(n_features: int, k: int) -> bool:
    return k % 8 == 0 and k >= 8


_plans: dict = {}


def gemm_plan(mode: int, n_tokens: int, n_features: int, k: int, sms: int) -> tuple[int, int]:
    """(token tile, K splits) the library chooses for a product of these sizes (kept: a step asks
    for the same few products hundreds of times)."""
    key = (mode, n_tokens, n_features, k, sms)
    plan = _plans.get(key)
    if plan is None:
        if len(_plans) > 4096:
            _plans.clear()
        plan = _plans[key] = _gemm_plan(*key)
    return plan


def _gemm_plan(mode: int, n_tokens: int, n_features: int, k: int, sms: int) -> tuple[int, int]:
    lib = _build.load("tensor")
    bn, splits = ctypes.c_int(0), ctypes.c_int(0)
    lib.mdma_gemm_tc_plan(_i(mode), _i(n_tokens), _i(n_features), _i(k), _i(sms),
                          ctypes.byref(bn), ctypes.byref(splits))
    return bn.value, splits.value


def gemm_scratch_floats(bn: int, splits: int, m: int, n: int, sms: int) -> int:
    """Floats of scratch a product of m tokens x n features needs with this token tile and K split: the partial
    sums of a split through global memory, or the partial tiles of the block-pair kernel (`bn` 512)."""
    if bn == 512:
        return pair_scratch_floats(sms)
    return splits * m * n if splits > 1 else 0


class Pending:
    """Partial sums of a K-split product that still wait in the scratch to be added
    up into (or onto) `target`: [splits, rows, cols] floats."""
    __slots__ = ("target_ptr", "target", "mode", "splits", "rows", "cols")

    def __init__(self, target, mode, splits, rows, cols):
        self.target, self.target_ptr = target, target.data_ptr()
        self.mode, self.splits, self.rows, self.cols = mode, splits, rows, cols


def flush_pending(device: torch.device, st: Optional[TensorState] = None) -> None:
    """Finish a deferred K-split reduction with the plain reduce kernel."""
    st = st or _default.get(device.index)
    if st is None or st.pending is None:
        return
    pend, st.pending = st.pending, None
    out = pend.target
    _call("tensor", "mdma_splitk_reduce", _i(pend.mode), _ptr(st.scratch), _i(pend.splits), _i(pend.rows),
          _i(pend.cols), _ptr(out), _i(out.stride(0)), _i(int(out.dtype == torch.float32)), _stream())


def take_pending(target: torch.Tensor, mode: int, rows: int, st: Optional[TensorState] = None):
    """If partial sums for exactly this target wait in the scratch, hand them to the caller, who
    will add them up itself: returns (scratch, splits, floats per split) or None."""
    st = st or _default.get(target.device.index)
    if st is None or st.pending is None:
        return None
    pend = st.pending
    if (pend.target_ptr != target.data_ptr() or pend.mode != mode or pend.rows != rows
            or pend.cols != target.shape[1] or target.stride(0) != pend.cols):
        return None
    st.pending = None
    return st.scratch, pend.splits, pend.rows * pend.cols


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = ops.GEMM_STORE,
         w2: Optional[torch.Tensor] = None, m: Optional[int] = None,
         bn: Optional[int] = None, splits: Optional[int] = None, defer: bool = False,
         st: Optional[TensorState] = None, bias: Optional[torch.Tensor] = None,
         bias2: Optional[torch.Tensor] = None, act: int = ops.ACT_SILU) -> None:
    """out[:m] (=, +=) a[:m] @ w.T (+ bias) on the tensor cores; the gated mode takes gate=w, up=w2 and
    gives act(gate) * up.
    `defer`: if the product is split over K, leave its partial sums for the next kernel
    (a norm or the rotary write) to add up; see `take_pending`.  `st`: the engine's state."""
    _need_cuda(a, w, out, w2)
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the tensor-core product takes bfloat16 operands")
    assert a.dim() == 2 and w.dim() == 2 and a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
    M = a.shape[0] if m is None else m
    N, K = w.shape
    assert a.shape[1] == K and out.shape[1] == N and out.shape[0] >= M and a.shape[0] >= M
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"output dtype {out.dtype} is not supported")
    st = st or _device_state(a.device)
    flush_pending(a.device, st)
    if bn is None or splits is None:
        pbn, psplits = gemm_plan(mode, M, N, K, st.sms)
        bn = bn or pbn
        splits = splits or psplits
    st.need(gemm_scratch_floats(bn, splits, M, N, st.sms), "a K-split product")
    used = ctypes.c_int(1)
    _call("tensor", "mdma_gemm_tc", _i(mode), _ptr(a), _i(a.stride(0)), _ptr(w), _ptr(w2), _ptr(out),
          _i(int(out.dtype == torch.float32)), _i(out.stride(0)), _i(M), _i(N), _i(K), _i(bn), _i(splits),
          _ptr(st.scratch), ctypes.c_long(st.scratch.numel()), _ptr(st.status),
          _i(int(defer)), ctypes.byref(used), _ptr(st.sk_flags) if EVEN_SPLIT else None,
          *ops.ending_args(N, bias, bias2, act), _stream(),
          launches=2 if (splits > 1 and not defer) else 1)
    if defer and used.value > 1:
        st.pending = Pending(out, mode, used.value, M, N)


def attention_supported(n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    return (n_kv_heads > 0 and n_heads % n_kv_heads == 0 and head_dim % 16 == 0 and 16 <= head_dim <= 128
            and n_heads // n_kv_heads <= 64)


def attention_splits(n_seqs: int, max_new: int, max_len: int, n_heads: int, n_kv_heads: int, sms: int,
                     most_seqs: Optional[int] = None) -> int:
    """How many ways to divide a tile's keys so that the grid fills the device.  `most_seqs`: the most
    sequences the engine can hold; the choice for a handful of sequences is made from it, not from the
    live batch, so that a request's arithmetic does not change when a batch mate ends."""
    group = n_heads // n_kv_heads
    key_blocks = max(1, -(-max_len // 64))
    if max_new == 1 and group <= 16:
        # decode kernel: a block's warps each take 32-key tiles in turn.  One block of eight warps per
        # (sequence, kv head) and no merge kernel, unless that leaves most of the device idle:
        #  - an engine for a handful of sequences (their blocks x 4 within three quarters of the SMs): four blocks per
        #    (sequence, kv head), six for long contexts; a round of tiles costs a block about 1.3 us and a
        #    merge kernel about as much (measured in the layer chain at the 8B shape, context 580: batch 1
        #    94.1 -> 89.9 us, batch 2 95.0 -> 91.2, batch 3 93.8 -> 92.3, batch 4 no gain);
        #  - contexts beyond 1,024 with fewer blocks than SMs: as many splits as keep every block resident
        #    with four warps (three blocks per SM).
        # The choice is made from the context rounded up to 1,024, as the replayed decode graphs see it, so
        # that a step run on its own and the same step replayed add up in the same order.
        max_len = -(-max_len // 1024) * 1024
        blocks = n_seqs * n_kv_heads
        if blocks >= sms:
            return 1
        few = (most_seqs or n_seqs) * n_kv_heads * 4 <= (3 * sms) // 4
        if max_len <= 1024:
            return 4 if few else 1
        if few:
            return 6
        rounds = -(-max_len // (32 * 4))           # four warps x 32 keys per round
        return max(2, min(3 * sms // blocks, rounds, 32))
    tile_tokens = max(1, 64 // group)
    blocks = -(-max_new // tile_tokens) * n_seqs * n_kv_heads
    if blocks >= 2 * sms:
        return 1
    return max(1, min(-(-2 * sms // blocks), key_blocks, 32))


def attention_tc_supported(n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return (attention_supported(n_heads, n_kv_heads, head_dim) and n_heads // n_kv_heads <= 128
            and page_size % 64 == 0)


def attention(ctx, qkv: torch.Tensor, view, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
              window: int, scale: float, splits: Optional[int] = None, impl: Optional[str] = None,
              st: Optional[TensorState] = None) -> None:
    """Causal grouped-query attention of the step's tokens over the paged cache (bfloat16).
    Steps that bring many tokens per sequence run on the tcgen05 kernel, single tokens on the
    decode kernel, what is between (or outside the tcgen05 kernel's limits) on the mma.sync kernel;
    `impl` ("tc" or "mma") forces one."""
    group = n_heads // n_kv_heads
    if impl is None and FORCED_ATTENTION:
        impl = FORCED_ATTENTION
    if impl is None:
        impl = "tc" if (ctx.max_new * group > 64 and splits is None
                        and attention_tc_supported(n_heads, n_kv_heads, head_dim, view.page_size)) else "mma"
    if impl == "tc":
        _need_cuda(qkv, view.k, view.v, out, view.page_table)
        if qkv.dtype != torch.bfloat16 or view.k.dtype != torch.bfloat16:
            raise KernelError("the tensor-core attention takes bfloat16")
        assert qkv.stride(1) == 1 and out.is_contiguous() and out.shape[1] == n_heads * head_dim
        assert view.k.is_contiguous() and view.v.is_contiguous()
        st = st or _device_state(qkv.device)
        flush_pending(qkv.device, st)
        _call("tensor", "mdma_attention_tc", _ptr(qkv), _i(qkv.stride(0)), _i(qkv.shape[0]), _ptr(view.k),
              _ptr(view.v), _i(view.k.shape[0]), _ptr(ctx.seq_start), _ptr(ctx.seq_pos0), _ptr(ctx.seq_slot),
              _ptr(view.page_table), _i(view.max_pages), _i(view.page_size), _ptr(out), _i(ctx.n_tokens),
              _i(ctx.n_seqs), _i(ctx.max_new), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(window), _f(scale),
              _ptr(st.status), _stream())
        return
    _need_cuda(qkv, view.k, view.v, out, view.page_table)
    if qkv.dtype != torch.bfloat16 or view.k.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention takes bfloat16")
    assert qkv.stride(1) == 1 and out.is_contiguous() and out.shape[1] == n_heads * head_dim
    st = st or _device_state(qkv.device)
    flush_pending(qkv.device, st)
    if splits is None:
        splits = attention_splits(ctx.n_seqs, ctx.max_new, ctx.max_len, n_heads, n_kv_heads, st.sms,
                                  getattr(ctx, "most_seqs", None))
    st.need(ctx.n_tokens * n_heads * splits * (head_dim + 2) if splits > 1 else 0, "attention over split keys")
    _call("tensor", "mdma_attention_mma_paged", _ptr(qkv), _i(qkv.stride(0)), _ptr(view.k), _ptr(view.v),
          _i(view.k.shape[0] if view.k.is_contiguous() and view.v.is_contiguous() else 0), _ptr(ctx.seq_start), _ptr(ctx.seq_pos0), _ptr(ctx.seq_slot), _ptr(view.page_table),
          _i(view.max_pages), _i(view.page_size), _ptr(out), _i(ctx.n_tokens), _i(ctx.n_seqs),
          _i(ctx.max_new), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(window), _f(scale), _i(splits),
          _ptr(st.scratch), ctypes.c_long(st.scratch.numel()), _ptr(st.status), _stream(),
          launches=2 if splits > 1 else 1)


def fused_rotary_supported(n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, rotary_dim: int) -> bool:
    """Whether single-token steps of this geometry can rotate q and k and write the cache inside the
    attention kernel (`attention_decode_rotary`)."""
    return (attention_supported(n_heads, n_kv_heads, head_dim) and n_heads // n_kv_heads <= 16
            and page_size % 32 == 0 and rotary_dim % 2 == 0 and 2 <= rotary_dim <= head_dim)


def attention_decode_rotary(ctx, qkv: torch.Tensor, view, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                            head_dim: int, window: int, scale: float, inv_freq: torch.Tensor, rotary_dim: int,
                            interleaved: bool, splits: Optional[int] = None, st: Optional[TensorState] = None) -> None:
    """A step of one token per sequence: the projection rows `qkv` (or the K-split partial sums a
    deferred product left for them) are rotated, the keys and values written to the cache and the
    attention computed by ONE kernel; it asks for all its key and value tiles before it waits for
    the projection, because it takes the token's own key and value from registers, not from the cache."""
    _need_cuda(qkv, view.k, view.v, out, view.page_table, inv_freq)
    if qkv.dtype != torch.bfloat16 or view.k.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention takes bfloat16")
    assert qkv.stride(1) == 1 and out.is_contiguous() and out.shape[1] == n_heads * head_dim
    assert view.k.is_contiguous() and view.v.is_contiguous() and inv_freq.dtype == torch.float32
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim and ctx.max_new == 1
    st = st or _device_state(qkv.device)
    pend = take_pending(qkv, ops.GEMM_STORE, ctx.n_tokens, st)
    partial, proj_splits, stride = (None, 0, 0)
    if pend is not None:
        partial, proj_splits, stride = pend
    else:
        flush_pending(qkv.device, st)
    if splits is None:
        splits = attention_splits(ctx.n_seqs, 1, ctx.max_len, n_heads, n_kv_heads, st.sms, getattr(ctx, "most_seqs", None))
    # the attention's own partials (keys split over blocks) lie behind the projection's
    used = -(-proj_splits * stride // 64) * 64
    need = ctx.n_tokens * n_heads * splits * (head_dim + 2) if splits > 1 else 0
    st.need(used + need, "attention over split keys")
    own = st.scratch[used:]
    _call("tensor", "mdma_attention_decode_rotary", _ptr(qkv), _i(qkv.stride(0)), _ptr(partial), _i(proj_splits),
          ctypes.c_long(stride), _ptr(inv_freq), _i(rotary_dim), _i(int(interleaved)), _ptr(view.k), _ptr(view.v),
          _i(view.k.shape[0]), _ptr(ctx.seq_start), _ptr(ctx.seq_pos0), _ptr(ctx.seq_slot), _ptr(view.page_table),
          _i(view.max_pages), _i(view.page_size), _ptr(out), _i(ctx.n_seqs), _i(n_heads), _i(n_kv_heads), _i(head_dim),
          _i(window), _f(scale), _i(splits), _ptr(own), ctypes.c_long(own.numel()), _ptr(st.status), _stream(),
          launches=2 if splits > 1 else 1)


def set_wait_limit(seconds: float) -> None:
    """The wall-clock limit of the bounded waits in the matrix-product kernels (2 s by default)."""
    _call("tensor", "mdma_set_wait_limit_ns", ctypes.c_ulonglong(int(seconds * 1e9)), launches=0)


def wait_probe(mode: int, flag: torch.Tensor, st: Optional[TensorState] = None) -> None:
    """Launch the kernel that only waits, on an mbarrier nobody arrives on (mode 0) or on `flag` (mode 1),
    with the product kernels' own wait routines; a wait that runs out sets the status word."""
    st = st or _device_state(flag.device)
    _call("tensor", "mdma_wait_probe", _i(mode), _ptr(flag), _ptr(st.status), _stream())
