"""Each kernel alone against a plain PyTorch float32/float64 statement of the same
operation, at sizes other than the engine tests use: tails that are no multiple
of a tile, widths and vocabularies that are no power of two, a canary after
every output."""
import math

import pytest
import torch

from plain_llama import plain_attention, plain_inv_freq, plain_rmsnorm, plain_rope, plain_sample

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops_mod():
    from mdma_b200 import ops
    return ops


def close(got, want, atol, rtol=0.0):
    got, want = got.double().cpu(), want.double().cpu()
    assert torch.isfinite(got).all(), "non-finite output"
    err = (got - want).abs()
    bound = atol + rtol * want.abs()
    assert bool((err <= bound).all()), f"max err {err.max().item():.3g} (bound {atol:.3g}+{rtol:.3g}*|x|)"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_rows(dtype):
    ops = ops_mod()
    table = torch.randn(331, 120, device=DEV).to(dtype)
    ids = torch.tensor([0, 330, 7, 7, 119], dtype=torch.int32, device=DEV)
    out = torch.full((7, 120), 9.0, device=DEV)
    ops.embed_rows(table, ids, out)
    close(out[:5], table[ids.long()].float(), 0.0)
    assert bool((out[5:] == 9.0).all())


@pytest.mark.parametrize("width", [4099, 96, 8, 4096, 12000, 20000])
@pytest.mark.parametrize("odt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
def test_rmsnorm(width, odt, wdt):
    ops = ops_mod()
    torch.manual_seed(width)
    x = torch.randn(6, width, device=DEV) * 3 + 0.5
    w = (torch.randn(width, device=DEV) * 0.5 + 1).to(wdt)
    out = torch.full((5, width), 9.0, device=DEV, dtype=odt)
    ops.rmsnorm(x, w, 3e-6, out, n_rows=4)
    want = plain_rmsnorm(x[:4].double().cpu(), w.double().cpu(), 3e-6)
    close(out[:4], want, 1e-5 if odt == torch.float32 else 0, 0 if odt == torch.float32 else 1e-2)
    assert bool((out[4:] == 9.0).all())
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    ops.rmsnorm(x, w, 3e-6, out, rows=rows)
    want = plain_rmsnorm(x[[5, 0, 5]].double().cpu(), w.double().cpu(), 3e-6)
    close(out[:3], want, 1e-5 if odt == torch.float32 else 0, 0 if odt == torch.float32 else 1e-2)


@pytest.mark.parametrize("width,splits", [(4096, 5), (120, 2), (9000, 3), (17000, 2)])
def test_rmsnorm_adds_split_partials_first(width, splits):
    """x += sum of the partial sums, then the norm of the completed row; x itself is updated."""
    ops = ops_mod()
    torch.manual_seed(width)
    T = 5
    x = torch.randn(T + 1, width, device=DEV)
    x0 = x.clone()
    partial = torch.randn(splits, T, width, device=DEV)
    w = (torch.rand(width, device=DEV) + 0.5).bfloat16()
    out = torch.full((T + 1, width), 9.0, device=DEV, dtype=torch.bfloat16)
    ops.rmsnorm(x, w, 1e-5, out, None, T, partial, splits, T * width)
    full = x0[:T].double().cpu()
    for s_ in range(splits):
        full = (full.float() + partial[s_].cpu()).double()        # float adds in split order, as the kernel does
    close(x[:T], full, 0.0)
    assert torch.equal(x[T:], x0[T:]) and bool((out[T:] == 9.0).all())
    close(out[:T], plain_rmsnorm(full, w.double().cpu(), 1e-5), 0, 1e-2)


def test_rope_reads_split_partials():
    ops = ops_mod()
    torch.manual_seed(3)
    H, K, hd, page, max_pages, T, splits = 4, 2, 32, 16, 8, 6, 3
    width = (H + 2 * K) * hd
    partial = torch.randn(splits, T, width, device=DEV)
    summed = partial.sum(0)
    inv = plain_inv_freq(hd, 1e4, None).to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    table = torch.arange(8, dtype=torch.int32, device=DEV).reshape(1, 8)
    res = []
    for use_partial in (True, False):
        qkv = torch.zeros(T, width, device=DEV, dtype=torch.bfloat16) if use_partial else summed.bfloat16()
        kc, vc = paged_cache(8, page, K, hd, torch.bfloat16)
        ops.rope_cache_write(qkv, T, i32([0] * T), i32(list(range(20, 20 + T))), i32([0]), inv, kc, vc, table,
                             max_pages, page, H, K, hd, hd, False, True,
                             partial if use_partial else None, splits, T * width)
        res.append((qkv[:, :H * hd].clone(), kc.clone(), vc.clone()))
    for a, b in zip(*res):
        close(a, b.double(), 2e-2, 1e-2)          # the partial path rounds once, the other twice
    want_q = plain_rope(summed[:, :H * hd].double().cpu().reshape(T, H, hd), torch.arange(20, 20 + T), inv.cpu(), "split_half")
    close(res[0][0].reshape(T, H, hd), want_q, 1e-2, 1e-2)


def paged_cache(n_pages, page, kvh, d, dtype):
    k = torch.zeros(n_pages, page, kvh, d, device=DEV, dtype=dtype)
    return k, torch.zeros_like(k)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout,hd,rot", [("interleaved", 48, 48), ("split_half", 80, 80), ("split_half", 64, 32)])
def test_rope_cache_write(dtype, layout, hd, rot):
    """Positions up to 30,000 with theta 1e6 (the reference's hard case,
    src/backend/cuda/tests.rs:601-647); scattered pages; partial rotary width."""
    ops = ops_mod()
    torch.manual_seed(0)
    H, K, page, max_pages = 3, 2, 16, 2048
    pos = [0, 1, 17, 30000, 29999, 5]
    seq = [0, 0, 0, 1, 1, 2]
    T = len(pos)
    qkv = torch.randn(T, (H + 2 * K) * hd, device=DEV).to(dtype)
    orig = qkv.clone()
    inv = plain_inv_freq(rot, 1e6, None).to(DEV)
    kc, vc = paged_cache(40, page, K, hd, dtype)
    table = torch.zeros(3, max_pages, dtype=torch.int32, device=DEV)
    table[0, 0], table[0, 1], table[1, 29999 // page], table[1, 30000 // page], table[2, 0] = 7, 3, 11, 30, 1
    slots = torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV)
    ops.rope_cache_write(qkv, T, torch.tensor(seq, dtype=torch.int32, device=DEV),
                         torch.tensor(pos, dtype=torch.int32, device=DEV), slots, inv, kc, vc, table,
                         max_pages, page, H, K, hd, rot, layout == "interleaved", True)
    o = orig.double().cpu().reshape(T, H + 2 * K, hd)
    p = torch.tensor(pos)
    want_q = o[:, :H].clone()
    want_k = o[:, H:H + K].clone()
    want_q[..., :rot] = plain_rope(o[:, :H, :rot], p, inv.cpu(), layout)
    want_k[..., :rot] = plain_rope(o[:, H:H + K, :rot], p, inv.cpu(), layout)
    tol = dict(atol=2e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    close(qkv.reshape(T, H + 2 * K, hd)[:, :H], want_q, **tol)
    assert torch.equal(qkv.reshape(T, H + 2 * K, hd)[:, H:], orig.reshape(T, H + 2 * K, hd)[:, H:])
    used = set()
    for t in range(T):
        pg = int(table[seq[t], pos[t] // page])
        used.add((pg, pos[t] % page))
        close(kc[pg, pos[t] % page], want_k[t], **tol)
        close(vc[pg, pos[t] % page], o[t, H + K:], 0.0)
    mask = torch.ones(40, page, dtype=torch.bool)
    for pg, r in used:
        mask[pg, r] = False
    assert bool((kc.cpu()[mask] == 0).all()) and bool((vc.cpu()[mask] == 0).all())   # nothing else written


@pytest.mark.parametrize("hd,rot,H,K", [(128, 128, 5, 2), (80, 64, 3, 3), (64, 32, 4, 1)])
def test_rope_cache_write_many_tokens(hd, rot, H, K):
    """300+ bfloat16 tokens take the kernel with 16-byte accesses: two sequences whose pages are scattered,
    one starting far into its context; every other cache row stays untouched."""
    ops = ops_mod()
    torch.manual_seed(1)
    page, max_pages = 16, 1300
    lens, starts = [170, 150], [0, 20000]
    pos = [starts[s] + i for s in range(2) for i in range(lens[s])]
    seq = [s for s in range(2) for _ in range(lens[s])]
    T = len(pos)
    qkv = torch.randn(T + 1, (H + 2 * K) * hd, device=DEV).bfloat16()
    orig = qkv.clone()
    inv = plain_inv_freq(rot, 5e5, None).to(DEV)
    n_pages = 40
    kc, vc = paged_cache(n_pages, page, K, hd, torch.bfloat16)
    order = torch.randperm(n_pages).tolist()
    table = torch.zeros(2, max_pages, dtype=torch.int32)
    cur = 0
    for s in range(2):
        for pg in range(starts[s] // page, (starts[s] + lens[s] - 1) // page + 1):
            table[s, pg] = order[cur]
            cur += 1
    table = table.to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ops.rope_cache_write(qkv, T, i32(seq), i32(pos), i32([0, 1]), inv, kc, vc, table, max_pages, page, H, K, hd, rot, False, True)
    o = orig[:T].double().cpu().reshape(T, H + 2 * K, hd)
    p_ = torch.tensor(pos)
    want_q, want_k = o[:, :H].clone(), o[:, H:H + K].clone()
    want_q[..., :rot] = plain_rope(o[:, :H, :rot], p_, inv.cpu(), "split_half")
    want_k[..., :rot] = plain_rope(o[:, H:H + K, :rot], p_, inv.cpu(), "split_half")
    got = qkv[:T].reshape(T, H + 2 * K, hd)
    close(got[:, :H], want_q, 2e-2, 1e-2)
    assert torch.equal(got[:, H:], orig[:T].reshape(T, H + 2 * K, hd)[:, H:]) and torch.equal(qkv[T], orig[T])
    tbl = table.cpu()
    pgs = torch.tensor([int(tbl[seq[t], pos[t] // page]) for t in range(T)])
    rows = torch.tensor([pos[t] % page for t in range(T)])
    close(kc.cpu()[pgs, rows], want_k, 2e-2, 1e-2)
    assert torch.equal(vc.cpu()[pgs, rows].double(), o[:, H + K:])
    mask = torch.ones(n_pages, page, dtype=torch.bool)
    mask[pgs, rows] = False
    assert bool((kc.cpu()[mask] == 0).all()) and bool((vc.cpu()[mask] == 0).all())


def fill_cache(seq_lens, K, hd, page, dtype, seed=0, scatter=True, poison=False):
    """Random keys/values for sequences, stored in shuffled pages. Returns dense and paged forms.
    `poison`: every cache row that belongs to no sequence (free pages, rows beyond a sequence's
    length) holds NaN, as after an earlier occupant whose values were not finite."""
    g = torch.Generator().manual_seed(seed)
    n_pages_each = [-(-n // page) for n in seq_lens]
    total = sum(n_pages_each) + 3
    order = torch.randperm(total, generator=g).tolist() if scatter else list(range(total))
    kc, vc = paged_cache(total, page, K, hd, dtype)
    if poison:
        kc.fill_(float("nan"))
        vc.fill_(float("nan"))
    max_pages = max(n_pages_each) + 1
    table = torch.zeros(len(seq_lens), max_pages, dtype=torch.int32)
    dense = []
    cur = 0
    for s, n in enumerate(seq_lens):
        k = torch.randn(n, K, hd, generator=g).to(dtype)
        v = torch.randn(n, K, hd, generator=g).to(dtype)
        dense.append((k, v))
        for pi in range(n_pages_each[s]):
            pg = order[cur]; cur += 1
            table[s, pi] = pg
            rows = slice(pi * page, min(n, (pi + 1) * page))
            kc[pg, : rows.stop - rows.start] = k[rows].to(DEV)
            vc[pg, : rows.stop - rows.start] = v[rows].to(DEV)
    return kc, vc, table.to(DEV), max_pages, dense


def reference_attention(q, dense, tok_seq, tok_pos, scale, window):
    """q [T,H,D] float64.  Token t at position p of its sequence sees the keys [first, p], first = 0 or
    p + 1 - window; kv head = head // group; s = (q.k) * scale; p = exp(s - max) / sum; o = sum p v
    (src/backend/cpu.rs:530-590), in float64."""
    T, H, D = q.shape
    out = torch.zeros(T, H * D, dtype=torch.float64)
    for t in range(T):
        k, v = dense[tok_seq[t]]
        n = tok_pos[t] + 1
        first = 0 if window == 0 else max(0, n - window)
        kk, vv = k[first:n].double(), v[first:n].double()
        group = H // kk.shape[1]
        for h in range(H):
            s = (kk[:, h // group, :] @ q[t, h]) * scale
            p = torch.exp(s - s.max())
            out[t, h * D:(h + 1) * D] = (p / p.sum()) @ vv[:, h // group, :]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,K,hd,window", [(6, 2, 48, 0), (4, 4, 16, 0), (8, 1, 128, 0), (6, 3, 80, 37), (5, 5, 256, 0)])
def test_attention_simple(dtype, H, K, hd, window):
    ops = ops_mod()
    torch.manual_seed(1)
    page = 16
    seq_lens = [300, 41, 1]
    kc, vc, table, max_pages, dense = fill_cache(seq_lens, K, hd, page, dtype)
    tok_seq = [0, 0, 0, 1, 1, 2]
    tok_pos = [299, 150, 0, 40, 16, 0]
    T = len(tok_seq)
    q = torch.randn(T, H * hd + 24, device=DEV).to(dtype)          # padded row: queries are a prefix
    out = torch.full((T + 1, H * hd), 9.0, device=DEV, dtype=dtype)
    scale = 0.77 / math.sqrt(hd)
    ops.attention_simple(q, T, kc, vc, torch.tensor(tok_seq, dtype=torch.int32, device=DEV),
                         torch.tensor(tok_pos, dtype=torch.int32, device=DEV),
                         torch.arange(3, dtype=torch.int32, device=DEV), table, max_pages, page, out,
                         H, K, hd, window, scale)
    want = reference_attention(q[:, :H * hd].double().cpu().reshape(T, H, hd), dense, tok_seq, tok_pos, scale, window)
    close(out[:T], want, 2e-5 if dtype == torch.float32 else 3e-2)
    assert bool((out[T:] == 9.0).all())


def test_attention_finds_one_far_key():
    """One key among hundreds is made to dominate; random weights would hide a miss."""
    ops = ops_mod()
    H, K, hd, page = 2, 1, 32, 16
    kc, vc, table, max_pages, dense = fill_cache([700], K, hd, page, torch.float32, seed=3)
    k, v = dense[0]
    q = torch.randn(1, H * hd)
    target = 123
    k[target, 0] = q[0, :hd] * 4.0                               # head 0 points at key 123
    pg = int(table[0, target // page])
    kc[pg, target % page, 0] = k[target, 0].to(DEV)
    out = torch.zeros(1, H * hd, device=DEV)
    ops.attention_simple(q.to(DEV), 1, kc, vc, torch.zeros(1, dtype=torch.int32, device=DEV),
                         torch.tensor([699], dtype=torch.int32, device=DEV),
                         torch.zeros(1, dtype=torch.int32, device=DEV), table, max_pages, page, out,
                         H, K, hd, 0, 1.0)
    close(out[0, :hd], v[target, 0], 1e-4)                      # softmax is one-hot on the far key
    want = reference_attention(q.double().reshape(1, H, hd), dense, [0], [699], 1.0, 0)
    close(out, want, 2e-5)


class StepMeta:
    """Sequences with `new` tokens each on top of `cached` tokens already in the cache."""

    def __init__(self, cached, new):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        starts = [0]
        for n in new:
            starts.append(starts[-1] + n)
        self.n_seqs, self.n_tokens = len(new), starts[-1]
        self.max_new, self.max_len = max(new), max(c + n for c, n in zip(cached, new))
        self.seq_start, self.seq_pos0, self.seq_slot = i32(starts), i32(cached), i32(list(range(len(new))))
        self.tok_seq = [s for s, n in enumerate(new) for _ in range(n)]
        self.tok_pos = [c + j for c, n in zip(cached, new) for j in range(n)]


@pytest.mark.parametrize("H,K,hd,window", [(8, 2, 128, 0), (6, 2, 48, 0), (4, 4, 16, 0), (12, 2, 64, 0),
                                           (6, 1, 80, 0), (8, 2, 128, 100), (5, 5, 112, 33), (32, 8, 128, 0),
                                           (40, 2, 64, 0), (64, 1, 32, 0)])      # groups of 20 and 64 query heads
@pytest.mark.parametrize("case", ["prefill", "chunked", "decode", "decode_split", "decode_long", "decode_many1",
                                  "decode_many3", "decode_many4", "decode_many5", "decode_page16", "prefill_tc", "chunked_tc"])
@pytest.mark.parametrize("poison", [False, True])
def test_attention_tensor(H, K, hd, window, case, poison):
    """The tensor-core attention against the float64 statement of the reference's loop:
    whole prompts, prompts on top of a cached prefix, single tokens (one block of eight warps; keys
    split over blocks, by hand and by the kernel's own choice for a long context; so many sequences
    that blocks of four, three and two warps and of one warp are taken; pages that the tile loads cannot use), with and
    without NaN in every cache row that belongs to nobody."""
    from mdma_b200 import ops_tensor
    torch.manual_seed(H * 1000 + hd)
    page = 16 if case == "decode_page16" else 64
    impl = "tc" if case.endswith("_tc") else "mma"
    case = case.replace("_tc", "")
    if case == "prefill":
        cached, new = [0, 0, 0], [150, 3, 65]
    elif case == "chunked":
        cached, new = [70, 129, 1], [100, 20, 64]
    elif case == "decode_long":
        cached, new = [2500, 1030, 7], [1, 1, 1]          # beyond 1024: the kernel splits the keys itself
    elif case.startswith("decode_many"):
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        n = -(-int(case[-1]) * sms // K) + 1              # sequences x kv heads just beyond 1, 3, 4, 5 x SMs: blocks of 4, 3, 2 warps, 1 warp
        g = torch.Generator().manual_seed(7)
        cached, new = torch.randint(0, 150, (n,), generator=g).tolist(), [1] * n
    else:
        cached, new = [299, 0, 64, 1000], [1, 1, 1, 1]
    lens = [c + n for c, n in zip(cached, new)]
    kc, vc, table, max_pages, dense = fill_cache(lens, K, hd, page, torch.bfloat16, seed=hd, poison=poison)
    meta = StepMeta(cached, new)
    T = meta.n_tokens
    q = (torch.randn(T, (H + 2 * K) * hd, device=DEV)).bfloat16()
    out = torch.full((T + 1, H * hd), 9.0, device=DEV, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)

    class View:
        pass
    view = View()
    view.k, view.v, view.page_table, view.max_pages, view.page_size = kc, vc, table, max_pages, page
    splits = {"decode_split": 5, "chunked": 2}.get(case) if impl == "mma" else None
    ops_tensor.attention(meta, q, view, out, H, K, hd, window, scale, splits=splits, impl=impl)
    ops_tensor.check_status(torch.device(DEV))
    want = reference_attention(q[:, :H * hd].double().cpu().reshape(T, H, hd), dense, meta.tok_seq, meta.tok_pos,
                               scale, window)
    close(out[:T], want, 2e-2, 2e-2)
    assert bool((out[T:] == 9.0).all())


@pytest.mark.parametrize("H,K,hd,rot,layout,window", [(8, 2, 128, 128, "split_half", 0), (6, 2, 48, 48, "interleaved", 0),
                                                       (4, 4, 16, 16, "split_half", 0), (12, 2, 64, 32, "split_half", 70),
                                                       (32, 8, 128, 128, "split_half", 0), (5, 5, 112, 64, "interleaved", 33)])
@pytest.mark.parametrize("proj_splits,key_splits", [(0, None), (4, None), (3, 3), (0, 4)])
def test_attention_decode_with_the_rotary_encoding_inside(H, K, hd, rot, layout, window, proj_splits, key_splits):
    """Single tokens: one kernel sums the projection's partial rows, rotates q and k, writes k and v to the
    cache and attends.  Against the separate rotary kernel (the same cache rows, bit for bit) and against
    the float64 statement of rotation and attention; the cache starts with NaN in every row nobody owns."""
    from mdma_b200 import ops_tensor
    from mdma_b200.parts.rotary import inverse_frequencies
    ops = ops_mod()
    torch.manual_seed(H * 100 + hd + proj_splits)
    page = 64
    cached = [299, 0, 64, 1000, 31]
    B = len(cached)
    lens = [c + 1 for c in cached]
    kc, vc, table, max_pages, dense = fill_cache(lens, K, hd, page, torch.bfloat16, seed=hd, poison=True)
    width = (H + 2 * K) * hd
    inv_freq = inverse_frequencies(rot, 10000.0).to(DEV)
    rows = torch.randn(B, width)
    if proj_splits:
        parts = torch.randn(proj_splits, B, width) * 0.5
        parts[-1] = rows - parts[:-1].sum(0)
        total = torch.zeros(B, width)
        for sidx in range(proj_splits):                       # the kernels' order of summation
            total = total + parts[sidx]
        rows = total
    qkv = rows.bfloat16().to(DEV)                             # read only when there are no partial sums
    meta = StepMeta(cached, [1] * B)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tok_seq, tok_pos = i32(list(range(B))), i32(cached)
    # the separate kernel on copies: rotated q in its buffer, k and v in its caches
    kc2, vc2, qkv2 = kc.clone(), vc.clone(), qkv.clone()
    part_dev = parts.to(DEV).contiguous() if proj_splits else None
    ops.rope_cache_write(qkv2, B, tok_seq, tok_pos, meta.seq_slot, inv_freq, kc2, vc2, table, max_pages, page, H, K, hd,
                         rot, layout == "interleaved", True, part_dev, proj_splits, B * width)

    class View:
        pass
    view = View()
    view.k, view.v, view.page_table, view.max_pages, view.page_size = kc, vc, table, max_pages, page
    out = torch.full((B + 1, H * hd), 9.0, device=DEV, dtype=torch.bfloat16)
    st = ops_tensor._device_state(torch.device(DEV))
    if proj_splits:
        st.need(proj_splits * B * width, "test")
        st.scratch[:proj_splits * B * width].copy_(part_dev.reshape(-1))
        st.pending = ops_tensor.Pending(qkv, ops.GEMM_STORE, proj_splits, B, width)
    scale = 1.0 / math.sqrt(hd)
    ops_tensor.attention_decode_rotary(meta, qkv, view, out, H, K, hd, window, scale, inv_freq, rot,
                                       layout == "interleaved", splits=key_splits)
    ops_tensor.check_status(torch.device(DEV))
    # the cache rows of the new tokens, and nothing else, were written: exactly what the separate kernel writes
    assert torch.equal(kc.view(torch.int16), kc2.view(torch.int16)) and torch.equal(vc.view(torch.int16), vc2.view(torch.int16))
    # attention over the (now complete) sequences, in float64, with the rotated queries of the separate kernel
    for sidx, n in enumerate(lens):
        kd, vd = dense[sidx]
        pg = int(table[sidx, (n - 1) // page])
        kd[n - 1], vd[n - 1] = kc2[pg, (n - 1) % page].cpu(), vc2[pg, (n - 1) % page].cpu()
    q = qkv2[:, :H * hd].double().cpu().reshape(B, H, hd)
    want = reference_attention(q, dense, list(range(B)), cached, scale, window)
    close(out[:B], want, 2e-2, 2e-2)
    assert bool((out[B:] == 9.0).all())
    # and the rotation itself against the plain statement
    from plain_llama import plain_rope
    for sidx in range(B):
        qr = plain_rope(rows[sidx, :H * hd].double().reshape(1, H, hd)[..., :rot], torch.tensor([cached[sidx]]),
                        inv_freq.cpu(), layout)
        close(qkv2[sidx, :H * hd].reshape(H, hd)[:, :rot], qr[0], 2e-2, 1e-2)


@pytest.mark.parametrize("path", ["decode", "decode_split", "prefill_tc", "chunked_tc", "chunked_mma"])
def test_attention_tensor_finds_one_far_key_and_the_window_edge(path):
    """One key among 900 is made to dominate the last query's head 0: inside the window it must be
    found, one place before the window it must not be seen; on every kernel that serves the engine."""
    from mdma_b200 import ops_tensor
    H, K, hd, page = 4, 1, 64, 64
    kc, vc, table, max_pages, dense = fill_cache([900], K, hd, page, torch.bfloat16, seed=5)
    k, v = dense[0]
    cached, new = {"decode": (899, 1), "decode_split": (899, 1), "prefill_tc": (0, 900),
                   "chunked_tc": (600, 300), "chunked_mma": (880, 20)}[path]
    q = torch.randn(new, (H + 2 * K) * hd).bfloat16()
    for target, window, seen in ((123, 0, True), (899 - 99, 100, True), (899 - 100, 100, False)):
        kk = k.clone()
        kk[target, 0] = (q[-1, :hd].float() * 3.0).bfloat16()         # head 0 of the last token points at one key
        pg = int(table[0, target // page])
        kc2 = kc.clone()
        kc2[pg, target % page, 0] = kk[target, 0].to(DEV)
        meta = StepMeta([cached], [new])
        out = torch.zeros(new, H * hd, device=DEV, dtype=torch.bfloat16)

        class View:
            pass
        view = View()
        view.k, view.v, view.page_table, view.max_pages, view.page_size = kc2, vc, table, max_pages, page
        ops_tensor.attention(meta, q.to(DEV), view, out, H, K, hd, window, 1.0,
                             splits=3 if path == "decode_split" else None,
                             impl="tc" if path.endswith("_tc") else "mma")
        ops_tensor.check_status(torch.device(DEV))
        hit = (out[-1, :hd].float().cpu() - v[target, 0].float()).abs().max().item() < 0.05
        assert hit == seen, (path, target, window)


@pytest.mark.parametrize("M,N,K", [(1, 5, 3), (67, 130, 100), (5, 331, 120), (200, 64, 17)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_gemm_simt(M, N, K, dt):
    ops = ops_mod()
    torch.manual_seed(M)
    a = torch.randn(M + 1, K + 8, device=DEV).to(dt)[:, :K]      # a pitch wider than K
    w = (torch.randn(N, K, device=DEV) * 0.1).to(dt)
    w2 = (torch.randn(N, K, device=DEV) * 0.1).to(dt)
    ref = a[:M].double() @ w.double().t()
    tol = dict(atol=1e-5) if dt == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    out = torch.full((M + 1, N), 9.0, device=DEV, dtype=dt)
    ops.gemm_simt(a, w, out, ops.GEMM_STORE, None, M)
    close(out[:M], ref, **tol)
    assert bool((out[M:] == 9.0).all())
    x = torch.randn(M + 1, N, device=DEV)
    x0 = x.clone()
    if dt == torch.bfloat16:
        ops.gemm_simt(a, w, x, ops.GEMM_ACCUMULATE, None, M)
        close(x[:M], x0[:M].double() + ref, 1e-5 * K)
        assert torch.equal(x[M:], x0[M:])
    ref2 = a[:M].double() @ w2.double().t()
    ops.gemm_simt(a, w, out, ops.GEMM_SWIGLU, w2, M)
    close(out[:M], ref / (1 + torch.exp(-ref)) * ref2, **tol)


def test_gemm_simt_rows_do_not_depend_on_their_neighbours():
    ops = ops_mod()
    a = torch.randn(70, 96, device=DEV)
    w = torch.randn(50, 96, device=DEV)
    big = torch.empty(70, 50, device=DEV)
    one = torch.empty(1, 50, device=DEV)
    ops.gemm_simt(a, w, big)
    ops.gemm_simt(a[37:38], w, one)
    assert torch.equal(big[37:38], one)                           # bitwise: fixed order of additions


@pytest.mark.parametrize("M,N,K,mode", [(1, 128, 64, 0), (9, 200, 72, 0), (130, 1000, 1032, 0), (600, 264, 256, 0),
                                        (7, 520, 2048, 1), (300, 136, 512, 1), (3, 300, 264, 2), (257, 384, 640, 2),
                                        (2, 331, 8, 0),
                                        # 129-512 tokens and few feature tiles: one block per tile, K split by the plan
                                        (200, 520, 4096, 0), (300, 136, 2048, 1), (512, 264, 1024, 1), (129, 128, 8192, 0)])
def test_gemm_tensor(M, N, K, mode):
    from mdma_b200 import ops_tensor
    ops = ops_mod()
    torch.manual_seed(N)
    a = (torch.randn(M + 3, K + 16, device=DEV) * 0.5).bfloat16()[:, :K]
    w = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    w2 = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    ref = a[:M].double() @ w.double().t()
    if mode == 1:
        x = torch.randn(M + 2, N, device=DEV)
        x0 = x.clone()
        ops_tensor.gemm(a, w, x, ops.GEMM_ACCUMULATE, None, M)
        close(x[:M], x0[:M].double() + ref, 2e-5 * max(K, 64) ** 0.5 + 1e-5)
        assert torch.equal(x[M:], x0[M:])
    else:
        for odt in (torch.bfloat16, torch.float32) if mode == 0 else (torch.bfloat16,):
            out = torch.full((M + 2, N), 9.0, device=DEV, dtype=odt)
            ops_tensor.gemm(a, w, out, mode, w2 if mode == 2 else None, M)
            want = ref if mode == 0 else ref / (1 + torch.exp(-ref)) * (a[:M].double() @ w2.double().t())
            close(out[:M], want, 1e-4 if odt == torch.float32 else 1e-2, 0 if odt == torch.float32 else 1e-2)
            assert bool((out[M:] == 9.0).all())
    ops_tensor.check_status(torch.device(DEV))


def _ending_reference(a, w, w2, b, b2, mode, act, x0):
    ref = a.double() @ w.double().t() + b.double()
    if mode == 0:
        return ref
    if mode == 1:
        return x0.double() + ref
    up = a.double() @ w2.double().t() + b2.double()
    if act == 0:
        return ref / (1 + torch.exp(-ref)) * up
    return 0.5 * ref * (1 + torch.tanh(math.sqrt(2 / math.pi) * (ref + 0.044715 * ref ** 3))) * up


@pytest.mark.parametrize("bias_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K,mode,act,kw", [
    (7, 520, 2048, 0, 0, {}),                       # the plan splits K: the bias goes into the first partial sum only
    (7, 520, 2048, 1, 0, {}),
    (5, 300, 1024, 1, 0, dict(splits=-3)),          # K split inside a cluster
    (17, 264, 1536, 2, 1, dict(splits=-2)),
    (64, 264, 512, 2, 1, {}), (9, 200, 72, 2, 0, {}),
    (300, 520, 1032, 0, 0, {}), (200, 136, 4096, 1, 0, {}),      # one block per tile with a K split (129-512 tokens)
    (700, 264, 512, 1, 0, {}), (600, 384, 640, 2, 1, {}),        # block pairs
])
def test_gemm_tensor_bias_and_gate_activation(M, N, K, mode, act, kw, bias_dtype):
    """out = a W^T + b (stored, or added to the residual stream), and act(a Wg^T + bg) * (a Wu^T + bu) with SiLU
    or GELU as the gate: on every kernel and split of the tensor-core product."""
    from mdma_b200 import ops_tensor
    torch.manual_seed(N + K)
    a = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    w2 = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    b = torch.randn(N, device=DEV).to(bias_dtype)
    b2 = torch.randn(N, device=DEV).to(bias_dtype)
    x0 = torch.randn(M + 1, N, device=DEV)
    out = x0.clone() if mode == 1 else torch.full((M + 1, N), 9.0, device=DEV, dtype=torch.bfloat16)
    ops_tensor.gemm(a, w, out, mode, w2 if mode == 2 else None, M, bias=b, bias2=b2 if mode == 2 else None, act=act, **kw)
    ops_tensor.check_status(torch.device(DEV))
    want = _ending_reference(a, w, w2, b, b2, mode, act, x0[:M])
    close(out[:M], want, 1e-3 if mode == 1 else 2e-2, 0 if mode == 1 else 1e-2)
    assert torch.equal(out[M:], x0[M:]) if mode == 1 else bool((out[M:] == 9.0).all())


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode,act", [(0, 0), (1, 0), (2, 0), (2, 1)])
def test_gemm_simt_bias_and_gate_activation(dt, mode, act):
    ops = ops_mod()
    M, N, K = 67, 130, 100
    torch.manual_seed(mode)
    a = (torch.randn(M, K, device=DEV) * 0.5).to(dt)
    w, w2 = (torch.randn(N, K, device=DEV) * 0.1).to(dt), (torch.randn(N, K, device=DEV) * 0.1).to(dt)
    b, b2 = torch.randn(N, device=DEV).to(dt), torch.randn(N, device=DEV).to(dt)
    x0 = torch.randn(M, N, device=DEV)
    out = x0.clone() if mode == 1 else torch.empty(M, N, device=DEV, dtype=dt)
    ops.gemm_simt(a, w, out, mode, w2 if mode == 2 else None, M, b, b2 if mode == 2 else None, act)
    want = _ending_reference(a, w, w2, b, b2, mode, act, x0)
    tol = dict(atol=2e-5) if dt == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    close(out, want, **(tol if mode != 1 else dict(atol=1e-4 if dt == torch.float32 else 1e-3)))


@pytest.mark.parametrize("splits", [2, 3, 7])
def test_gemm_tensor_split_k_is_reproducible(splits):
    from mdma_b200 import ops_tensor
    ops = ops_mod()
    a = (torch.randn(5, 1024, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(200, 1024, device=DEV) * 0.1).bfloat16()
    ref = a.double() @ w.double().t()
    outs = []
    for _ in range(2):
        out = torch.zeros(5, 200, device=DEV)
        ops_tensor.gemm(a, w, out, ops.GEMM_STORE, None, 5, bn=16, splits=splits)
        outs.append(out)
    close(outs[0], ref, 1e-4)
    assert torch.equal(outs[0], outs[1])
    ops_tensor.check_status(torch.device(DEV))


@pytest.mark.parametrize("cluster", [2, 3, 8])
@pytest.mark.parametrize("M,N,K,mode", [(8, 520, 2048, 0), (5, 300, 1024, 1), (17, 264, 1536, 2), (1, 128, 4096, 1)])
def test_gemm_tensor_cluster_split(cluster, M, N, K, mode):
    """K divided among the blocks of a cluster, summed through shared memory in rank order."""
    from mdma_b200 import ops_tensor
    ops = ops_mod()
    torch.manual_seed(K + cluster)
    a = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    w2 = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    ref = a.double() @ w.double().t()
    outs = []
    for _ in range(2):
        if mode == 1:
            out = torch.ones(M + 1, N, device=DEV)
            ops_tensor.gemm(a, w, out, ops.GEMM_ACCUMULATE, None, M, splits=-cluster)
            want = ref + 1.0
        else:
            out = torch.full((M + 1, N), 9.0, device=DEV, dtype=torch.float32 if mode == 0 else torch.bfloat16)
            ops_tensor.gemm(a, w, out, mode, w2 if mode == 2 else None, M, splits=-cluster)
            want = ref if mode == 0 else ref / (1 + torch.exp(-ref)) * (a.double() @ w2.double().t())
        close(out[:M], want, 1e-4 if out.dtype == torch.float32 else 1e-2, 0 if out.dtype == torch.float32 else 1e-2)
        assert bool((out[M:] == (1.0 if mode == 1 else 9.0)).all())
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    ops_tensor.check_status(torch.device(DEV))


@pytest.mark.parametrize("M,N,K,mode", [(256, 256, 64, 0), (300, 520, 1032, 0), (1000, 264, 512, 1), (257, 384, 640, 2),
                                        (2048, 1024, 2048, 2), (130, 100, 72, 0),
                                        # more tiles than block pairs: every pair walks over several tiles
                                        (1100, 5000, 256, 0), (1100, 5000, 256, 1), (1100, 5000, 256, 2), (2300, 8200, 192, 1),
                                        # tiles shared by two pairs (K blocks split evenly), several K blocks per part
                                        (1100, 5000, 1032, 0), (1100, 5000, 1032, 1), (700, 9000, 2048, 2), (2048, 4096, 4096, 0),
                                        # token tiles of 32, 96, 192 and 224 (the tokens divided evenly over the fewest tiles)
                                        (129, 520, 256, 0), (20, 300, 512, 1), (90, 600, 256, 2), (380, 1000, 320, 2), (640, 3000, 512, 0)])
def test_gemm_tensor_block_pairs(M, N, K, mode):
    """The two-block kernel (cta_group::2): a pair covers 256 features x a token tile of up to 256."""
    from mdma_b200 import ops_tensor
    ops = ops_mod()
    torch.manual_seed(M + N)
    a = (torch.randn(M + 2, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    w2 = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    ref = a[:M].double() @ w.double().t()
    if mode == 1:
        x = torch.randn(M + 2, N, device=DEV)
        x0 = x.clone()
        ops_tensor.gemm(a, w, x, ops.GEMM_ACCUMULATE, None, M, bn=512, splits=1)
        close(x[:M], x0[:M].double() + ref, 2e-5 * max(K, 64) ** 0.5 + 1e-5)
        assert torch.equal(x[M:], x0[M:])
    else:
        out = torch.full((M + 2, N), 9.0, device=DEV, dtype=torch.bfloat16)
        ops_tensor.gemm(a, w, out, mode, w2 if mode == 2 else None, M, bn=512, splits=1)
        want = ref if mode == 0 else ref / (1 + torch.exp(-ref)) * (a[:M].double() @ w2.double().t())
        close(out[:M], want, 1e-2, 1e-2)
        assert bool((out[M:] == 9.0).all())
        again = torch.full_like(out, 9.0)       # a second call finds the scratch and its flags as the first left them
        ops_tensor.gemm(a, w, again, mode, w2 if mode == 2 else None, M, bn=512, splits=1)
        assert torch.equal(out, again)
    ops_tensor.check_status(torch.device(DEV))


def test_gemm_tensor_refuses_what_it_cannot_do():
    from mdma_b200 import ops_tensor
    from mdma_b200.ops import KernelError
    a = torch.zeros(4, 100, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(16, 100, device=DEV, dtype=torch.bfloat16)
    assert not ops_tensor.gemm_supported(16, 100)
    with pytest.raises(KernelError, match="multiple of 8"):
        ops_tensor.gemm(a, w, torch.zeros(4, 16, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(KernelError, match="bfloat16"):
        ops_tensor.gemm(a.float(), w.float(), torch.zeros(4, 16, device=DEV))


def test_kernels_refuse_cpu_tensors():
    ops = ops_mod()
    from mdma_b200.ops import KernelError
    with pytest.raises(KernelError, match="no CPU path"):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-5, torch.zeros(2, 8))


def test_argmax_lowest_index_and_flags():
    ops = ops_mod()
    logits = torch.randn(5, 33001, device=DEV)
    logits[0, 777] = logits[0, 31000] = 50.0                      # tie: the lowest index
    logits[1, 33000] = 60.0                                       # last element
    logits[2, 5] = float("nan")
    logits[3, 9] = float("inf")
    tok = torch.zeros(6, dtype=torch.int32, device=DEV)
    flags = torch.zeros(6, dtype=torch.int32, device=DEV)
    ops.argmax(logits, tok, flags, 5)
    assert tok[:2].tolist() == [777, 33000] and int(tok[4]) == int(logits[4].argmax())
    assert flags[:5].tolist() == [0, 0, 1, 1, 0]


@pytest.mark.parametrize("impl", [1, 2])          # one block per row; a cluster of eight blocks per row
@pytest.mark.parametrize("vocab", [331, 5000, 40003])
@pytest.mark.parametrize("opts", [dict(temperature=0.8, top_p=0.95, min_p=0.05, repetition_penalty=1.1),
                                  dict(temperature=1.3, top_p=1.0, min_p=0.0, repetition_penalty=1.0),
                                  dict(temperature=0.5, top_p=0.3, min_p=0.0, repetition_penalty=1.0),
                                  dict(temperature=1.0, top_p=1.0, min_p=0.2, repetition_penalty=1.5),
                                  dict(temperature=0.0, top_p=1.0, min_p=0.0, repetition_penalty=1.7)])
def test_sample_matches_the_host_sampler(vocab, opts, impl):
    """Same uniform number, same token as the plain sampler (src/sampler.rs:34-135)."""
    ops = ops_mod()
    torch.manual_seed(vocab)
    n = 24 if vocab < 20000 else 5
    logits = torch.randn(n, vocab) * 3
    logits[3, 10] = logits[3, 20] = logits[3].max() + 1           # tied leaders
    hist = torch.randint(0, vocab, (n, 64), dtype=torch.int32)
    hist[:, 0] = logits.argmax(1).int()                           # penalise the leader
    hlen = torch.full((n,), 64, dtype=torch.int32)
    u = torch.rand(n)
    tok = torch.zeros(n, dtype=torch.int32, device=DEV)
    flags = torch.zeros(n, dtype=torch.int32, device=DEV)
    scratch = torch.empty(ops.sample_scratch_words(n, vocab), device=DEV)
    ops.sample(logits.to(DEV), u.to(DEV), tok, scratch, opts["temperature"], opts["top_p"], opts["min_p"],
               opts["repetition_penalty"], 64, hist.to(DEV), hlen.to(DEV), flags, impl=impl)
    want = [plain_sample(logits[i].tolist(), hist[i].tolist(), float(u[i]), opts["temperature"], opts["top_p"],
                         opts["min_p"], opts["repetition_penalty"], 64) for i in range(n)]
    got = tok.tolist()
    mism = [i for i in range(n) if got[i] != want[i]]
    assert not mism, f"rows {mism}: got {[got[i] for i in mism]}, want {[want[i] for i in mism]}"
    assert flags.sum().item() == 0


@pytest.mark.parametrize("opts", [dict(temperature=0.8, top_p=0.95, min_p=0.05, repetition_penalty=1.1),
                                  dict(temperature=0.8, top_p=1.0, min_p=0.0, repetition_penalty=1.0)])
def test_sample_at_the_vocabulary_of_the_benchmark(opts):
    """128,256 entries, where a block of the cluster holds 64 KB of the row: the kernel's own choice of
    variant, four rows, the default options and temperature alone; also with the options read from
    device memory, as the replayed decode loop passes them."""
    ops = ops_mod()
    from mdma_b200.sampling import SamplingParams
    from mdma_b200.sampling.sampler import params_words
    vocab, n = 128256, 4
    torch.manual_seed(11)
    logits = torch.randn(n, vocab) * 2.5
    logits[1, 100] = logits[1, 128255] = logits[1].max() + 0.5    # tied leaders, one of them the last entry
    hist = torch.randint(0, vocab, (n, 64), dtype=torch.int32)
    hist[:, 0] = logits.argmax(1).int()
    hlen = torch.full((n,), 64, dtype=torch.int32)
    u = torch.tensor([0.03, 0.5, 0.77, 0.999])
    tok = torch.zeros(n, dtype=torch.int32, device=DEV)
    flags = torch.zeros(n, dtype=torch.int32, device=DEV)
    scratch = torch.empty(ops.sample_scratch_words(n, vocab), device=DEV)
    args = (opts["temperature"], opts["top_p"], opts["min_p"], opts["repetition_penalty"], 64)
    ops.sample(logits.to(DEV), u.to(DEV), tok, scratch, *args, hist.to(DEV), hlen.to(DEV), flags)
    got = tok.tolist()
    assert flags.sum().item() == 0
    if opts["min_p"] > 0:             # a handful of candidates: the plain sampler's token exactly
        want = [plain_sample(logits[i].tolist(), hist[i].tolist(), float(u[i]), *args) for i in range(n)]
        assert got == want
    else:
        # Every entry is a candidate, each with about 1e-5 of the mass: a float32 running sum over 128,256
        # terms (the plain sampler's) is itself uncertain by more than that, so the check is made in
        # float64: the uniform number must lie in the selected token's interval of the descending order
        # (ties by token id), give or take 1e-6 of the mass for the float32 exponentials.
        for i in range(n):
            x = logits[i].double() / opts["temperature"]      # penalty 1: the history does not matter
            p = torch.exp(x - x.max())
            p = p / p.sum()
            order = sorted(range(vocab), key=lambda t: (-float(p[t]), t))
            cum = torch.cumsum(p[order], 0)
            r = order.index(got[i])
            lo = float(cum[r - 1]) if r else 0.0
            assert lo - 1e-6 <= float(u[i]) <= float(cum[r]) + 1e-6, (i, got[i], lo, float(u[i]), float(cum[r]))
    words = torch.from_numpy(params_words(SamplingParams(*args, seed=0))).to(DEV)
    tok2 = torch.zeros_like(tok)
    ops.sample(logits.to(DEV), u.to(DEV), tok2, scratch, 1.0, 1.0, 0.0, 1.0, 0, hist.to(DEV), hlen.to(DEV), flags,
               dev_params=words)
    assert tok2.tolist() == got


@pytest.mark.parametrize("impl", [1, 2])
def test_sample_follows_the_distribution(impl):
    ops = ops_mod()
    vocab, n = 50, 4000
    row = torch.randn(vocab) * 2
    logits = row.repeat(n, 1).to(DEV)
    u = torch.rand(n, generator=torch.Generator().manual_seed(0)).to(DEV)
    tok = torch.zeros(n, dtype=torch.int32, device=DEV)
    scratch = torch.empty(ops.sample_scratch_words(n, vocab), device=DEV)
    ops.sample(logits, u, tok, scratch, 1.0, 1.0, 0.0, 1.0, 0, impl=impl)
    freq = torch.bincount(tok.long().cpu(), minlength=vocab).double() / n
    p = torch.softmax(row.double(), 0)
    assert (freq - p).abs().max() < 4 * (p.max() * (1 - p.max()) / n) ** 0.5 + 0.01


def test_a_wait_that_runs_out_is_reported_and_leaves_the_library_usable():
    """Every wait of the tensor-core kernels has a limit; when it runs out the block gives up, the status
    word is set and the host raises.  Seen here without breaking anything: the limit is shortened to
    20 ms and a kernel that only waits (with the product kernels' wait routines) is given an mbarrier
    that nobody arrives on, then a flag that nothing sets.  Afterwards the flags are clear and the next
    product is right."""
    import time
    from mdma_b200 import ops_tensor
    ops = ops_mod()
    dev = torch.device(DEV)
    st = ops_tensor._device_state(dev)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops_tensor.set_wait_limit(0.02)
    try:
        for mode in (0, 1):
            st.sk_flags[3] = 1                      # as a block pair that gave up would leave it
            t0 = time.perf_counter()
            ops_tensor.wait_probe(mode, flag)
            torch.cuda.synchronize()
            assert time.perf_counter() - t0 < 1.0   # it gave up after the short limit, not after 2 s
            with pytest.raises(ops.KernelError, match="wait limit"):
                ops_tensor.check_status(dev)
            assert int(st.status[0]) == 0 and int(st.sk_flags.sum()) == 0
            ops_tensor.check_status(dev)            # and stays quiet
        flag.fill_(1)                               # a flag that IS set: the wait ends at once, nothing is reported
        ops_tensor.wait_probe(1, flag)
        ops_tensor.check_status(dev)
    finally:
        ops_tensor.set_wait_limit(2.0)
    a = torch.randn(5, 256, device=DEV).bfloat16()
    w = torch.randn(130, 256, device=DEV).bfloat16()
    out = torch.zeros(5, 130, device=DEV, dtype=torch.bfloat16)
    ops_tensor.gemm(a, w, out)
    ops_tensor.check_status(dev)
    close(out, a.double().cpu() @ w.double().cpu().t(), 0.2, 2e-2)
