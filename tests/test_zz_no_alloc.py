"""The allocation-free attention entry point, called through its exported C symbol.

Some hosts of these kernels cannot allocate device memory: their memory was
planned and handed out before the first step, and a decode loop cannot pay for
a cudaMalloc that may stall the device.  `mdma_attention_mma_noalloc` keeps the
split-K partials in a fixed array inside the library instead of a caller's
buffer.  This test checks that it gives, bit for bit, what the ordinary entry
point gives (the same kernels with the same splits), that both are right
against a plain float64 statement of the attention formula, twice in a row
(the array is shared and keeps the last call's contents), and that it refuses
a call that would not fit.  It is collected last so that a run
that stops at the first failure has run everything else before.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_FLOATS = 4 * 1024 * 1024


def make_case(seed, lens, H, K, hd, page=64):
    g = torch.Generator().manual_seed(seed)
    n_pages_each = [-(-n // page) for n in lens]
    total = sum(n_pages_each) + 2
    order = torch.randperm(total, generator=g).tolist()
    kc = torch.zeros(total, page, K, hd, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    max_pages = max(n_pages_each) + 1
    table = torch.zeros(len(lens), max_pages, dtype=torch.int32)
    cur = 0
    dense = []
    for s, n in enumerate(lens):
        ks, vs = [], []
        for pi in range(n_pages_each[s]):
            pg = order[cur]
            cur += 1
            table[s, pi] = pg
            rows = min(page, n - pi * page)
            kc[pg, :rows] = torch.randn(rows, K, hd, generator=g).bfloat16()
            vc[pg, :rows] = torch.randn(rows, K, hd, generator=g).bfloat16()
            ks.append(kc[pg, :rows].clone())
            vs.append(vc[pg, :rows].clone())
        dense.append((torch.cat(ks), torch.cat(vs)))
    B = len(lens)
    q = torch.randn(B, (H + 2 * K) * hd, generator=g).bfloat16()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return dict(q=q.to(DEV), k=kc.to(DEV), v=vc.to(DEV), table=table.to(DEV), max_pages=max_pages, page=page,
                seq_start=i32(list(range(B + 1))), seq_pos0=i32([n - 1 for n in lens]), seq_slot=i32(list(range(B))),
                B=B, H=H, K=K, hd=hd, dense=dense, lens=list(lens))


def call(fn, c, out, splits, extra=()):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    i = ctypes.c_int
    return fn(p(c["q"]), i(c["q"].stride(0)), p(c["k"]), p(c["v"]), p(c["seq_start"]), p(c["seq_pos0"]),
              p(c["seq_slot"]), p(c["table"]), i(c["max_pages"]), i(c["page"]), p(out), i(c["B"]), i(c["B"]), i(1),
              i(c["H"]), i(c["K"]), i(c["hd"]), i(0), ctypes.c_float(1.0 / math.sqrt(c["hd"])), i(splits), *extra,
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_entry_point_matches_the_ordinary_one_twice():
    from mdma_b200.csrc import build
    lib = build.load("noalloc")            # the exported C symbols, nothing in between
    ordinary = build.load("tensor")
    lib.mdma_last_error.restype = ctypes.c_char_p
    torch.cuda.set_device(0)
    for round_, (seed, lens, H, K, hd, splits) in enumerate([(0, [700, 65, 1, 300], 8, 2, 128, 4),
                                                             (1, [130, 512, 2000], 12, 3, 128, 6)]):
        c = make_case(seed, lens, H, K, hd)
        want = torch.zeros(c["B"], H * hd, dtype=torch.bfloat16, device=DEV)
        need = c["B"] * H * splits * (hd + 2)
        scratch = torch.empty(need, dtype=torch.float32, device=DEV)
        rc = call(ordinary.mdma_attention_mma, c, want, splits,
                  extra=(ctypes.c_void_p(scratch.data_ptr()), ctypes.c_long(need)))
        assert rc == 0, ordinary.mdma_last_error()
        got = torch.full_like(want, 7.0)
        free_before = torch.cuda.mem_get_info()[0]
        rc = call(lib.mdma_attention_mma_noalloc, c, got, splits)
        assert rc == 0, lib.mdma_last_error()
        torch.cuda.synchronize()
        if round_ == 1:        # by the second call the set-up is done: the call itself takes no device memory
            assert torch.cuda.mem_get_info()[0] >= free_before
        # the same kernels with the same splits: the same bits
        assert torch.equal(got, want), f"call {round_}: differs from the ordinary entry point"
        # and right: the attention formula in float64 (tolerance of the kernel tests)
        from test_kernels import reference_attention
        ref = reference_attention(c["q"][:, :H * hd].double().cpu().reshape(c["B"], H, hd), c["dense"],
                                  list(range(c["B"])), [n - 1 for n in c["lens"]], 1.0 / math.sqrt(hd), 0)
        err = (got.double().cpu() - ref).abs()
        assert bool((err <= 2e-2 + 2e-2 * ref.abs()).all()), f"call {round_}: max difference {err.max().item()}"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from mdma_b200.csrc import build
    lib = build.load("noalloc")
    lib.mdma_last_error.restype = ctypes.c_char_p
    c = make_case(2, [64] * 4, 8, 2, 128)
    c["B"] = 2048                           # sizes only: the call must be refused before it touches memory
    out = torch.zeros(4, 8 * 128, dtype=torch.bfloat16, device=DEV)
    assert 2048 * 8 * 4 * 130 > MAX_FLOATS
    rc = call(lib.mdma_attention_mma_noalloc, c, out, 4)
    assert rc != 0
    msg = lib.mdma_last_error().decode()
    assert "floats" in msg and str(MAX_FLOATS) in msg
    torch.cuda.synchronize()
