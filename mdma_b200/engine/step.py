"""The engine: weights, cache, workspace and the one step function.

`Engine.step(entries)` takes, for each sequence of a batch, its slot, the
tokens it brings now and the places among them whose logits are wanted.  It
runs exactly those tokens as one flat batch (no padding is computed) on top of
what the cache holds and returns float32 logits [wanted, vocab].  Prompts of
unequal lengths go in one step, later steps bring one token per sequence;
more tokens at once on a filled cache (a prompt cut in pieces) work the same
way.  A request is checked as a whole before anything is launched; a bad one
leaves the cache untouched (the reference's rule for its single-sequence
prefill/forward: src/model.rs:338-353, 406-428).

Memory is planned before it is taken: weights, cache pages, per-sequence
state and workspace are added up and compared with the device's free memory
less a reserve (src/model/planning.rs:55-125, src/bin/mdma/run.rs:66-71).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache import SequenceCache
from ..config import load_config
from ..parts.base import Runtime
from ..weights import load_tensors, random_tensors, resident_dtype
from .model import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class StepError(ValueError):
    """The step's request is not valid; nothing was run and the cache is unchanged."""


class MemoryBudgetError(RuntimeError):
    """The plan does not fit the device."""

    def __init__(self, requested: int, available: int, plan: dict):
        self.requested, self.available, self.plan = requested, available, plan
        super().__init__(f"the memory plan needs {requested} bytes, {available} are available: {plan}")


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


class StepContext:
    """What the parts see of one forward pass."""

    def __init__(self, rt: Runtime, workspace: dict[str, torch.Tensor]):
        self.rt = rt
        self._workspace = workspace
        self.n_tokens = self.n_seqs = self.n_want = 0
        self.max_new = self.max_len = 0
        self.ids = self.tok_seq = self.tok_pos = self.seq_slot = self.seq_start = self.seq_pos0 = None
        self.want_rows = None

    def buf(self, name: str, cols: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        t = self._workspace.get(name)
        if t is None:
            raise KeyError(f"no workspace buffer {name!r}; a part must declare it in workspace()")
        if t.shape[1] != cols:
            t = t[:, :cols] if t.shape[1] > cols else None
        if t is None or (dtype is not None and t.dtype != dtype):
            raise KeyError(f"workspace buffer {name!r} does not have {cols} columns of {dtype}")
        return t


def memory_plan(model: DecoderModel, expected, dtype, max_tokens, max_slots, max_context, page_size,
                chunk_tokens, stored: Optional[dict] = None) -> dict:
    """Bytes the engine will hold, from sizes alone (src/model/planning.rs:55-125).  `stored` gives
    the dtype each tensor has in the file (vectors stay as stored); without it bfloat16 is assumed."""
    elem = 4 if dtype == torch.float32 else 2
    weights = 0
    for name, ts in expected.items():
        n = int(np.prod(ts.shape))
        held = resident_dtype(ts, (stored or {}).get(name, torch.bfloat16), dtype)
        weights += n * torch.empty((), dtype=held).element_size()
    cache = SequenceCache(model.kv_needs(), model.state_needs(), max_tokens, max_slots, max_context, dtype,
                          "meta", page_size, allocate=False)
    ws = sum(chunk_tokens * cols * (4 if kind == "f32" else elem)
             for cols, kind in model.workspace_columns().values())
    return {"weights_bytes": weights, "cache_bytes": cache.bytes, "workspace_bytes": ws,
            "total_bytes": weights + cache.bytes + ws, "cache_pages": cache.n_pages,
            "page_size": page_size, "slots": max_slots, "chunk_tokens": chunk_tokens}


def plan_only(model_dir: str, dtype="bfloat16", max_batch: int = 1, max_context: Optional[int] = None,
              chunk_tokens: int = 8192, page_size: int = 64) -> dict:
    """The memory plan of a model folder without touching a device or reading weights."""
    arch, config = load_config(model_dir)
    spec = arch.describe(config)
    model = DecoderModel(spec)
    ctx = int(max_context or spec.max_positions)
    max_tokens = max_batch * (-(-ctx // page_size)) * page_size
    stored = {}
    try:
        from ..weights import open_model_files
        for sf in open_model_files(model_dir):
            stored.update({n: e.dtype for n, e in sf.entries.items()})
    except Exception:
        stored = None                       # a folder without weights can still be planned
    return memory_plan(model, model.expected_tensors(), _DTYPES[dtype], max_tokens, max_batch, ctx,
                       page_size, max(1, min(chunk_tokens, max_tokens)), stored)


class Engine:
    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[dict] = None,
                 seed: Optional[int] = None, dtype="bfloat16", max_tokens: Optional[int] = None,
                 max_batch: int = 8, max_context: Optional[int] = None, chunk_tokens: int = 8192,
                 device="cuda:0", reserve_mib: int = 256, kernels: str = "auto", page_size: int = 64,
                 vram_bytes: Optional[int] = None, context_hint: Optional[int] = None):
        if dtype not in _DTYPES:
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")
        self.dtype = _DTYPES[dtype]
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; the engine has no CPU path")
        if (model_dir is None) == (config is None):
            raise ValueError("give either a model folder or a configuration dictionary (with a seed)")
        self.arch, self.config = load_config(model_dir if model_dir is not None else config)
        self.spec = self.arch.describe(self.config)
        self.model = DecoderModel(self.spec)
        self.vocab_size = self.spec.vocab_size

        self.max_context = int(max_context or self.spec.max_positions)
        if max_context is None and context_hint is not None:
            # a caller that knows its longest sequence need not pay for the model's full context
            self.max_context = max(1, min(self.max_context, int(context_hint)))
        self.page_size = page_size
        pages_per_seq = -(-self.max_context // page_size)
        if max_tokens is None:
            max_tokens = max_batch * pages_per_seq * page_size
            self.max_slots = max_batch
        else:
            self.max_slots = max(1, min(-(-max_tokens // page_size), 4096))
        self.max_tokens = -(-int(max_tokens) // page_size) * page_size
        self.chunk_tokens = max(1, min(int(chunk_tokens), self.max_tokens))

        if kernels == "auto":
            kernels = "tensor" if self.dtype == torch.bfloat16 else "plain"
        if kernels not in ("tensor", "plain"):
            raise ValueError("kernels must be 'auto', 'tensor' or 'plain'")
        if kernels == "tensor" and self.dtype != torch.bfloat16:
            raise ValueError("the tensor-core kernels are bfloat16 only")
        self.rt = Runtime(self.dtype, self.device,
                          gemm="tensor" if kernels == "tensor" else "simt",
                          attention="fast" if kernels == "tensor" else "simple")

        # ---- plan, then allocate ----------------------------------------
        expected = self.model.expected_tensors()
        stored = None
        if model_dir is not None:
            from ..weights import open_model_files
            stored = {n: e.dtype for sf in open_model_files(model_dir) for n, e in sf.entries.items()}
        self.plan = self._plan(expected, stored)
        free, _total = torch.cuda.mem_get_info(self.device)
        if vram_bytes is not None:
            free = min(free, int(vram_bytes))
        need = self.plan["total_bytes"] + reserve_mib * (1 << 20)
        if need > free:
            raise MemoryBudgetError(need, free, self.plan)

        with torch.cuda.device(self.device):
            if model_dir is not None:
                tensors = load_tensors(model_dir, expected, self.dtype, self.device)
            else:
                if seed is None:
                    raise ValueError("random weights need a seed")
                tensors = {}
                for name, ts in expected.items():
                    stored = torch.float32 if self.dtype == torch.float32 else torch.bfloat16
                    tensors.update(random_tensors({name: ts}, seed,
                                                  resident_dtype(ts, stored, self.dtype), self.device))
            self.model.bind(tensors, self.rt)
            del tensors
            self.cache = SequenceCache(self.model.kv_needs(), self.model.state_needs(), self.max_tokens,
                                       self.max_slots, self.max_context, self.dtype, self.device, page_size)
            self.workspace = {}
            for name, (cols, kind) in self.model.workspace_columns().items():
                dt = torch.float32 if kind == "f32" else self.dtype
                self.workspace[name] = torch.empty((self.chunk_tokens, cols), dtype=dt, device=self.device)
            # step metadata goes up in one copy from pinned memory; two host buffers
            # take turns so that one can be filled while the other's copy is in flight
            self._meta_cap = 6 * self.chunk_tokens + 4 * self.max_slots + 16
            self._meta_host = [torch.empty(self._meta_cap, dtype=torch.int32).pin_memory() for _ in range(2)]
            self._meta_event = [torch.cuda.Event() for _ in range(2)]
            self._meta_turn = 0
            self._meta_dev = torch.empty(self._meta_cap, dtype=torch.int32, device=self.device)
        self.ctx = StepContext(self.rt, self.workspace)
        self.forward_passes = 0

    # ---- planning ----------------------------------------------------------
    def _plan(self, expected, stored=None) -> dict:
        return memory_plan(self.model, expected, self.dtype, self.max_tokens, self.max_slots,
                           self.max_context, self.page_size, self.chunk_tokens, stored)

    def held_bytes(self) -> dict:
        """Bytes actually resident, in the plan's categories."""
        cache = sum(g.k.numel() * g.k.element_size() * 2 + g.table_host.nbytes for g in self.cache.groups)
        cache += sum(t.numel() * t.element_size() for t in self.cache.states.values())
        ws = sum(t.numel() * t.element_size() for t in self.workspace.values())
        return {"weights_bytes": self.model.resident_bytes(), "cache_bytes": cache, "workspace_bytes": ws}

    def generate(self, prompts, max_tokens: int = 32, temperature: float = 0.0, seed: int = 0,
                 stop_ids=None, top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
                 repetition_window: int = 64, use_graphs: bool = True):
        """Generate from token-id prompts on this engine; see `mdma_b200.generate`."""
        from ..sampling.params import SamplingParams
        from ..sampling.sampler import DeviceSampler
        from .generate import Generator
        if getattr(self, "_generator", None) is None:
            self._generator = Generator(self, DeviceSampler(self.vocab_size, self.max_slots, self.device), use_graphs)
        params = SamplingParams(temperature, top_p, min_p, repetition_penalty, repetition_window, seed)
        stop = self.spec.stop_token_ids if stop_ids is None else stop_ids
        return self._generator.generate(prompts, max_tokens, params, stop)

    def decode_session(self, sampler, params=None):
        """A `DecodeSession` over this engine (decode steps replayed as CUDA graphs)."""
        from .graphs import DecodeSession
        return DecodeSession(self, sampler, params)

    # ---- sequences ---------------------------------------------------------
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def fits(self, sizes) -> bool:
        """Whether sequences of (prompt length, token budget) can be live together in an empty cache."""
        if len(sizes) > self.max_slots:
            return False
        pages = sum(-(-(p + b - 1) // self.page_size) for p, b in sizes)
        return pages <= self.cache.n_pages and all(p + b - 1 <= self.max_context for p, b in sizes)

    # ---- the step ----------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one sequence")
        seen = set()
        for e in entries:
            if e.slot not in self.cache.lengths:
                raise StepError(f"slot {e.slot} is not held by a sequence")
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"the sequence in slot {e.slot} brings no tokens")
            toks = np.asarray(e.tokens)
            if toks.dtype.kind not in "iu" or toks.ndim != 1:
                raise StepError(f"token ids of slot {e.slot} must be a flat list of integers")
            lo, hi = int(toks.min()), int(toks.max())
            if lo < 0 or hi >= self.vocab_size:
                bad = lo if lo < 0 else hi
                raise StepError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"wanted place {w} is outside the {n} tokens of slot {e.slot}")
        why = self.cache.can_extend({e.slot: len(e.tokens) for e in entries})
        if why:
            raise StepError(why)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens; returns float32 logits [sum of wants, vocab] on the device,
        in the order of the entries and of each entry's `want`."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._validate(entries)
        ext = {e.slot: len(e.tokens) for e in entries}
        self.cache.extend(ext)
        n_want = sum(len(e.want) for e in entries)
        logits = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.device)
        # where each wanted row goes in the result: entries' order, then want's order
        out_row = {}
        r = 0
        for i, e in enumerate(entries):
            for w in e.want:
                out_row.setdefault((i, int(w)), []).append(r)
                r += 1
        # cut the flat token list into passes of at most chunk_tokens tokens
        cursor = [0] * len(entries)
        base = [self.cache.length(e.slot) for e in entries]
        while True:
            room = self.chunk_tokens
            pieces = []
            for i, e in enumerate(entries):
                left = len(e.tokens) - cursor[i]
                if left <= 0 or room <= 0:
                    continue
                take = min(left, room)
                pieces.append((i, cursor[i], take))
                room -= take
            if not pieces:
                break
            self._forward(entries, pieces, base, out_row, logits)
            for i, start, take in pieces:
                cursor[i] = start + take
        self.cache.commit(ext)
        return logits

    def _forward(self, entries, pieces, base, out_row, logits) -> None:
        ids, tok_seq, tok_pos, seq_slot, seq_start, seq_pos0 = [], [], [], [], [0], []
        want_rows, dest_rows = [], []
        max_new = max_len = 0
        n_rows = 0
        for s, (i, start, take) in enumerate(pieces):
            e = entries[i]
            pos0 = base[i] + start
            seq_slot.append(e.slot)
            seq_pos0.append(pos0)
            first_row = n_rows
            ids.append(np.asarray(e.tokens[start:start + take], dtype=np.int32))
            tok_seq.append(np.full(take, s, dtype=np.int32))
            tok_pos.append(np.arange(pos0, pos0 + take, dtype=np.int32))
            n_rows += take
            seq_start.append(n_rows)
            max_new = max(max_new, take)
            max_len = max(max_len, pos0 + take)
            for j in sorted({int(w) for w in e.want}):
                if start <= j < start + take:
                    for dest in out_row.get((i, j), ()):
                        want_rows.append(first_row + j - start)
                        dest_rows.append(dest)
        if want_rows:          # keep the result rows in the order of the entries and of each `want`
            order = sorted(range(len(dest_rows)), key=dest_rows.__getitem__)
            want_rows = [want_rows[k] for k in order]
            dest_rows = [dest_rows[k] for k in order]
        ids, tok_seq, tok_pos = np.concatenate(ids), np.concatenate(tok_seq), np.concatenate(tok_pos)
        T, B, W = len(ids), len(pieces), len(want_rows)
        fields = [ids, tok_seq, tok_pos, seq_slot, seq_start, seq_pos0, want_rows]
        flat = np.concatenate([np.asarray(f, dtype=np.int32) for f in fields]) if T else None
        n = flat.size
        if n > self._meta_cap:
            raise StepError("too many wanted places for one pass")
        turn = self._meta_turn = self._meta_turn ^ 1
        self._meta_event[turn].synchronize()
        self._meta_host[turn][:n].copy_(torch.from_numpy(flat))
        self._meta_dev[:n].copy_(self._meta_host[turn][:n], non_blocking=True)
        self._meta_event[turn].record()
        ctx = self.ctx
        off = 0
        views = []
        for f in fields:
            views.append(self._meta_dev[off:off + len(f)])
            off += len(f)
        (ctx.ids, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, ctx.seq_start, ctx.seq_pos0, ctx.want_rows) = views
        ctx.n_tokens, ctx.n_seqs, ctx.n_want = T, B, W
        ctx.max_new, ctx.max_len = max_new, max_len
        ctx.host_seq_new = [take for _, _, take in pieces]
        ctx.host_seq_pos0 = list(seq_pos0)
        ctx.host_seq_slot = list(seq_slot)
        contiguous = dest_rows == list(range(dest_rows[0], dest_rows[0] + W)) if W else True
        if W and contiguous:
            out = logits[dest_rows[0]:dest_rows[0] + W]
            self.model.forward(ctx, self.cache, out)
        elif W:
            tmp = torch.empty((W, self.vocab_size), dtype=torch.float32, device=self.device)
            self.model.forward(ctx, self.cache, tmp)
            logits.index_copy_(0, torch.as_tensor(dest_rows, device=self.device), tmp)
        else:
            self.model.forward(ctx, self.cache, None)
        self.forward_passes += 1
