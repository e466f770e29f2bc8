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
from ..weights import load_tensors, random_tensor, resident_dtype, stored_dtypes
from .arena import Carver
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
        self.most_seqs = None               # the most sequences the engine holds (kernels may plan for it)
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


class Layout:
    """Everything an engine keeps on the device, as views of its arena (None when only planned)."""
    pass


def lay_out(model: DecoderModel, carver: Carver, *, dtype, device, sms: int, max_tokens: int, max_slots: int,
            max_context: int, page_size: int, chunk_tokens: int, logit_rows: int, history_cap: int,
            run_ahead: int = 8, stored: Optional[dict] = None) -> Layout:
    """Carve the engine's memory, in a fixed order: weights, cache, workspace, logits, step
    metadata, sampler, kernel scratch, tables the parts derive.  Run with a planning carver this
    is the memory plan (src/model/planning.rs:55-125); run over the arena it is the allocation."""
    from ..sampling.sampler import DeviceSampler
    lay = Layout()
    expected = model.expected_tensors()

    def held(name, ts):
        return resident_dtype(ts, (stored or {}).get(name, torch.bfloat16), dtype)
    lay.tensors = model.lay_out_weights(expected, held, carver.taker("weights"))
    lay.cache = SequenceCache(model.kv_needs(), model.state_needs(), max_tokens, max_slots, max_context, dtype,
                              device, page_size, alloc=carver.taker("cache"))
    lay.workspace = {}
    for name, (cols, kind) in model.workspace_columns().items():
        dt = torch.float32 if kind == "f32" else dtype
        lay.workspace[name] = carver.take("workspace", (chunk_tokens, cols), dt)
    lay.logits = carver.take("logits", (logit_rows, model.spec.vocab_size), torch.float32)
    lay.meta_cap = 6 * chunk_tokens + 4 * max_slots + logit_rows + 16
    lay.meta_dev = carver.take("metadata", (lay.meta_cap,), torch.int32)
    # the replayed decode step reads its inputs from here: ids, positions (twice), slots, 0..cap
    lay.decode = {name: carver.take("metadata", (max_slots + (1 if name == "arange" else 0),), torch.int32)
                  for name in ("ids", "tok_pos", "seq_slot", "seq_pos0", "arange")}
    lay.sampler = DeviceSampler(model.spec.vocab_size, max_slots, device, history_cap, alloc=carver.taker("sampler"))
    # the result words (tokens, flags, status) of the last `run_ahead` replayed decode steps
    lay.token_ring = carver.take("sampler", (max(1, run_ahead), 2 * max_slots + 4), torch.int32)
    lay.ring_counter = carver.take("sampler", (1,), torch.int32)
    shapes = []
    for b in model.blocks:
        m = b.mixer
        if all(hasattr(m, a) for a in ("n_heads", "n_kv_heads", "head_dim")):
            shapes.append((m.n_heads, m.n_kv_heads, m.head_dim))
    floats = 0
    if dtype == torch.bfloat16:
        from .. import ops_tensor
        floats = ops_tensor.scratch_floats_bound(sms, chunk_tokens, max_slots, shapes)
    lay.scratch_floats = floats
    lay.tc_sk_flags = carver.take("kernel_scratch", (max(512, 4 * sms),), torch.int32)
    lay.tc_scratch = carver.take("kernel_scratch", (max(floats, 1),), torch.float32)
    lay.tables = carver.take("tables", (max(model.device_tensor_bytes(), 1),), torch.uint8)
    return lay


def _plan_dict(carver: Carver, cache: SequenceCache, page_size, max_slots, chunk_tokens, logit_rows) -> dict:
    plan = {f"{k}_bytes": v for k, v in carver.by_category.items()}
    plan.update(total_bytes=carver.offset, cache_pages=cache.n_pages, page_size=page_size, slots=max_slots,
                chunk_tokens=chunk_tokens, logit_rows=logit_rows)
    return plan


def plan_only(model_dir: str, dtype="bfloat16", max_batch: int = 1, max_context: Optional[int] = None,
              chunk_tokens: int = 8192, page_size: int = 64, sms: int = 148, history_cap: int = 256) -> dict:
    """The memory plan of a model folder without touching a device or reading weights.  `sms`:
    the multiprocessor count the kernels' scratch is sized for (a B200 has 148)."""
    arch, config = load_config(model_dir)
    spec = arch.describe(config)
    model = DecoderModel(spec)
    ctx = int(max_context or spec.max_positions)
    max_tokens = max_batch * (-(-ctx // page_size)) * page_size
    try:
        stored = stored_dtypes(model_dir)
    except Exception:
        stored = None                       # a folder without weights can still be planned
    chunk = max(1, min(chunk_tokens, max_tokens), max_batch)
    carver = Carver()
    lay = lay_out(model, carver, dtype=_DTYPES[dtype], device="meta", sms=sms, max_tokens=max_tokens,
                  max_slots=max_batch, max_context=ctx, page_size=page_size, chunk_tokens=chunk,
                  logit_rows=max_batch, history_cap=history_cap, stored=stored)
    return _plan_dict(carver, lay.cache, page_size, max_batch, chunk, max_batch)


class Engine:
    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[dict] = None,
                 seed: Optional[int] = None, dtype="bfloat16", max_tokens: Optional[int] = None,
                 max_batch: int = 8, max_context: Optional[int] = None, chunk_tokens: int = 8192,
                 device="cuda:0", reserve_mib: int = 256, kernels: str = "auto", page_size: int = 64,
                 vram_bytes: Optional[int] = None, context_hint: Optional[int] = None,
                 logit_rows: Optional[int] = None, history_cap: int = 256, init_std: Optional[float] = None,
                 run_ahead: int = 8):
        """`logit_rows`: the most places one step may want logits at (default: one per sequence slot);
        `history_cap`: the longest repetition window the sampler keeps room for; `run_ahead`: how many
        replayed decode steps may run before the host reads their tokens; `init_std`: the standard
        deviation of seeded random matrices (default 0.02)."""
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
        if model_dir is None and seed is None:
            raise ValueError("random weights need a seed")
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
        # a pass holds at least one token of every slot: the replayed decode step runs all live sequences at once
        self.chunk_tokens = max(1, min(int(chunk_tokens), self.max_tokens), self.max_slots)
        # (never fewer than the slots: the replayed decode step writes a row of logits per live sequence)
        self.logit_rows = max(1, int(logit_rows if logit_rows is not None else self.max_slots), self.max_slots)

        if kernels == "auto":
            kernels = "tensor" if self.dtype == torch.bfloat16 else "plain"
        if kernels not in ("tensor", "plain"):
            raise ValueError("kernels must be 'auto', 'tensor' or 'plain'")
        if kernels == "tensor" and self.dtype != torch.bfloat16:
            raise ValueError("the tensor-core kernels are bfloat16 only")
        self.rt = Runtime(self.dtype, self.device,
                          gemm="tensor" if kernels == "tensor" else "simt",
                          attention="fast" if kernels == "tensor" else "simple")
        # sizes the kernels cannot take are refused here, before anything is read or allocated
        # (the reference's backend limit at admission: src/model/arch/llama/preflight.rs:35-42)
        for part in self.model.all_parts():
            check = getattr(part, "check_limits", None)
            if check is not None:
                check(self.rt)

        # ---- plan, then allocate ----------------------------------------
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        stored = stored_dtypes(model_dir) if model_dir is not None else None
        if stored is not None:          # the folder's headers are checked before the device is touched
            from ..weights import check_entries, open_model_files
            entries = {}
            for sf in open_model_files(model_dir):
                entries.update(sf.entries)
            check_entries(entries, self.model.expected_tensors(), where=model_dir)
        sizes = dict(dtype=self.dtype, device=self.device, sms=sms, max_tokens=self.max_tokens,
                     max_slots=self.max_slots, max_context=self.max_context, page_size=page_size,
                     chunk_tokens=self.chunk_tokens, logit_rows=self.logit_rows, history_cap=history_cap,
                     run_ahead=run_ahead, stored=stored)
        planner = Carver()
        planned = lay_out(self.model, planner, **sizes)
        self.plan = _plan_dict(planner, planned.cache, page_size, self.max_slots, self.chunk_tokens, self.logit_rows)
        free, _total = torch.cuda.mem_get_info(self.device)
        if vram_bytes is not None:
            free = min(free, int(vram_bytes))
        need = self.plan["total_bytes"] + reserve_mib * (1 << 20)
        if need > free:
            raise MemoryBudgetError(need, free, self.plan)

        with torch.cuda.device(self.device):
            self.arena = torch.zeros(self.plan["total_bytes"], dtype=torch.uint8, device=self.device)
            carver = Carver(self.arena)
            lay = lay_out(self.model, carver, **sizes)
            assert carver.offset == planner.offset and carver.by_category == planner.by_category
            self._held = dict(carver.by_category)
            expected = self.model.expected_tensors()
            if model_dir is not None:
                load_tensors(model_dir, expected, self.dtype, self.device, into=lay.tensors)
            else:
                from ..weights.random_init import INIT_STD, quantile_table
                table = torch.from_numpy(quantile_table()).to(self.device)
                for name, ts in expected.items():
                    random_tensor(name, ts, seed, lay.tensors[name].dtype, out=lay.tensors[name], table=table,
                                  std=INIT_STD if init_std is None else init_std)
                torch.cuda.synchronize(self.device)
                del table
            self.sampler = lay.sampler
            if self.rt.gemm == "tensor":
                from .. import ops_tensor
                # the kernels' status word lies beside the sampler's tokens: one copy brings both to the host
                self.rt.tc = ops_tensor.TensorState(self.device, lay.scratch_floats, sms=sms, status=self.sampler.extra,
                                                    sk_flags=lay.tc_sk_flags, scratch=lay.tc_scratch)
            tables = Carver(lay.tables)
            self.rt.alloc = tables.taker("tables")
            self.model.bind(lay.tensors, self.rt)
            self.cache = lay.cache
            self.workspace = lay.workspace
            self.logits = lay.logits
            self.decode_buffers = lay.decode
            self.token_ring, self.ring_counter = lay.token_ring, lay.ring_counter
            self.decode_buffers["arange"].copy_(torch.arange(self.max_slots + 1, dtype=torch.int32))
            # step metadata goes up in one copy from pinned memory; two host buffers
            # take turns so that one can be filled while the other's copy is in flight
            self._meta_cap = lay.meta_cap
            self._meta_host = [torch.empty(self._meta_cap, dtype=torch.int32).pin_memory() for _ in range(2)]
            self._meta_event = [torch.cuda.Event() for _ in range(2)]
            self._meta_turn = 0
            self._meta_dev = lay.meta_dev
            self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
            self._status_event = None
        self.ctx = StepContext(self.rt, self.workspace)
        self.ctx.most_seqs = self.max_slots
        self.forward_passes = 0
        self.h2d_bytes = self.d2h_bytes = 0     # bytes of step inputs copied up / results copied down so far
        self._session = None
        self._generator = None

    # ---- planning ----------------------------------------------------------
    def memory_plan(self) -> dict:
        return dict(self.plan)

    def held_bytes(self) -> dict:
        """Bytes actually resident, in the plan's categories: the arena is the only device memory
        the engine keeps, carved by the function that made the plan."""
        held = {f"{k}_bytes": v for k, v in self._held.items()}
        held["total_bytes"] = self.arena.numel()
        return held

    # ---- kernel status -------------------------------------------------------
    def check_status(self, sync: bool = True) -> None:
        """Raise `KernelError` if a tensor-core kernel gave up on a bounded wait since the last
        check (its output is then not valid).  `sync=False` looks only at the copy of the status
        word that the last `step` left on the host, if it has arrived."""
        tc = self.rt.tc
        if tc is None:
            return
        if sync:
            self._status_host.copy_(tc.status, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        elif self._status_event is None or not self._status_event.query():
            return
        self._status_event = None
        self.raise_on_status(int(self._status_host[0]))

    def raise_on_status(self, word: int) -> None:
        if word != 0:
            from ..ops import KernelError
            self.rt.tc.clear()
            raise KernelError(f"a tensor-core kernel ran into its wait limit (status {word}); "
                              "the results of this step are not valid")

    def generate(self, prompts, max_tokens: int = 32, temperature: float = 0.0, seed: int = 0,
                 stop_ids=None, top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
                 repetition_window: int = 64, use_graphs: bool = True):
        """Generate from token-id prompts on this engine; see `mdma_b200.generate`."""
        from ..sampling.params import SamplingParams
        from .generate import Generator
        if self._generator is None:
            self._generator = Generator(self)
        params = SamplingParams(temperature, top_p, min_p, repetition_penalty, repetition_window, seed)
        stop = self.spec.stop_token_ids if stop_ids is None else stop_ids
        return self._generator.generate(prompts, max_tokens, params, stop, use_graphs=use_graphs)

    def decode_session(self):
        """The engine's `DecodeSession` (decode steps replayed as CUDA graphs).  There is one:
        its graphs serve every request, whatever its sampling options."""
        from .graphs import DecodeSession
        if self._session is None:
            self._session = DecodeSession(self)
        return self._session

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
            if len({int(w) for w in e.want}) != len(e.want):
                raise StepError(f"a wanted place of slot {e.slot} is listed twice")
        n_want = sum(len(e.want) for e in entries)
        if n_want > self.logit_rows:
            raise StepError(f"the step wants logits at {n_want} places, the engine has room for "
                            f"{self.logit_rows} (Engine(logit_rows=...))")
        why = self.cache.can_extend({e.slot: len(e.tokens) for e in entries})
        if why:
            raise StepError(why)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens; returns float32 logits [sum of wants, vocab] on the device,
        in the order of the entries and of each entry's `want`.  The result is a view of the
        engine's own logits buffer: it holds until the next step."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._validate(entries)
        self.check_status(sync=False)
        ext = {e.slot: len(e.tokens) for e in entries}
        self.cache.extend(ext)
        n_want = sum(len(e.want) for e in entries)
        logits = self.logits[:n_want]
        # where each wanted row goes in the result: entries' order, then want's order
        out_row = {}
        r = 0
        for i, e in enumerate(entries):
            for w in e.want:
                out_row[(i, int(w))] = r
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
        if self.rt.tc is not None:
            # the kernels' status word follows the step to the host; the next step (or
            # `check_status`) looks at it, so a wait that ran out does not pass unnoticed
            self._status_host.copy_(self.rt.tc.status, non_blocking=True)
            self._status_event = torch.cuda.Event()
            self._status_event.record()
        return logits

    def _forward(self, entries, pieces, base, out_row, logits) -> None:
        ids, tok_seq, tok_pos, seq_slot, seq_start, seq_pos0 = [], [], [], [], [0], []
        wanted = []                     # (row of the result, row of this pass)
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
            for w in e.want:
                if start <= int(w) < start + take:
                    wanted.append((out_row[(i, int(w))], first_row + int(w) - start))
        wanted.sort()                   # in the order of the result rows
        want_rows = [row for _, row in wanted]
        ids, tok_seq, tok_pos = np.concatenate(ids), np.concatenate(tok_seq), np.concatenate(tok_pos)
        T, B, W = len(ids), len(pieces), len(want_rows)
        fields = [ids, tok_seq, tok_pos, seq_slot, seq_start, seq_pos0, want_rows]
        flat = np.concatenate([np.asarray(f, dtype=np.int32) for f in fields])
        n = flat.size
        assert n <= self._meta_cap
        turn = self._meta_turn = self._meta_turn ^ 1
        self._meta_event[turn].synchronize()
        self._meta_host[turn][:n].copy_(torch.from_numpy(flat))
        self._meta_dev[:n].copy_(self._meta_host[turn][:n], non_blocking=True)
        self._meta_event[turn].record()
        self.h2d_bytes += 4 * n
        ctx = self.ctx
        off = 0
        views = []
        for f in fields:
            views.append(self._meta_dev[off:off + len(f)])
            off += len(f)
        (ctx.ids, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, ctx.seq_start, ctx.seq_pos0, ctx.want_rows) = views
        ctx.n_tokens, ctx.n_seqs, ctx.n_want = T, B, W
        ctx.max_new, ctx.max_len = max_new, max_len
        ctx.decode_only = False
        ctx.host_seq_new = [take for _, _, take in pieces]
        ctx.host_seq_pos0 = list(seq_pos0)
        ctx.host_seq_slot = list(seq_slot)
        self.model.forward(ctx, self.cache, None)
        # logits of the wanted rows, written where they belong: one head call per run of result
        # rows that follow one another (one run, unless a `want` list is out of order across a cut)
        k = 0
        while k < W:
            j = k + 1
            while j < W and wanted[j][0] == wanted[j - 1][0] + 1:
                j += 1
            dest0 = wanted[k][0]
            self.model.logits_of(ctx, ctx.want_rows[k:j], j - k, logits[dest0:dest0 + (j - k)])
            k = j
        self.forward_passes += 1
