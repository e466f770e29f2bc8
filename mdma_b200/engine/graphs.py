"""Decode steps as CUDA graphs.

A decode step of B live sequences is a fixed chain of a few hundred small
kernels; launched one by one the host is slower than the device.  A
`DecodeSession` keeps the step's inputs (token ids, positions, slots) in fixed
device buffers, captures forward + token selection + "advance" once per batch
size and replays it: the sampled tokens become the next step's inputs on the
device, the host only reserves cache pages ahead and reads the tokens back.
The reference replays its single-sequence decode the same way, with (token,
position) read from device memory so that replay needs no re-capture
(src/backend/cuda/graph.rs:46-49, 217-250); its test asks for logits equal to
the eager path's (src/backend/test_support/graph.rs:16-75), and so does ours.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from ..sampling.params import SamplingParams
from ..cache.slots import CacheFull
from .step import StepContext, StepError


class DecodeSession:
    def __init__(self, engine, sampler, params: Optional[SamplingParams] = None):
        self.engine, self.sampler = engine, sampler
        self.params = params or SamplingParams.greedy()
        self.graphs: dict = {}
        self.slots: list[int] = []
        self.requests: list[int] = []
        dev, cap = engine.device, engine.max_slots
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
        self.ids, self.tok_pos, self.seq_slot, self.seq_pos0 = i32(cap), i32(cap), i32(cap), i32(cap)
        self.arange = torch.arange(cap + 1, dtype=torch.int32, device=dev)
        self.logits = torch.empty((cap, engine.vocab_size), dtype=torch.float32, device=dev)
        self._host = torch.empty(3 * cap, dtype=torch.int32).pin_memory()
        self._host_np = self._host.numpy()            # the same pinned words, written without a tensor in between
        self._tok_host = torch.empty(2 * sampler.max_rows, dtype=torch.int32).pin_memory()
        self.ctx = StepContext(engine.rt, engine.workspace)
        self.steps_done: list[int] = []
        self.launches_per_step = 0          # kernels in one step (counted at the eager first run)
        self._state_stale, self._use_hist = True, False
        self._bucket = engine.max_context

    @property
    def graph_safe(self) -> bool:
        return all(getattr(b.mixer, "graph_safe", False) for b in self.engine.model.blocks)

    # ---- membership ------------------------------------------------------
    def start(self, slots: Sequence[int], tokens: Sequence[int], requests: Optional[Sequence[int]] = None,
              steps: Optional[Sequence[int]] = None) -> None:
        """Set the live sequences: their slots and the token each feeds next."""
        B = len(slots)
        if B == 0 or B > self.engine.max_slots:
            raise StepError(f"a decode session takes 1..{self.engine.max_slots} sequences")
        self.slots = list(slots)
        self._state_stale = True
        self.requests = list(requests) if requests is not None else list(range(B))
        self.steps_done = list(steps) if steps is not None else [0] * B
        pos = [self.engine.cache.length(s) for s in slots]
        cap = self.engine.max_slots
        h = self._host
        h[:B] = torch.as_tensor(list(tokens), dtype=torch.int32)
        h[cap:cap + B] = torch.as_tensor(pos, dtype=torch.int32)
        h[2 * cap:2 * cap + B] = torch.as_tensor(self.slots, dtype=torch.int32)
        torch.cuda.current_stream().synchronize()
        self.ids[:B].copy_(h[:B], non_blocking=True)
        self.tok_pos[:B].copy_(h[cap:cap + B], non_blocking=True)
        self.seq_pos0[:B].copy_(h[cap:cap + B], non_blocking=True)
        self.seq_slot[:B].copy_(h[2 * cap:2 * cap + B], non_blocking=True)

    def feed(self, tokens: Sequence[int]) -> None:
        """The same sequences go on: only this step's input tokens go up (from pinned memory,
        asynchronously; positions and slots are already on the device).  The caller has read the
        previous step's tokens, so the staging buffer is free."""
        B = len(self.slots)
        if len(tokens) != B:
            raise StepError(f"{len(tokens)} tokens for {B} live sequences")
        self._host_np[:B] = tokens
        self.ids[:B].copy_(self._host[:B], non_blocking=True)

    # ---- one step ----------------------------------------------------------
    def _body(self, B: int) -> None:
        ctx = self.ctx
        ctx.ids, ctx.tok_pos, ctx.seq_slot, ctx.seq_pos0 = self.ids[:B], self.tok_pos[:B], self.seq_slot[:B], self.seq_pos0[:B]
        ctx.tok_seq, ctx.seq_start, ctx.want_rows = self.arange[:B], self.arange[:B + 1], self.arange[:B]
        ctx.n_tokens = ctx.n_seqs = ctx.n_want = B
        ctx.max_new, ctx.max_len = 1, self._bucket
        ctx.decode_only = True
        ctx.host_seq_new, ctx.host_seq_pos0, ctx.host_seq_slot = [1] * B, None, list(self.slots)
        self.engine.model.forward(ctx, self.engine.cache, self.logits[:B])
        p = self.params
        s = self.sampler
        if p.temperature <= 0.0 and (p.repetition_penalty == 1.0 or p.repetition_window == 0):
            ops.argmax(self.logits[:B], s.tokens, s.flags, B)
        else:
            # uniform numbers, step counts and histories live on the device (see `step_async`)
            s.sample_resident(self.logits[:B], p, self._use_hist)
        ops.advance_decode(s.tokens, self.ids, self.tok_pos, self.seq_pos0, B)

    def step_async(self, histories=None, use_graph: bool = True) -> None:
        """Run one decode step for the live sequences; tokens stay on the device."""
        B = len(self.slots)
        ext = {s: 1 for s in self.slots}
        try:
            self.engine.cache.extend(ext)
        except CacheFull as e:
            raise StepError(str(e)) from None
        p = self.params
        if self._state_stale and (p.temperature > 0.0 or (p.repetition_penalty != 1.0 and p.repetition_window > 0)):
            # once per batch: requests, step counts and recent tokens go up; from then on the sampling
            # kernel keeps them (it appends what it selects and counts the steps)
            self._use_hist = self.sampler.load_state(p, self.requests, self.steps_done, histories)
        self._state_stale = False
        # kernels choose their grids from an upper bound of the context: the live maximum rounded up
        # to 1024, so a graph stays valid until a sequence grows past its bucket
        longest = max(self.engine.cache.length(s_) for s_ in self.slots) + 1
        self._bucket = min(self.engine.max_context, -(-longest // 1024) * 1024)
        if use_graph and self.graph_safe:
            g = self.graphs.get((B, self._bucket, self._use_hist))
            if g is None:
                # The first step at this batch size runs eagerly (it loads kernels and sizes
                # scratch); the same chain is then captured, without running, for the next ones.
                before = ops.LAUNCHES
                self._body(B)
                self.launches_per_step = ops.LAUNCHES - before
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._body(B)
                self.graphs[(B, self._bucket, self._use_hist)] = g
            else:
                g.replay()
        else:
            self._body(B)
        self.engine.cache.commit(ext)
        self.steps_done = [n + 1 for n in self.steps_done]

    def read_tokens(self) -> tuple[list[int], list[int]]:
        """The tokens (and non-finite flags) the last step selected."""
        B, cap = len(self.slots), self.sampler.max_rows
        self._tok_host.copy_(self.sampler.tokens_and_flags.view(-1), non_blocking=True)     # one copy: 2 x rows integers
        torch.cuda.current_stream().synchronize()
        return self._tok_host[:B].tolist(), self._tok_host[cap:cap + B].tolist()
