"""Decode steps as CUDA graphs.

A decode step of B live sequences is a fixed chain of a few hundred small
kernels; launched one by one the host is slower than the device.  The
engine's `DecodeSession` keeps the step's inputs (token ids, positions, slots)
in fixed device buffers, captures forward + token selection + "advance" once
per batch size and replays it: the sampled tokens become the next step's
inputs on the device and are kept in a small ring, so several steps can run
back to back before the host reads their tokens in one copy.  The reference
replays its single-sequence decode the same way, with (token, position) read
from device memory so that replay needs no re-capture
(src/backend/cuda/graph.rs:46-49, 217-250); its test asks for logits equal to
the eager path's (src/backend/test_support/graph.rs:16-75), and so does ours.

One session serves every request: the sampling options and the seed live in
device memory that the sampling kernel reads, so graphs are keyed only by the
batch size, the length bucket (the attention kernel's grid depends on it) and
whether tokens are drawn or the largest logit is taken.
"""
from __future__ import annotations

import gc
from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..sampling.params import SamplingParams
from ..cache.slots import CacheFull
from .step import StepContext, StepError

BUCKET = 1024          # graphs are captured per this many positions of the longest sequence


class DecodeSession:
    def __init__(self, engine):
        self.engine, self.sampler = engine, engine.sampler
        self.params = SamplingParams.greedy()
        self.graphs: dict = {}
        self.slots: list[int] = []
        self.requests: list[int] = []
        cap = engine.max_slots
        b = engine.decode_buffers
        self.ids, self.tok_pos, self.seq_slot, self.seq_pos0, self.arange = (
            b["ids"], b["tok_pos"], b["seq_slot"], b["seq_pos0"], b["arange"])
        self.ring, self.ring_counter = engine.token_ring, engine.ring_counter
        self.logits = engine.logits
        self._host = torch.empty(3 * cap, dtype=torch.int32).pin_memory()
        self._host_np = self._host.numpy()            # the same pinned words, written without a tensor in between
        self._ring_host = torch.empty(tuple(self.ring.shape), dtype=torch.int32).pin_memory()
        self.ctx = StepContext(engine.rt, engine.workspace)
        self.ctx.most_seqs = engine.max_slots
        self.steps_done: list[int] = []
        self.launches_per_step = 0          # kernels in one step (counted at the eager first run)
        self._state_stale = True
        self._bucket = engine.max_context
        self._kept = 0                      # steps whose tokens wait in the ring
        self._steps_total = 0               # steps launched so far: the device's ring counter
        self._ring_base = 0                 # value of the ring counter at the first kept step

    @property
    def graph_safe(self) -> bool:
        return all(getattr(b.mixer, "graph_safe", False) for b in self.engine.model.blocks)

    @property
    def max_run(self) -> int:
        return self.ring.shape[0]

    # ---- membership ------------------------------------------------------
    def start(self, slots: Sequence[int], tokens: Sequence[int], requests: Optional[Sequence[int]] = None,
              steps: Optional[Sequence[int]] = None, params: Optional[SamplingParams] = None) -> None:
        """Set the live sequences: their slots and the token each feeds next."""
        B = len(slots)
        if B == 0 or B > self.engine.max_slots:
            raise StepError(f"a decode session takes 1..{self.engine.max_slots} sequences")
        self.slots = list(slots)
        self.params = params or SamplingParams.greedy()
        self._state_stale = True
        self.requests = list(requests) if requests is not None else list(range(B))
        self.steps_done = list(steps) if steps is not None else [0] * B
        pos = [self.engine.cache.length(s) for s in slots]
        cap = self.engine.max_slots
        h = self._host_np
        torch.cuda.current_stream().synchronize()       # earlier copies out of the staging words are done
        h[:B] = np.asarray(list(tokens), dtype=np.int32)
        h[cap:cap + B] = np.asarray(pos, dtype=np.int32)
        h[2 * cap:2 * cap + B] = np.asarray(self.slots, dtype=np.int32)
        self.ids[:B].copy_(self._host[:B], non_blocking=True)
        self.tok_pos[:B].copy_(self._host[cap:cap + B], non_blocking=True)
        self.seq_pos0[:B].copy_(self._host[cap:cap + B], non_blocking=True)
        self.seq_slot[:B].copy_(self._host[2 * cap:2 * cap + B], non_blocking=True)
        self.engine.h2d_bytes += 16 * B

    # ---- one step ----------------------------------------------------------
    @property
    def _draws(self) -> bool:
        return not self.params.is_greedy

    def set_context(self, B: int) -> StepContext:
        """The step context of one token for each of the first B live sequences, read from the
        session's device buffers (what the captured step sees)."""
        ctx = self.ctx
        ctx.ids, ctx.tok_pos, ctx.seq_slot, ctx.seq_pos0 = self.ids[:B], self.tok_pos[:B], self.seq_slot[:B], self.seq_pos0[:B]
        ctx.tok_seq, ctx.seq_start, ctx.want_rows = self.arange[:B], self.arange[:B + 1], self.arange[:B]
        ctx.n_tokens = ctx.n_seqs = ctx.n_want = B
        ctx.max_new, ctx.max_len = 1, self._bucket
        ctx.decode_only = True
        ctx.host_seq_new, ctx.host_seq_pos0, ctx.host_seq_slot = [1] * B, None, list(self.slots)
        return ctx

    def _body(self, B: int, draws: bool) -> None:
        ctx = self.set_context(B)
        self.engine.model.forward(ctx, self.engine.cache, self.logits[:B])
        s = self.sampler
        if draws:
            # options, uniform numbers, step counts and histories live on the device (see `run`)
            s.sample_resident(self.logits[:B])
        else:
            s.argmax(self.logits[:B], B)
        ops.advance_decode(s.out, self.ids, self.tok_pos, self.seq_pos0, B, self.ring, self.ring_counter)

    def run(self, n_steps: int = 1, histories=None, use_graph: bool = True) -> int:
        """Run up to `n_steps` decode steps of the live sequences back to back; their tokens stay on
        the device until `read`.  Fewer steps are run when the cache, the context or the length
        bucket of the captured graph ends earlier; returns how many were."""
        B = len(self.slots)
        cache = self.engine.cache
        longest = max(cache.length(s_) for s_ in self.slots)
        room = self.engine.max_context - longest
        n = max(1, min(n_steps, self.max_run, room))
        # kernels choose their grids from an upper bound of the context: the live maximum rounded up
        # to the bucket, so a graph stays valid until a sequence grows past it
        self._bucket = min(self.engine.max_context, -(-(longest + 1) // BUCKET) * BUCKET)
        n = max(1, min(n, self._bucket - longest))
        while True:
            ext = {s: n for s in self.slots}
            why = cache.can_extend(ext)
            if why is None:
                break
            if n == 1:
                raise StepError(why)
            n = max(1, n // 2)
        try:
            cache.extend(ext)
        except CacheFull as e:
            raise StepError(str(e)) from None
        p = self.params
        if self._state_stale and self._draws:
            # once per batch: options, requests, step counts and recent tokens go up; from then on the
            # sampling kernel keeps them (it appends what it selects and counts the steps)
            self.sampler.load_state(p, self.requests, self.steps_done, histories)
        self._state_stale = False
        if self._kept == 0:
            self._ring_base = self._steps_total
        draws = self._draws
        for _ in range(n):
            if use_graph and self.graph_safe:
                key = (B, self._bucket, draws)
                g = self.graphs.get(key)
                if g is None:
                    # The first step at this batch size runs eagerly (it loads kernels); the same
                    # chain is then captured, without running, for the next ones.
                    before = ops.LAUNCHES
                    self._body(B, draws)
                    self.launches_per_step = ops.LAUNCHES - before
                    g = torch.cuda.CUDAGraph()
                    # The collector must not run while the stream is captured: finalising an engine
                    # that went out of use (its graphs, events, pinned buffers) makes CUDA calls that
                    # are not allowed then and would spoil the capture.
                    gc.collect()
                    was_enabled = gc.isenabled()
                    gc.disable()
                    try:
                        with torch.cuda.graph(g):
                            self._body(B, draws)
                    finally:
                        if was_enabled:
                            gc.enable()
                    self.graphs[key] = g
                else:
                    g.replay()
            else:
                self._body(B, draws)
        cache.commit(ext)
        self.steps_done = [c + n for c in self.steps_done]
        self._kept += n
        self._steps_total += n
        if self._kept > self.max_run:       # nobody read them: the oldest steps' rows were written over
            self._ring_base += self._kept - self.max_run
            self._kept = self.max_run
        return n

    def read(self) -> list[tuple[list[int], list[int]]]:
        """The tokens and non-finite flags of every step since the last read, oldest first
        (one copy for all of them; synchronises).  Raises `KernelError` if a kernel's bounded
        wait ran out in one of the steps."""
        B, cap, n = len(self.slots), self.sampler.max_rows, self._kept
        if n == 0:
            return []
        self._ring_host.copy_(self.ring, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.engine.d2h_bytes += self.ring.numel() * 4
        rows = self.ring.shape[0]
        out = []
        status = 0
        for j in range(n):
            row = self._ring_host[(self._ring_base + j) % rows]
            out.append((row[:B].tolist(), row[cap:cap + B].tolist()))
            status = status or int(row[2 * cap])
        self._kept = 0
        if self.engine.rt.tc is not None:
            self.engine.raise_on_status(status)
        return out
