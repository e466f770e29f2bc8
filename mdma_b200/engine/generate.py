"""The generation loop above the step function.

Requests (token-id prompts of unequal lengths) are taken in batches that
start together: all prompts of a batch in one step, then one token per live
sequence per step.  A sequence ends on a stop token (which is not emitted), on
its token budget, or at the context limit; it then leaves the batch and gives
its slot and pages back, and the others go on.  When a batch is empty the next
one starts, until every request is served.  The rules are the reference's
(src/inference.rs:44-124, src/session/worker.rs:59-101, 244-332): the last
sampled token is never fed back, so a budget of n tokens needs n-1 decode
steps and prompt + n - 1 cache rows; a request whose budget was cut by the
context ends with reason "context_limit".

The loop decides; it does not compute.  It needs an object with `acquire()`,
`release(slot)`, `step(entries) -> logits`, `max_context`, `max_slots`,
`fits(list of (prompt length, budget))`, and a sampler with
`sample(logits, params, requests, steps, histories) -> (tokens, flags)`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..sampling.params import SamplingParams
from .step import StepEntry

FINISH_STOP = "stop"                    # the reference's Eos
FINISH_LENGTH = "length"                # MaxTokens
FINISH_CONTEXT = "context_limit"        # ContextLimit
FINISH_NONFINITE = "nonfinite_logits"
FINISH_CANCELLED = "cancelled"


class ContextLimitError(ValueError):
    """A prompt is empty or leaves no room in the context (src/inference.rs:60-66)."""


@dataclass
class Output:
    prompt_tokens: list
    tokens: list = field(default_factory=list)
    finish_reason: Optional[str] = None


@dataclass
class _Live:
    request: int
    slot: int
    budget: int
    context_limited: bool
    next_token: int = -1
    steps: int = 0


def token_budget(prompt_len: int, max_tokens: int, max_context: int) -> tuple[int, bool]:
    """How many tokens a request may emit, and whether the context cut its budget.
    Emitting n tokens holds prompt + n - 1 cache rows."""
    if prompt_len <= 0:
        raise ContextLimitError("a prompt must hold at least one token")
    if max_tokens <= 0:
        raise ContextLimitError("max_tokens must be positive")
    if prompt_len > max_context:
        raise ContextLimitError(f"a prompt of {prompt_len} tokens does not fit the context of {max_context}")
    room = max_context - prompt_len + 1
    return (max_tokens, False) if max_tokens <= room else (room, True)


class Generator:
    """`run_ahead`: how many decode steps are replayed back to back before the host reads their
    tokens (a sequence that stops inside such a run has computed a few tokens for nothing)."""

    def __init__(self, engine, sampler=None, use_graphs: bool = True, run_ahead: int = 8):
        self.engine, self.use_graphs, self.run_ahead = engine, use_graphs, max(1, run_ahead)
        self.sampler = sampler if sampler is not None else engine.sampler

    def plan_batches(self, sizes: Sequence[tuple[int, int]]) -> list[list[int]]:
        """Cut request indices, in order, into batches the cache can hold at once."""
        batches, cur = [], []
        for i, size in enumerate(sizes):
            trial = cur + [i]
            if len(trial) <= self.engine.max_slots and self.engine.fits([sizes[j] for j in trial]):
                cur = trial
                continue
            if not cur:
                raise ContextLimitError(
                    f"request {i} (prompt {size[0]}, budget {size[1]}) does not fit the cache even alone")
            batches.append(cur)
            cur = [i]
            if not self.engine.fits([size]):
                raise ContextLimitError(
                    f"request {i} (prompt {size[0]}, budget {size[1]}) does not fit the cache even alone")
        if cur:
            batches.append(cur)
        return batches

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 32,
                 params: Optional[SamplingParams] = None, stop_ids: Sequence[int] = (),
                 cancelled: Optional[Callable[[], bool]] = None,
                 on_token: Optional[Callable[[int, int], None]] = None,
                 use_graphs: Optional[bool] = None) -> list[Output]:
        params = params or SamplingParams.greedy()
        params.validate()
        stop = frozenset(int(s) for s in stop_ids)
        if params.repetition_penalty != 1.0 and hasattr(self.sampler, "ensure_history"):
            self.sampler.ensure_history(params.repetition_window)       # refuses a window it has no room for
        budgets = [token_budget(len(p), max_tokens, self.engine.max_context) for p in prompts]
        outputs = [Output(list(p)) for p in prompts]
        sizes = [(len(p), b) for p, (b, _) in zip(prompts, budgets)]
        graphs = self.use_graphs if use_graphs is None else use_graphs
        for batch in self.plan_batches(sizes):
            self._run_batch(batch, prompts, budgets, outputs, params, stop, cancelled, on_token, graphs)
        return outputs

    def _absorb(self, live, tokens, flags, outputs, stop, on_token) -> list:
        """One step's tokens: append, or end the sequence.  Returns the sequences that go on."""
        survivors = []
        for s, tok, bad in zip(live, tokens, flags):
            out = outputs[s.request]
            if s.slot < 0:                  # ended at an earlier step of the same run
                continue
            s.steps += 1
            if bad:
                out.finish_reason = FINISH_NONFINITE       # src/inference.rs:111-113
            elif tok in stop:
                out.finish_reason = FINISH_STOP            # not emitted: src/inference.rs:115-118
            else:
                out.tokens.append(tok)
                if on_token is not None:
                    on_token(s.request, tok)
                if len(out.tokens) >= s.budget:            # the last token is not fed back
                    out.finish_reason = FINISH_CONTEXT if s.context_limited else FINISH_LENGTH
                else:
                    s.next_token = tok
                    survivors.append(s)
                    continue
            self.engine.release(s.slot)
            s.slot = -1
        return survivors

    def _run_batch(self, batch, prompts, budgets, outputs, params, stop, cancelled, on_token, graphs) -> None:
        live = [_Live(r, self.engine.acquire(), budgets[r][0], budgets[r][1]) for r in batch]
        penalised = params.repetition_penalty != 1.0 and params.repetition_window > 0
        session = None
        session_fresh = False          # whether the session's device buffers describe the live sequences

        def histories_of(seqs):
            if not penalised:
                return None
            return [outputs[s.request].prompt_tokens + outputs[s.request].tokens for s in seqs]

        def cancel_all():
            for s in live:
                outputs[s.request].finish_reason = FINISH_CANCELLED
        try:
            if cancelled is not None and cancelled():
                cancel_all()
                return
            # all prompts of the batch in one step
            entries = [StepEntry(s.slot, list(prompts[s.request]), [len(prompts[s.request]) - 1]) for s in live]
            logits = self.engine.step(entries)
            tokens, flags = self.sampler.sample(logits, params, [s.request for s in live],
                                                [s.steps for s in live], histories_of(live))
            if hasattr(self.engine, "check_status"):
                self.engine.check_status()
            live = self._absorb(live, tokens, flags, outputs, stop, on_token)
            if live and graphs and hasattr(self.engine, "decode_session"):
                session = self.engine.decode_session()
                if not session.graph_safe:
                    session = None
            while live:
                if cancelled is not None and cancelled():
                    cancel_all()
                    break
                if session is None:
                    entries = [StepEntry(s.slot, [s.next_token], [0]) for s in live]
                    logits = self.engine.step(entries)
                    tokens, flags = self.sampler.sample(logits, params, [s.request for s in live],
                                                        [s.steps for s in live], histories_of(live))
                    if hasattr(self.engine, "check_status"):
                        self.engine.check_status()
                    live = self._absorb(live, tokens, flags, outputs, stop, on_token)
                    continue
                # decode: a run of steps replayed as graphs; the tokens a step selects are the next
                # step's inputs on the device, the host reads the run's tokens in one copy
                slots_now = [s.slot for s in live]
                if not (session_fresh and session.slots == slots_now):
                    session.start(slots_now, [s.next_token for s in live], [s.request for s in live],
                                  [s.steps for s in live], params)
                    session_fresh = True
                # no sequence runs past its own budget (a stop token may still end one inside the run)
                n = min(self.run_ahead, min(s.budget - len(outputs[s.request].tokens) for s in live))
                session.run(n, histories_of(live))
                run = list(live)
                for tokens, flags in session.read():
                    self._absorb(run, tokens, flags, outputs, stop, on_token)
                live = [s for s in run if s.slot >= 0]
        finally:
            for s in live:
                if s.slot >= 0:
                    self.engine.release(s.slot)
                    s.slot = -1


def generate(model_dir: str, prompts: Sequence[Sequence[int]], max_tokens: int = 32,
             temperature: float = 0.0, seed: int = 0, stop_ids: Optional[Sequence[int]] = None,
             dtype: str = "bfloat16", top_p: float = 1.0, min_p: float = 0.0,
             repetition_penalty: float = 1.0, repetition_window: int = 64,
             max_batch: int = 8, max_context: Optional[int] = None, use_graphs: bool = True,
             **engine_args) -> list[Output]:
    """One call from a model folder and token-id prompts to generated token ids."""
    from .step import Engine
    engine = Engine(model_dir, dtype=dtype, max_batch=max_batch, max_context=max_context, **engine_args)
    params = SamplingParams(temperature, top_p, min_p, repetition_penalty, repetition_window, seed)
    if stop_ids is None:
        stop_ids = engine.spec.stop_token_ids
    return Generator(engine, use_graphs=use_graphs).generate(prompts, max_tokens, params, stop_ids)
