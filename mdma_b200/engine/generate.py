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
    def __init__(self, engine, sampler, use_graphs: bool = True):
        self.engine, self.sampler, self.use_graphs = engine, sampler, use_graphs
        self._sessions: dict = {}

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
                 on_token: Optional[Callable[[int, int], None]] = None) -> list[Output]:
        params = params or SamplingParams.greedy()
        params.validate()
        stop = frozenset(int(s) for s in stop_ids)
        if params.repetition_penalty != 1.0 and hasattr(self.sampler, "ensure_history"):
            if self.sampler.ensure_history(params.repetition_window):
                self._sessions.clear()          # their graphs hold the old history buffers
        budgets = [token_budget(len(p), max_tokens, self.engine.max_context) for p in prompts]
        outputs = [Output(list(p)) for p in prompts]
        sizes = [(len(p), b) for p, (b, _) in zip(prompts, budgets)]
        for batch in self.plan_batches(sizes):
            self._run_batch(batch, prompts, budgets, outputs, params, stop, cancelled, on_token)
        return outputs

    def _run_batch(self, batch, prompts, budgets, outputs, params, stop, cancelled, on_token) -> None:
        live = [_Live(r, self.engine.acquire(), budgets[r][0], budgets[r][1]) for r in batch]
        penalised = params.repetition_penalty != 1.0 and params.repetition_window > 0
        session = None
        session_fresh = False          # whether the session's device buffers describe this batch
        try:
            entries = [StepEntry(s.slot, list(prompts[s.request]), [len(prompts[s.request]) - 1]) for s in live]
            first = True
            while live:
                if cancelled is not None and cancelled():
                    for s in live:
                        outputs[s.request].finish_reason = FINISH_CANCELLED
                    break
                histories = None
                if penalised:
                    histories = [outputs[s.request].prompt_tokens + outputs[s.request].tokens for s in live]
                if first or session is None:
                    logits = self.engine.step(entries)
                    tokens, flags = self.sampler.sample(logits, params, [s.request for s in live],
                                                        [s.steps for s in live], histories)
                else:
                    # decode: this step's input tokens go up from the host, the step is replayed
                    # as a graph, the selected tokens come back
                    slots_now = [s.slot for s in live]
                    if session.slots == slots_now and session_fresh:
                        session.feed([s.next_token for s in live])
                        session.steps_done = [s.steps for s in live]
                    else:
                        session.start(slots_now, [s.next_token for s in live],
                                      [s.request for s in live], [s.steps for s in live])
                        session_fresh = True
                    session.step_async(histories)
                    tokens, flags = session.read_tokens()
                survivors = []
                for s, tok, bad in zip(live, tokens, flags):
                    out = outputs[s.request]
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
                live = survivors
                if first and live and self.use_graphs and hasattr(self.engine, "decode_session"):
                    session = self._sessions.get(params)
                    if session is None:
                        session = self._sessions[params] = self.engine.decode_session(self.sampler, params)
                    if not session.graph_safe:
                        session = None
                first = False
                if session is None:
                    entries = [StepEntry(s.slot, [s.next_token], [0]) for s in live]
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
    from ..sampling.sampler import DeviceSampler
    from .step import Engine
    engine = Engine(model_dir, dtype=dtype, max_batch=max_batch, max_context=max_context, **engine_args)
    sampler = DeviceSampler(engine.vocab_size, engine.max_slots, engine.device)
    params = SamplingParams(temperature, top_p, min_p, repetition_penalty, repetition_window, seed)
    if stop_ids is None:
        stop_ids = engine.spec.stop_token_ids
    return Generator(engine, sampler, use_graphs).generate(prompts, max_tokens, params, stop_ids)
