"""Token selection on the device for a batch of logits rows."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams, uniform


class DeviceSampler:
    """Owns the small device buffers the sampling kernels need for up to
    `max_rows` rows; `sample` returns host lists (tokens, non-finite flags)."""

    def __init__(self, vocab_size: int, max_rows: int, device, history_cap: int = 64):
        self.vocab, self.max_rows, self.device = vocab_size, max_rows, device
        # selected tokens and non-finite flags side by side, so that one copy brings both to the host
        self.tokens_and_flags = torch.zeros(2, max_rows, dtype=torch.int32, device=device)
        self.tokens, self.flags = self.tokens_and_flags[0], self.tokens_and_flags[1]
        self.uniforms = torch.zeros(max_rows, dtype=torch.float32, device=device)
        self.history_cap = max(1, history_cap)
        self.history = torch.zeros((max_rows, self.history_cap), dtype=torch.int32, device=device)
        self.history_len = torch.zeros(max_rows, dtype=torch.int32, device=device)
        # a decode loop that is replayed as a graph keeps what a draw depends on here: the kernel makes
        # the uniform numbers from (seed, request, step), counts the steps and appends to the histories
        self.requests = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.steps = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._probs: Optional[torch.Tensor] = None
        self._out_host = torch.empty(2 * max_rows, dtype=torch.int32).pin_memory()

    def ensure_history(self, window: int) -> bool:
        """Room for the last `window` tokens of every row.  Returns True if the buffers were replaced
        (graphs that captured the old ones must not be replayed)."""
        if window <= self.history_cap:
            return False
        self.history_cap = window
        self.history = torch.zeros((self.max_rows, window), dtype=torch.int32, device=self.device)
        self.history_len.zero_()
        return True

    def ensure_probs(self) -> None:
        if self._probs is None:
            self._probs = torch.empty(ops.sample_scratch_words(self.max_rows, self.vocab), dtype=torch.float32,
                                      device=self.device)

    def stage_inputs(self, params: SamplingParams, requests, steps, histories=None) -> bool:
        """Upload what the sampled path reads: one uniform number per row, keyed by
        (seed, request, step), and the rows' recent tokens.  Returns whether histories are in use."""
        n = len(requests)
        u = np.asarray([uniform(params.seed, r, s) for r, s in zip(requests, steps)], dtype=np.float32)
        self.uniforms[:n].copy_(torch.from_numpy(u))
        if params.repetition_penalty != 1.0 and params.repetition_window > 0 and histories is not None:
            w = min(params.repetition_window, self.history_cap)
            rows = np.zeros((n, self.history_cap), dtype=np.int32)
            lens = np.zeros(n, dtype=np.int32)
            for i, h in enumerate(histories):
                tail = list(h[-w:])
                rows[i, :len(tail)] = tail
                lens[i] = len(tail)
            self.history[:n].copy_(torch.from_numpy(rows))
            self.history_len[:n].copy_(torch.from_numpy(lens))
            return True
        return False

    def load_state(self, params: SamplingParams, requests, steps, histories=None) -> bool:
        """Put the rows' requests, step counts and recent tokens on the device, once per batch; after that
        `sample_resident` needs nothing from the host.  Returns whether histories are in use."""
        n = len(requests)
        self.requests[:n].copy_(torch.from_numpy(np.asarray(list(requests), dtype=np.int32)))
        self.steps[:n].copy_(torch.from_numpy(np.asarray(list(steps), dtype=np.int32)))
        return self.stage_inputs(params, requests, steps, histories)

    def sample_resident(self, logits: torch.Tensor, params: SamplingParams, use_hist: bool) -> None:
        """Fill self.tokens/flags for the rows of `logits` from the state that `load_state` left and
        move it on by one step (graph-safe: no host data)."""
        self.ensure_probs()
        ops.sample(logits, None, self.tokens, self._probs, params.temperature, params.top_p, params.min_p,
                   params.repetition_penalty, min(params.repetition_window, self.history_cap),
                   self.history if use_hist else None, self.history_len if use_hist else None, self.flags,
                   logits.shape[0], requests=self.requests, steps=self.steps, seed=params.seed, advance=True)

    def sample_device(self, logits: torch.Tensor, params: SamplingParams, requests: Sequence[int],
                      steps: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None) -> None:
        """Fill self.tokens[:n] and self.flags[:n] for the n rows of `logits`."""
        n = logits.shape[0]
        assert n <= self.max_rows and logits.shape[1] == self.vocab
        penalised = params.repetition_penalty != 1.0 and params.repetition_window > 0 and histories is not None
        if params.temperature <= 0.0 and not penalised:
            ops.argmax(logits, self.tokens, self.flags, n)
            return
        use_hist = self.stage_inputs(params, requests, steps, histories)
        self.ensure_probs()
        ops.sample(logits, self.uniforms, self.tokens, self._probs, params.temperature, params.top_p,
                   params.min_p, params.repetition_penalty, min(params.repetition_window, self.history_cap),
                   self.history if use_hist else None, self.history_len if use_hist else None, self.flags, n)

    def sample(self, logits, params, requests, steps, histories=None) -> tuple[list[int], list[int]]:
        n = logits.shape[0]
        self.sample_device(logits, params, requests, steps, histories)
        self._out_host[:n].copy_(self.tokens[:n], non_blocking=True)
        self._out_host[self.max_rows:self.max_rows + n].copy_(self.flags[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._out_host[:n].tolist(), self._out_host[self.max_rows:self.max_rows + n].tolist()
