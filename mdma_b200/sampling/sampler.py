"""Token selection on the device for a batch of logits rows."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams, uniform

EXTRA_WORDS = 4          # words after tokens and flags that travel to the host in the same copy


def params_words(params: SamplingParams) -> np.ndarray:
    """The eight 32-bit words the sampling kernel reads its options from (see `ops.sample`)."""
    w = np.zeros(8, dtype=np.int32)
    w[:4] = np.asarray([params.temperature, params.top_p, params.min_p, params.repetition_penalty],
                       dtype=np.float32).view(np.int32)
    w[4] = int(params.repetition_window)
    seed = params.seed & ((1 << 64) - 1)
    w[6:8] = np.asarray([seed & 0xFFFFFFFF, seed >> 32], dtype=np.uint32).view(np.int32)
    return w


class DeviceSampler:
    """Owns the device buffers the sampling kernels need for up to `max_rows` rows; `sample`
    returns host lists (tokens, non-finite flags).  `alloc(shape, dtype)` says where the
    buffers come from (an engine passes its arena, and everything is then taken up front);
    without it they are allocated here, the large scratch on first use."""

    def __init__(self, vocab_size: int, max_rows: int, device, history_cap: int = 64, alloc=None):
        self.vocab, self.max_rows, self.device = vocab_size, max_rows, device
        self._fixed = alloc is not None
        if alloc is None:
            alloc = lambda shape, dtype: torch.zeros(shape, dtype=dtype, device=device)
        # selected tokens, non-finite flags and a few words of the owner's side by side: one copy brings all to the host
        self.out = alloc((2 * max_rows + EXTRA_WORDS,), torch.int32)
        self.uniforms = alloc((max_rows,), torch.float32)
        self.history_cap = max(1, history_cap)
        self.history = alloc((max_rows, self.history_cap), torch.int32)
        self.history_len = alloc((max_rows,), torch.int32)
        # a decode loop that is replayed as a graph keeps what a draw depends on here: the kernel makes
        # the uniform numbers from (seed, request, step), counts the steps and appends to the histories,
        # and reads its options from `dev_params`
        self.requests = alloc((max_rows,), torch.int32)
        self.steps = alloc((max_rows,), torch.int32)
        self.dev_params = alloc((8,), torch.int32)
        self.argmax_scratch = alloc((ops.argmax_scratch_words(max_rows, vocab_size),), torch.float32)
        self._probs = alloc((ops.sample_scratch_words(max_rows, vocab_size),), torch.float32) if self._fixed else None
        if self.out is None:          # sizes only
            return
        self.tokens, self.flags = self.out[:max_rows], self.out[max_rows:2 * max_rows]
        self.extra = self.out[2 * max_rows:]
        self._out_host = torch.empty(2 * max_rows + EXTRA_WORDS, dtype=torch.int32).pin_memory()
        self.d2h_bytes = 0          # bytes of results read back so far

    def ensure_history(self, window: int) -> bool:
        """Room for the last `window` tokens of every row.  Returns True if the buffers were replaced
        (graphs that captured the old ones must not be replayed).  A sampler whose memory was taken
        up front cannot grow: it refuses a longer window."""
        if window <= self.history_cap:
            return False
        if self._fixed:
            raise ValueError(f"repetition_window {window} is beyond the {self.history_cap} tokens of history "
                             f"this engine reserved (Engine(history_cap=...))")
        self.history_cap = window
        self.history = torch.zeros((self.max_rows, window), dtype=torch.int32, device=self.device)
        self.history_len.zero_()
        return True

    def ensure_probs(self) -> None:
        if self._probs is None:
            self._probs = torch.empty(ops.sample_scratch_words(self.max_rows, self.vocab), dtype=torch.float32,
                                      device=self.device)

    def _stage_histories(self, params: SamplingParams, n: int, histories) -> bool:
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

    def stage_inputs(self, params: SamplingParams, requests, steps, histories=None) -> bool:
        """Upload what the sampled path reads: one uniform number per row, keyed by
        (seed, request, step), and the rows' recent tokens.  Returns whether histories are in use."""
        n = len(requests)
        u = np.asarray([uniform(params.seed, r, s) for r, s in zip(requests, steps)], dtype=np.float32)
        self.uniforms[:n].copy_(torch.from_numpy(u))
        return self._stage_histories(params, n, histories)

    def load_state(self, params: SamplingParams, requests, steps, histories=None) -> None:
        """Put the options, the rows' requests, step counts and recent tokens on the device, once per
        batch; after that `sample_resident` needs nothing from the host."""
        n = len(requests)
        self.dev_params.copy_(torch.from_numpy(params_words(params)))
        self.requests[:n].copy_(torch.from_numpy(np.asarray(list(requests), dtype=np.int32)))
        self.steps[:n].copy_(torch.from_numpy(np.asarray(list(steps), dtype=np.int32)))
        if not self._stage_histories(params, n, histories):
            self.history_len[:n].zero_()

    def sample_resident(self, logits: torch.Tensor) -> None:
        """Fill self.tokens/flags for the rows of `logits` from the state that `load_state` left and
        move it on by one step (graph-safe: nothing comes from the host, not even the options)."""
        self.ensure_probs()
        ops.sample(logits, None, self.tokens, self._probs, 1.0, 1.0, 0.0, 1.0, 0, self.history, self.history_len,
                   self.flags, logits.shape[0], requests=self.requests, steps=self.steps, seed=0, advance=True,
                   dev_params=self.dev_params)

    def argmax(self, logits: torch.Tensor, n: Optional[int] = None) -> None:
        ops.argmax(logits, self.tokens, self.flags, logits.shape[0] if n is None else n, self.argmax_scratch)

    def sample_device(self, logits: torch.Tensor, params: SamplingParams, requests: Sequence[int],
                      steps: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None) -> None:
        """Fill self.tokens[:n] and self.flags[:n] for the n rows of `logits`."""
        n = logits.shape[0]
        assert n <= self.max_rows and logits.shape[1] == self.vocab
        penalised = params.repetition_penalty != 1.0 and params.repetition_window > 0 and histories is not None
        if params.temperature <= 0.0 and not penalised:
            self.argmax(logits, n)
            return
        use_hist = self.stage_inputs(params, requests, steps, histories)
        self.ensure_probs()
        ops.sample(logits, self.uniforms, self.tokens, self._probs, params.temperature, params.top_p,
                   params.min_p, params.repetition_penalty, min(params.repetition_window, self.history_cap),
                   self.history if use_hist else None, self.history_len if use_hist else None, self.flags, n)

    def read(self, n: int) -> tuple[list[int], list[int], list[int]]:
        """The first n tokens and flags and the extra words, in one copy (synchronises)."""
        self._out_host.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += self.out.numel() * 4
        host = self._out_host
        return (host[:n].tolist(), host[self.max_rows:self.max_rows + n].tolist(),
                host[2 * self.max_rows:].tolist())

    def sample(self, logits, params, requests, steps, histories=None) -> tuple[list[int], list[int]]:
        self.sample_device(logits, params, requests, steps, histories)
        tokens, flags, _ = self.read(logits.shape[0])
        return tokens, flags
