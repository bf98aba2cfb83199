"""Device-side token selection for a batch of rows (see csrc/sampling.cu)."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from ..kernels.lib import KernelError, NonFiniteLogits
from .options import GenerationOptions, seed_state



class Sampler:
    """Greedy when ``temperature`` is 0 (k forced to 1), else top-k / temperature /
    nucleus sampling with an optional repetition penalty.  One generator state per row."""

    def __init__(self, vocab_size: int, max_rows: int, options: GenerationOptions, device):
        options.validate()
        self.vocab, self.max_rows, self.options, self.device = vocab_size, max_rows, options, device
        self.rng = torch.zeros(max_rows, dtype=torch.int32, device=device)
        # chosen ids of the rows, then the error word: one buffer, so that both are read in one copy
        self._both = torch.zeros(max_rows + 1, dtype=torch.int32, device=device)
        self.out = self._both[:max_rows]
        self.flag = self._both[max_rows:]
        nbytes = ops.sample_scratch_bytes(max_rows, vocab_size, options.top_k)
        if nbytes < 0:
            raise ValueError("sampling scratch would exceed 2 GiB; lower the batch")
        self.greedy_plain = options.temperature <= 0 and not (options.repetition_penalty != 1.0)
        if self.greedy_plain:                # room for the candidates of the fused head as well
            nbytes = max(nbytes, max_rows * ops.head_candidates(vocab_size) * 8)
        self.scratch = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=device)
        self._pinned: Optional[torch.Tensor] = None
        self._event = None
        self._posted = 0
        self.bytes_read = 0
        self.penalised = options.repetition_penalty != 1.0
        self.seen: Optional[torch.Tensor] = None
        if self.penalised:
            self.seen = torch.zeros((max_rows, vocab_size), dtype=torch.uint8, device=device)

    def start(self, first_index: int, n_rows: int, seed: Optional[int] = None) -> None:
        """Seed rows 0..n_rows-1 for the requests first_index, first_index+1, ... (``seed``: instead of the
        options' own, so that one sampler, and the decode graphs that embed it, serve calls that differ in
        nothing but the seed)."""
        seed = self.options.seed if seed is None else seed
        states = np.array([seed_state(seed, first_index + i) for i in range(n_rows)], dtype=np.uint32)
        self.rng[:n_rows].copy_(torch.from_numpy(states.view(np.int32)))
        if self.seen is not None:
            self.seen[:n_rows].zero_()

    def mark_prompt(self, tokens: torch.Tensor, rows: torch.Tensor) -> None:
        """Prompt ids count as seen (src/models/QuickNN.Models.LLM.pas:735-742)."""
        if self.seen is not None:
            ops.mark_seen(tokens, rows, self.seen)

    def compact(self, keep_rows: Sequence[int]) -> None:
        """Rows that stay alive move to the front, in order."""
        idx = torch.tensor(list(keep_rows), dtype=torch.long, device=self.device)
        n = len(keep_rows)
        self.rng[:n] = self.rng[idx]
        if self.seen is not None:
            self.seen[:n] = self.seen[idx]

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        """logits [R, V] float32 -> chosen ids [R] int32 (device)."""
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"the sampler was built for {self.max_rows} rows, the step has {R}")
        o = self.options
        seen_rows = None
        if self.seen is not None:
            seen_rows = torch.arange(R, dtype=torch.int32, device=self.device)
        ops.sample(logits, o.top_k, o.temperature, o.top_p, o.repetition_penalty, self.rng, self.seen,
                   seen_rows, self.scratch, self.out, self.flag, ops.status_words(self.device)[0:1])
        return self.out[:R]

    def head(self, hidden: torch.Tensor, weight: torch.Tensor, cap: Optional[float]) -> Optional[torch.Tensor]:
        """Chosen ids straight from the rows that go into the output head (after the final norm),
        without the logits in between: for greedy selection without a repetition penalty the head
        product keeps only the best (value, id) of each group of 16 columns and the merge picks the
        largest.  Returns None when that does not apply; the caller then forms the logits and calls
        the sampler on them.  Same ids as that way (the same sums, compared in the same order)."""
        if not self.greedy_plain or weight.shape[0] != self.vocab or not ops.head_argmax_fusable(hidden, weight):
            return None
        R = hidden.shape[0]
        if R > self.max_rows:
            raise ValueError(f"the sampler was built for {self.max_rows} rows, the step has {R}")
        cand = self.scratch.view(torch.float32)
        ncand = ops.head_argmax(hidden, weight, cap, cand, self.flag)
        if ncand is None:
            return None
        ops.sample_candidates(cand, R, ncand, self.vocab, 1, 0.0, self.options.top_p, self.rng, None, None, self.out,
                              self.flag, ops.status_words(self.device)[0:1])
        return self.out[:R]

    def read(self, tokens: torch.Tensor) -> np.ndarray:
        """Chosen ids and the error word in one device-to-host read."""
        self.post(tokens)
        return self.collect()

    def post(self, tokens: torch.Tensor) -> None:
        """Queue the read of ``tokens`` (and the error word) into pinned memory; what is
        launched after this call does not delay it."""
        n = tokens.numel()
        if self._pinned is None:
            self._pinned = torch.empty(self.max_rows + 1, dtype=torch.int32, pin_memory=True)
            self._event = torch.cuda.Event()
        self._pinned[:n].copy_(tokens.reshape(-1), non_blocking=True)
        self._pinned[n:n + 1].copy_(self.flag, non_blocking=True)
        self._event.record()
        self._posted = n
        self.bytes_read += 4 * (n + 1)

    def collect(self) -> np.ndarray:
        """Wait for the read queued by ``post`` and return the ids."""
        self._event.synchronize()
        both = self._pinned[:self._posted + 1].numpy().copy()
        word = int(both[-1])
        if word != 0:
            self.flag.zero_()
            if word & 2:                      # a bounded wait of a tcgen05 kernel ran out during the step
                ops.status_words(self.device)[0:1].zero_()
                raise KernelError(ops.wait_status_message(word >> 8))
            raise NonFiniteLogits("the model produced non-finite logits")
        return both[:-1]
