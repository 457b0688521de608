"""Next-token selection: greedy, or sampling with temperature, top-k, top-p, min-p, with the
repetition penalty and the suppression of stop tokens before ``min_new_tokens``.

Order and meaning follow the reference: processors first (repetition penalty
logits_process.py:335-343, minimum of new tokens :215-223), then for sampling the warpers
temperature :288, top-k :512-518, top-p :453-465, min-p :578-595 in that order
(src/transformers/generation/utils.py:1057-1071), then softmax + one multinomial draw, or
argmax (utils.py:3275-3279). The draw here is keyed on (seed, request, step) instead of a
global generator, so a request samples the same tokens alone or in any batch.
All of it runs in one hand-written kernel per step (csrc/sampling.cu).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..config.generation import GenerationConfig


class DeviceSelector:
    """Selects tokens on the device from float32 logits [rows, vocab]."""

    def __init__(self, kernels, device, vocab_size: int, options: GenerationConfig, max_rows: int,
                 max_history: int = 0):
        self.k, self.device, self.vocab, self.opt = kernels, torch.device(device), int(vocab_size), options
        self.max_rows = max_rows
        self.work = torch.empty((max_rows, vocab_size), dtype=torch.float32, device=self.device)
        self.out = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self._host = self._landed = None      # page-locked landing place of the tokens, made at first use
        eos = options.eos_ids()
        self.suppress = torch.tensor(eos, dtype=torch.int32, device=self.device) if eos else None
        self.use_history = options.repetition_penalty != 1.0
        self.max_history = max_history
        self.history = (torch.zeros((max_rows, max(1, max_history)), dtype=torch.int32, device=self.device)
                        if self.use_history else None)
        self.history_len = torch.zeros(max_rows, dtype=torch.int32, device=self.device) if self.use_history else None

    def select(self, logits: torch.Tensor, request_ids: Sequence[int], step: int,
               histories: Optional[Sequence[Sequence[int]]] = None, suppress_stop: bool = False) -> List[int]:
        """One token per row. ``request_ids[r]`` and ``step`` key the draw of row r;
        ``histories[r]`` are the tokens that the repetition penalty looks at."""
        return self.finish(self.begin(logits, request_ids, step, histories, suppress_stop))

    def device_tokens(self, rows: int) -> torch.Tensor:
        """The tokens of the selection that ``begin`` started, on the device (int32 [rows]): a step may
        read them there (in stream order) before the host has them."""
        return self.out[:rows]

    def finish(self, rows: int) -> List[int]:
        """Wait for the tokens of the selection that ``begin`` started and return them."""
        self._landed.synchronize()
        return self._host[:rows].tolist()

    def begin(self, logits: torch.Tensor, request_ids: Sequence[int], step: int,
              histories: Optional[Sequence[Sequence[int]]] = None, suppress_stop: bool = False) -> int:
        """Launch the selection and the copy of its tokens to page-locked host memory without waiting:
        the host is free (to prepare the next step, say) until ``finish``."""
        rows = logits.shape[0]
        if rows > self.max_rows:
            raise ValueError(f"selector was sized for {self.max_rows} rows, got {rows}")
        o = self.opt
        streams = counters = None
        if o.do_sample:
            meta = torch.tensor([list(request_ids), [step] * rows], dtype=torch.int64).to(self.device)
            streams, counters = meta[0], meta[1]
        hist = hist_len = None
        if self.use_history:
            width = self.history.shape[1]
            host = torch.zeros((rows, width), dtype=torch.int32)
            lens = torch.zeros(rows, dtype=torch.int32)
            for r, h in enumerate(histories or ()):
                h = list(h)[-width:]
                host[r, :len(h)] = torch.tensor(h, dtype=torch.int32)
                lens[r] = len(h)
            self.history[:rows].copy_(host)
            self.history_len[:rows].copy_(lens)
            hist, hist_len = self.history, self.history_len
        self.k.sample(logits, self.work, self.out, do_sample=o.do_sample, temperature=float(o.temperature),
                      top_k=int(o.top_k), top_p=float(o.top_p), min_p=float(o.min_p or 0.0),
                      repetition_penalty=float(o.repetition_penalty), history=hist, history_len=hist_len,
                      suppress=self.suppress if suppress_stop else None, seed=int(o.seed), streams=streams,
                      counters=counters)
        if self._host is None:
            self._host = torch.empty(self.max_rows, dtype=torch.int32, pin_memory=self.device.type == "cuda")
            self._landed = torch.cuda.Event() if self.device.type == "cuda" else None
        self._host[:rows].copy_(self.out[:rows], non_blocking=True)
        self._landed.record(torch.cuda.current_stream(self.device))
        return rows
