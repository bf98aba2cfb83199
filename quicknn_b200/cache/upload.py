"""Small host arrays to the device without stalling the host.

A copy from ordinary host memory makes the caller wait until the stream has drained; a copy
from pinned memory does not, but reads the pinned bytes when the stream gets to it, by which
time the host may have written the next step's values.  So every array is first copied into
the next buffer of a ring of pinned buffers and sent from there; a buffer is reused only after
the copy that read it has run (an event per buffer says so).
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch


class PinnedUploader:
    def __init__(self, device, entries: int = 8, nbytes: int = 1 << 16):
        self.device = torch.device(device)
        self.on_gpu = self.device.type == "cuda"
        self.entries = entries
        self._nbytes = nbytes
        self._bufs: List[Optional[torch.Tensor]] = [None] * entries
        self._events: List[Optional[torch.cuda.Event]] = [None] * entries
        self._next = 0
        self.bytes_sent = 0

    def send(self, dst: torch.Tensor, src: np.ndarray) -> None:
        """dst (contiguous, on the device) = src, ordered on the current stream."""
        src = np.ascontiguousarray(src)
        n = src.nbytes
        if dst.numel() * dst.element_size() != n or not dst.is_contiguous():
            raise ValueError(f"upload of {n} bytes into a tensor of {dst.numel() * dst.element_size()} bytes")
        self.bytes_sent += n
        if n == 0:
            return
        if not self.on_gpu:
            dst.view(torch.uint8).reshape(-1).copy_(torch.from_numpy(src.view(np.uint8).reshape(-1)))
            return
        k = self._next
        self._next = (k + 1) % self.entries
        if self._events[k] is not None:
            self._events[k].synchronize()
        buf = self._bufs[k]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, self._nbytes), dtype=torch.uint8, pin_memory=True)
            self._bufs[k] = buf
        buf.numpy()[:n] = src.view(np.uint8).reshape(-1)
        dst.view(torch.uint8).reshape(-1).copy_(buf[:n], non_blocking=True)
        if self._events[k] is None:
            self._events[k] = torch.cuda.Event()
        self._events[k].record()
