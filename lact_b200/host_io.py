"""Host-resident inputs and outputs: the op is run slab by slab along dim 0, with the copies of
neighbouring slabs overlapped with the kernels.

Every merged (batch x head) entry is an independent recurrence, so a call on B entries equals
`n_slabs` calls on B / n_slabs entries each.  Three streams work on consecutive slabs at the same
time: host-to-device copies of slab i + 1 (pinned memory), the kernels of slab i, and the
device-to-host copy of slab i - 1's output; each input has two device buffers.  PCIe carries both
directions at once, so a step costs about max(H2D, kernels, D2H) instead of their sum.
"""
from __future__ import annotations

from typing import Callable, Dict

import torch


class HostPipeline:
    """`fn(**device_tensors) -> o` is the op (any of the chunk drivers, wrapped to take keywords);
    `host` maps argument names to pinned host tensors; tensors whose dim 0 equals the number of
    entries are cut into slabs, everything else is passed through unchanged.  `out_host` (pinned)
    receives the output."""

    def __init__(self, fn: Callable[..., torch.Tensor], host: Dict[str, torch.Tensor], out_host: torch.Tensor,
                 n_slabs: int, device: torch.device):
        self.fn, self.host, self.out_host, self.device = fn, host, out_host, device
        self.entries = out_host.shape[0]
        if n_slabs < 1 or self.entries % n_slabs:
            raise ValueError("the number of (batch x head) entries must be a multiple of n_slabs")
        self.n_slabs, self.per = n_slabs, self.entries // n_slabs
        for name, t in list(host.items()) + [("out", out_host)]:
            if torch.is_tensor(t) and not t.is_pinned():
                raise ValueError(f"{name} must be in pinned host memory")
        self.sliced = {k for k, v in host.items() if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == self.entries}
        self.bufs = [{k: torch.empty((self.per,) + tuple(host[k].shape[1:]), dtype=host[k].dtype, device=device)
                      for k in self.sliced} for _ in range(2)]
        self.h2d, self.d2h = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_done = [torch.cuda.Event() for _ in range(2)]

    def run(self) -> None:
        """One step: all inputs cross to the device, all outputs come back; returns once the work
        is queued, with the caller's current stream ordered after the last copy."""
        main = torch.cuda.current_stream(self.device)
        self.h2d.wait_stream(main)
        self.d2h.wait_stream(main)
        for s in range(self.n_slabs):
            slot, lo = s & 1, s * self.per
            with torch.cuda.stream(self.h2d):
                if s >= 2:
                    self.h2d.wait_event(self.ev_done[slot])  # the kernels of slab s - 2 have read this buffer
                for k in self.sliced:
                    self.bufs[slot][k].copy_(self.host[k][lo:lo + self.per], non_blocking=True)
                self.ev_in[slot].record(self.h2d)
            main.wait_event(self.ev_in[slot])
            args = {k: (self.bufs[slot][k] if k in self.sliced else v) for k, v in self.host.items()}
            o = self.fn(**args)
            self.ev_done[slot].record(main)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(self.ev_done[slot])
                self.out_host[lo:lo + self.per].copy_(o, non_blocking=True)
                o.record_stream(self.d2h)
        main.wait_stream(self.d2h)
        main.wait_stream(self.h2d)
