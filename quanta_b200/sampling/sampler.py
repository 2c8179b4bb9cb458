"""The device sampler: one row of float32 logits per request that samples this step.

Greedy when ``temperature <= 0`` (first maximum); else temperature, top-k, top-p, min-p and a
categorical draw, after the repetition / frequency / presence penalties over the tokens the request
has generated so far (src/quanta/minimax/generate.py:56-80, src/quanta/shim/omlx.py:344-363,
1796-1810).  The draw is Gumbel-max with counter-based noise keyed by (seed, token, draw number), so
the same seed gives the same tokens whatever else shares the batch.  A request's options and draw
number live in its state slot on the device (written when it is admitted), so a step's sampling takes
nothing from the host; one device->host copy of the sampled ids per step.
"""

from __future__ import annotations

import torch

from .. import kernels


class Sampled:
    """The ids a step sampled, on their way to the host: ``read()`` waits for this step's copy only, not
    for work queued on the device after it."""

    def __init__(self, host: torch.Tensor, n: int, event, status: torch.Tensor | None):
        self.host, self.n, self.event, self.status = host, n, event, status

    def read(self) -> list[int]:
        self.event.synchronize()
        if self.status is not None and int(self.host[self.n]):
            self.status.zero_()
            kernels.raise_on_status(self.host[self.n:])
        return [int(t) for t in self.host[: self.n]]


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, slots: torch.Tensor, row_slot: torch.Tensor, requests: list,
               status: torch.Tensor | None = None) -> list[int]:
        """``sample_async`` and the read of its result."""
        return self.sample_async(logits, slots, row_slot, requests, status).read()

    def sample_async(self, logits: torch.Tensor, slots: torch.Tensor, row_slot: torch.Tensor, requests: list,
                     status: torch.Tensor | None = None) -> Sampled:
        """Launch the sampling and the copy of the ids to the host; ``read()`` of the result gives them.

        ``logits`` ``[n, vocab]`` float32 on the device; ``slots`` the engine's state records and
        ``row_slot`` int32 ``[n]`` (device) the slot of each row: temperature, top-k, top-p, min-p, seed
        and the draw number are read there, and the kernel counts the draw and leaves the token in the
        record (a decode step launched before the host reads the token takes it from there).  Nothing
        about an unpenalised request travels from the host.  ``requests[i]`` (``.params``,
        ``.generated``) is read for the penalties, which need the tokens generated so far, and to see
        whether every row is greedy.  If ``status`` is given its words are read in the same copy and a
        device-side refusal raises."""
        n, V = logits.shape
        if n != len(requests) or row_slot.numel() != n:
            raise ValueError(f"{n} logits rows for {len(requests)} requests and {row_slot.numel()} slots")
        if logits.dtype != torch.float32:
            logits = logits.float()
        dev = self.device
        pl, prev, prev_off = [], [], [0]
        penalised = False
        for r in requests:
            p = r.params
            pl += [float(p.repetition_penalty), float(p.frequency_penalty), float(p.presence_penalty)]
            if p.repetition_penalty != 1.0 or p.frequency_penalty != 0.0 or p.presence_penalty != 0.0:
                penalised = True
                prev.extend(int(t) for t in r.generated)
            prev_off.append(len(prev))
        if penalised:
            logits = logits.clone()
            kernels.apply_penalties(logits, torch.tensor(prev or [0], dtype=torch.int32).to(dev),
                                    torch.tensor(prev_off, dtype=torch.int32).to(dev),
                                    torch.tensor(pl, dtype=torch.float32).to(dev))
        out = torch.empty(n + (4 if status is not None else 0), dtype=torch.int32, device=dev)
        kernels.sample_rows(logits.contiguous(), slots, row_slot.contiguous(), out[:n],
                            all_greedy=all(r.params.temperature <= 0.0 for r in requests))
        if status is not None:
            out[n:].copy_(status)
        host = torch.empty(out.shape, dtype=torch.int32, pin_memory=True)
        host.copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return Sampled(host, n, event, status)
