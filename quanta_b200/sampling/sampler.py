"""The device sampler: one row of float32 logits per request that samples this step.

Greedy when ``temperature <= 0`` (first maximum); else temperature, top-k, top-p, min-p and a
categorical draw, after the repetition / frequency / presence penalties over the tokens the request
has generated so far (src/quanta/minimax/generate.py:56-80, src/quanta/shim/omlx.py:344-363,
1796-1810).  The draw is Gumbel-max with counter-based noise keyed by (seed, token, draw number), so
the same seed gives the same tokens whatever else shares the batch.  One device->host copy of the
sampled ids per step.
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

    def sample(self, logits: torch.Tensor, requests: list, status: torch.Tensor | None = None) -> list[int]:
        """``logits`` [n, vocab] float32 on the device, ``requests[i]`` has ``.params`` and
        ``.generated``.  Returns n token ids (host).  If ``status`` is given its words are read in the
        same copy and a device-side refusal raises."""
        return self.sample_async(logits, requests, status).read()

    def sample_async(self, logits: torch.Tensor, requests: list, status: torch.Tensor | None = None, *,
                     drawn_before: int = 0, scatter=None) -> Sampled:
        """Launch the sampling and the copy of the ids to the host; ``read()`` of the result gives them.
        ``drawn_before``: tokens each request has sampled that are not in ``.generated`` yet (their draw
        numbers are taken).  ``scatter``: ``(table, rows)`` device tensors: ``table[rows[i]] = id i`` as
        well, for a step that takes its ids from the device."""
        n, V = logits.shape
        if n != len(requests):
            raise ValueError(f"{n} logits rows for {len(requests)} requests")
        if logits.dtype != torch.float32:
            logits = logits.float()
        fl, il, pl, prev, prev_off = [], [], [], [], [0]
        penalised = False
        for r in requests:
            p = r.params
            seed = int(p.seed) & 0xFFFFFFFFFFFFFFFF
            lo, hi = seed & 0xFFFFFFFF, seed >> 32
            fl += [float(p.temperature), float(p.top_p), float(p.min_p), 0.0]
            il += [int(p.top_k), lo - (1 << 32) if lo >= (1 << 31) else lo, hi - (1 << 32) if hi >= (1 << 31) else hi,
                   len(r.generated) + drawn_before]
            pl += [float(p.repetition_penalty), float(p.frequency_penalty), float(p.presence_penalty)]
            if p.repetition_penalty != 1.0 or p.frequency_penalty != 0.0 or p.presence_penalty != 0.0:
                penalised = True
                prev.extend(int(t) for t in r.generated)
            prev_off.append(len(prev))
        dev = self.device
        if all(r.params.temperature <= 0.0 for r in requests):
            fparams = iparams = None
        else:
            fparams = torch.tensor(fl, dtype=torch.float32).to(dev, non_blocking=True)
            iparams = torch.tensor(il, dtype=torch.int32).to(dev, non_blocking=True)
        if penalised:
            logits = logits.clone()
            kernels.apply_penalties(logits, torch.tensor(prev or [0], dtype=torch.int32).to(dev),
                                    torch.tensor(prev_off, dtype=torch.int32).to(dev),
                                    torch.tensor(pl, dtype=torch.float32).to(dev))
        out = torch.empty(n + (4 if status is not None else 0), dtype=torch.int32, device=dev)
        kernels.sample_rows(logits.contiguous(), fparams, iparams, out[:n])
        if scatter is not None:
            table, rows = scatter
            table.index_copy_(0, rows.long(), out[:n])
        if status is not None:
            out[n:].copy_(status)
        host = torch.empty(out.shape, dtype=torch.int32, pin_memory=True)
        host.copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return Sampled(host, n, event, status)
