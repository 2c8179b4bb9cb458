"""Partial rotary position encoding with optional sections.

``inv_freq[j] = theta ** (-2j / rotary_dim)`` for the ``rotary_dim / 2`` rotate-half pairs ``(j, j +
rotary_dim/2)`` of the first ``rotary_dim`` dims of a head; the rest of the head is not rotated
(src/quanta/minimax/model_m3.py:68-96).  With ``sections`` the pairs are split into runs, run ``a``
taking position axis ``a`` (src/quanta/minimax/model_vision_m3.py:155-163); a text token feeds its
one position to every axis, so the numbers equal the unsectioned ladder.
"""

from __future__ import annotations

import torch

from .base import PositionEncoding, register


@register("position", "partial_rotary")
class PartialRotary(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, rotary_dim: int, theta: float, sections=None):
        if rotary_dim % 2 or not 0 <= rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        if sections is not None and sum(sections) != rotary_dim // 2:
            raise ValueError(f"rope sections {list(sections)} do not sum to rotary_dim/2 = {rotary_dim // 2}")
        self.head_dim, self.rotary_dim, self.theta = int(head_dim), int(rotary_dim), float(theta)
        self.sections = None if sections is None else tuple(int(s) for s in sections)
        self.n_axes = 1 if self.sections is None else len(self.sections)
        self._tables = {}

    def inv_freq(self) -> torch.Tensor:
        rd = self.rotary_dim
        return 1.0 / (self.theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))

    def rotary_tables(self, device):
        if self.rotary_dim == 0:
            return None
        key = str(device)
        if key not in self._tables:
            inv = self.inv_freq().to(device)
            axis = None
            if self.sections is not None:
                axis = torch.cat([torch.full((n,), a, dtype=torch.int32) for a, n in enumerate(self.sections)])
                axis = axis.to(device)
            self._tables[key] = (inv, axis, self.rotary_dim, self.n_axes)
        return self._tables[key]
