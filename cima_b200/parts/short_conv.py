"""A short causal convolution over time in front of a sublayer, added to its input:

    u_t = h_t + sum_{j < taps} w[:, j] * h_(t - taps + 1 + j)         per channel, zeros before a sequence's start.

A sequence's newest ``taps - 1`` inputs travel with it as state (``StateRequest``: [slots, taps - 1, channels] in the
activations' dtype, zeroed when a slot opens, which is exactly the zeros before the start), so a step's first
rows find their predecessors whether the sequence starts, goes on by one token or by many.  The weight
[channels, taps] is kept in float32 and tap by tap ([taps, channels]: neighbouring threads read neighbouring
values); products and sums are float32.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.kv import StateRequest
from ..weights.loader import TensorSpec


class ShortConv:
    def __init__(self, spec, rt):
        if spec.taps < 1 or spec.taps > 16:
            raise ValueError(f"short_conv: {spec.taps} taps are outside 1..16")
        self.spec, self.rt = spec, rt
        self.weight = None

    def plan(self, name: str) -> Dict[str, TensorSpec]:
        return {name: TensorSpec((self.spec.channels, self.spec.taps), std=0.2)}

    def load(self, tensors, name: str) -> None:
        self.weight = self.rt.vector(tensors[name]).t().contiguous()          # [taps, channels]

    def state(self, name: str) -> Dict[str, torch.Tensor]:
        return {name: self.weight.t()}

    def nbytes(self) -> int:
        return self.weight.numel() * 4

    graph_safe = True

    @staticmethod
    def state_name(site: int) -> str:
        return f"short_conv.{site}"

    def cache_requests(self, site: int) -> List[object]:
        if self.spec.taps == 1:
            return []
        return [StateRequest(self.state_name(site), (self.spec.taps - 1, self.spec.channels), self.rt.dtype)]

    def forward(self, h: torch.Tensor, batch, cache, site: int) -> torch.Tensor:
        out = self.rt.empty(*h.shape)
        state = cache.state[self.state_name(site)] if self.spec.taps > 1 else None
        self.rt.kernels.short_conv(h, self.weight, state, batch, out)
        return out
