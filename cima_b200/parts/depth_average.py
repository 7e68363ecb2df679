"""Depth average of the residual streams: what a layer reads is a weighted sum of every stream before it.

With X_0 the embedding's output and X_(s+1) the stream as the layer at site s leaves it (its input plus its
sublayers' outputs), the next site, and after the last one the final norm, reads

    x = sum_{j <= s+1} a_s[j] * X_j                  a_s: the s + 2 values of site s's vector, float32.

A step keeps the streams as planes of one float32 buffer [sites + 2, rows, hidden]: plane s + 1 starts as the
input of site s and becomes X_(s+1) as its sublayers add into it, so the sum for site s is written straight into
plane s + 2, the next site's input; the norm that reads it runs in the same kernel.
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from ..weights.loader import TensorSpec
from .norm import RowsInfo


class DepthAverage:
    def __init__(self, names: Sequence[str], rt):
        self.names, self.rt = list(names), rt
        self.weights = [None] * len(self.names)

    def plan(self) -> Dict[str, TensorSpec]:
        return {n: TensorSpec((s + 2,), init="mean", std=0.3) for s, n in enumerate(self.names)}

    def load(self, tensors) -> None:
        self.weights = [self.rt.vector(tensors[n]) for n in self.names]

    def state(self) -> Dict[str, torch.Tensor]:
        return dict(zip(self.names, self.weights))

    def nbytes(self) -> int:
        return sum(w.numel() * 4 for w in self.weights)

    graph_safe = True

    def begin(self, rows: int, hidden: int) -> torch.Tensor:
        """The step's streams [sites + 2, rows, hidden]; the embedding goes to plane 0 (``start`` copies it on)."""
        return self.rt.empty(len(self.names) + 2, rows, hidden, dtype=torch.float32)

    def start(self, stack: torch.Tensor) -> torch.Tensor:
        stack[1].copy_(stack[0])
        return stack[1]

    def after(self, stack: torch.Tensor, site: int, next_norm=None, next_conv=None):
        """The input of the site after ``site`` (or of the final norm) and, where the norm that reads it is a plain
        RMSNorm, that norm's output with it.  ``next_conv = (conv, batch, cache, site)``: the short convolution that
        reads that norm's output; in a step of one row a sequence it runs in the same kernel, and its result travels
        with the rows (``RowsInfo.conv`` / ``.u``)."""
        x = stack[site + 2]
        if (next_norm is not None and getattr(next_norm, "weight", None) is not None
                and next_norm.spec.kind == "rmsnorm" and next_norm.spec.size == x.shape[1]):
            h = self.rt.empty(*x.shape)
            info = RowsInfo(norm=next_norm, h=h)
            fused = None
            if next_conv is not None and next_conv[1].n_rows == next_conv[1].n_seqs:
                conv, batch, cache, conv_site = next_conv
                u = self.rt.empty(*x.shape)
                state = cache.state[conv.state_name(conv_site)] if conv.spec.taps > 1 else None
                fused = (conv.weight, state, batch.seq_slot, u)
                info.conv, info.u = conv, u
            self.rt.kernels.depth_average(stack, site + 2, self.weights[site], x, next_norm.weight, next_norm.spec.eps, h,
                                          conv=fused)
            return x, info
        self.rt.kernels.depth_average(stack, site + 2, self.weights[site], x)
        return x, None
