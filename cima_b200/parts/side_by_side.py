"""Several mixers side by side (mixer kind ``side_by_side``): all read the same input, and the result is the mean of
their outputs, each first divided by its root mean square over the model width and multiplied by a weight of its own:

    y = (1 / B) * sum_b  rms(mixer_b(h)) * w_b                     rms(z) = z / sqrt(mean(z^2) + eps)

The branches are ordinary mixers, built through the registry from ``params["branches"]`` (a list of ``MixerSpec``) with
their tensor names from ``params["branch_names"]`` (one dict a branch; key "out" names the branch's weight w_b).
Each adds into a zeroed float32 buffer of its own; one kernel norms and averages them into the rows the mixer was
given.  Cache and state requests are the branches' own: at most one branch may keep keys and values (a site owns one
place in the cache's groups), any number may keep state.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.kv import KVRequest
from ..weights.loader import TensorSpec
from .registry import build_mixer, register_mixer


class SideBySide:
    def __init__(self, spec, layer: int, rt):
        p = spec.params
        self.spec, self.layer, self.rt = spec, layer, rt
        self.eps = float(p["eps"])
        self.branch_names: List[Dict[str, str]] = [dict(n) for n in p["branch_names"]]
        self.branches = [build_mixer(s, layer, rt) for s in p["branches"]]
        if not (1 <= len(self.branches) <= 4) or len(self.branch_names) != len(self.branches):
            raise ValueError(f"side_by_side: {len(self.branches)} branches with {len(self.branch_names)} name tables; 1 to 4 of each")
        self.weights = [None] * len(self.branches)

    def _out_name(self, prefix: str, i: int) -> str:
        n = self.branch_names[i]
        return f"{prefix}{n['out']}{n.get('suffix', '.weight')}"

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        p: Dict[str, TensorSpec] = {}
        for i, b in enumerate(self.branches):
            p.update(b.plan(prefix, self.branch_names[i]))
            p[self._out_name(prefix, i)] = TensorSpec((self.spec.hidden,), init="ones_normal")
        return p

    def load(self, tensors, prefix: str, names: Dict[str, str]) -> None:
        for i, b in enumerate(self.branches):
            b.load(tensors, prefix, self.branch_names[i])
            self.weights[i] = self.rt.vector(tensors[self._out_name(prefix, i)])

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for i, b in enumerate(self.branches):
            out.update(b.state(prefix, self.branch_names[i]))
            out[self._out_name(prefix, i)] = self.weights[i]
        return out

    def nbytes(self) -> int:
        return sum(b.nbytes() for b in self.branches) + sum(w.numel() * 4 for w in self.weights)

    def scratch_row(self) -> int:
        return max(int(getattr(b, "scratch_row", lambda: 0)()) for b in self.branches) + 2 * len(self.branches) * self.spec.hidden

    @property
    def graph_safe(self) -> bool:
        return all(getattr(b, "graph_safe", False) for b in self.branches)

    @property
    def short_context(self) -> int:
        named = [int(getattr(b, "short_context", 0) or 0) for b in self.branches]
        named = [n for n in named if n > 0]
        return min(named) if named else 0

    def cache_requests(self, site: int) -> List[object]:
        reqs: List[object] = []
        for b in self.branches:
            reqs += list(b.cache_requests(site))
        if sum(isinstance(r, KVRequest) for r in reqs) > 1:
            raise ValueError("side_by_side: more than one branch keeps keys and values; a site has one place in the cache")
        return reqs

    def _branch_outputs(self, h, like: torch.Tensor, batch, cache, site: int):
        """Every branch's output as float32 rows of its own: from its ``produce`` where it has one, else added into zeros."""
        ys = []
        for b in self.branches:
            if hasattr(b, "produce"):
                ys.append(b.produce(h, batch, cache, site))
            else:
                y = torch.zeros_like(like)
                b.forward(h, y, batch, cache, site)
                ys.append(y)
        return ys

    def forward(self, h, x: torch.Tensor, batch, cache, site: int, next_norm=None):
        if hasattr(h, "tensor"):
            h = h.tensor()
        self.rt.kernels.rms_mean(self._branch_outputs(h, x, batch, cache, site), self.weights, x, self.eps)
        return None

    def produce(self, h, batch, cache, site: int) -> torch.Tensor:
        if hasattr(h, "tensor"):
            h = h.tensor()
        y = self.rt.empty(h.shape[0], self.spec.hidden, dtype=torch.float32)
        self.rt.kernels.rms_mean(self._branch_outputs(h, y, batch, cache, site), self.weights, y, self.eps, assign=True)
        return y


register_mixer("side_by_side", SideBySide)
