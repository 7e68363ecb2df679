"""Linear attention with one constant decay a head (mixer kind ``decay_attention``).

    q, k = silu(W_q h), silu(W_k h)   [heads, dim];     v = silu(W_v h)   [heads, v_dim]
    S_t = d_h * S_(t-1) + k_t v_t^T;                    o_t = S_t^T q_t                    per head, no other scale
    y   = W_o ( rms(o over all heads) * w  *  sigmoid(W_g h) )

The state S [heads, dim, v_dim] is float32, starts at zero and travels with the sequence (a ``StateRequest``); a step
walks its rows in order from the state the steps before left, so prompts, pieces of prompts and single tokens are one
path.  q | k | v | g are one product; SiLU is applied where the recurrence loads them.  Sizes (heads, head_dim, ``v_dim``),
the decays (``decay``, one a head) and the norm's ``eps`` are the spec's.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.kv import StateRequest
from ..weights.loader import TensorSpec
from .linear import Linear
from .registry import register_mixer


class DecayAttention:
    def __init__(self, spec, layer: int, rt):
        p = spec.params
        self.heads, self.dim, self.vdim = spec.n_heads, spec.head_dim, int(p["v_dim"])
        self.eps = float(p["eps"])
        decay = [float(d) for d in p["decay"]]
        if min(self.heads, self.dim, self.vdim) <= 0 or self.dim > 256:
            raise ValueError(f"decay_attention: heads {self.heads}, key size {self.dim} (at most 256) and value size {self.vdim} must be positive")
        if len(decay) != self.heads:
            raise ValueError(f"decay_attention: {len(decay)} decays for {self.heads} heads")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.decay_host = decay
        self.qd, self.vd = self.heads * self.dim, self.heads * self.vdim
        self.decay = self.proj = self.out = self.norm = None

    KEYS = ("q", "k", "v", "g")

    @staticmethod
    def _n(prefix, names, key):
        return f"{prefix}{names[key]}{names.get('suffix', '.weight')}"

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        H = self.spec.hidden
        return {self._n(prefix, names, "q"): TensorSpec((self.qd, H)), self._n(prefix, names, "k"): TensorSpec((self.qd, H)),
                self._n(prefix, names, "v"): TensorSpec((self.vd, H)), self._n(prefix, names, "g"): TensorSpec((self.vd, H)),
                self._n(prefix, names, "o"): TensorSpec((H, self.vd)),
                self._n(prefix, names, "norm"): TensorSpec((self.vd,), init="ones_normal")}

    def load(self, tensors, prefix: str, names: Dict[str, str]) -> None:
        self.proj = Linear([tensors[self._n(prefix, names, k)] for k in self.KEYS], None, self.rt)
        self.out = Linear(tensors[self._n(prefix, names, "o")], None, self.rt)
        self.norm = self.rt.vector(tensors[self._n(prefix, names, "norm")])
        self.decay = torch.tensor(self.decay_host, dtype=torch.float32, device=self.rt.device)

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        w, r, out = self.proj.weight, 0, {}
        for key, rows in zip(self.KEYS, (self.qd, self.qd, self.vd, self.vd)):
            out[self._n(prefix, names, key)] = w[r:r + rows]
            r += rows
        out[self._n(prefix, names, "o")] = self.out.weight
        out[self._n(prefix, names, "norm")] = self.norm
        return out

    def nbytes(self) -> int:
        return self.proj.nbytes() + self.out.nbytes() + self.norm.numel() * 4

    def scratch_row(self) -> int:
        return 2 * self.qd + 5 * self.vd

    graph_safe = True

    @staticmethod
    def state_name(site: int) -> str:
        return f"decay_attention.{site}"

    def cache_requests(self, site: int) -> List[object]:
        return [StateRequest(self.state_name(site), (self.heads, self.dim, self.vdim), torch.float32)]

    def forward(self, h, x: torch.Tensor, batch, cache, site: int, next_norm=None):
        return self.out.accumulate(self._gated(h, batch, cache, site), x, next_norm)

    def produce(self, h, batch, cache, site: int) -> torch.Tensor:
        """The mixer's output as float32 rows of its own (what ``forward`` adds into x)."""
        return self.out.logits(self._gated(h, batch, cache, site))

    def _gated(self, h, batch, cache, site: int) -> torch.Tensor:
        K_, rt = self.rt.kernels, self.rt
        if hasattr(h, "tensor"):
            h = h.tensor()
        rows, qd, vd = h.shape[0], self.qd, self.vd
        p = self.proj.store(h)                                        # [rows, q | k | v | g]
        o = rt.empty(rows, vd, dtype=torch.float32)
        K_.recurrence(p[:, :qd], p[:, qd:2 * qd], p[:, 2 * qd:2 * qd + vd], cache.state[self.state_name(site)], batch, o,
                      self.heads, self.heads, self.dim, self.vdim, decay=self.decay)
        gated = rt.empty(rows, vd)
        K_.group_rmsnorm_gate(o, self.norm, p[:, 2 * qd + vd:], gated, 1, self.eps)
        return gated


register_mixer("decay_attention", DecayAttention)
