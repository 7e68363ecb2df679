"""The gated delta rule with one decay a key channel (mixer kind ``channel_delta``).

    q, k = silu(conv(W_q h)), silu(conv(W_k h))  [kv_heads, dim];   v = silu(conv(W_v h))  [heads, v_dim]
           conv: a causal convolution over time on each channel (``taps`` taps, zeros before the start, no bias)
    q, k  -> unit vectors per head, x / sqrt(sum x^2 + 1e-6);  q also times dim^(-1/2)
    beta  = sigmoid(W_b h)                                               one a head
    g     = exp(-exp(A_log[h]) * softplus(W_a2 (W_a1 h) + dt_bias))       one a head and key channel
    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q       per head, in this order
    y     = W_o ( rms(o over a head's values) * w * sigmoid(W_g2 (W_g1 h)) )

Head h reads q/k head h // (heads / kv_heads).  Per sequence the mixer keeps S [heads, dim, v_dim] in float32 and the
convolution's newest ``taps - 1`` inputs (two ``StateRequest``s, zeroed when a slot opens: those zeros are the zeros
before the start).  Unit norms, decays, step sizes and the recurrence are float32; projections and the convolution
with its activation run in the activations' dtype.  The ranks of the two low-rank pairs (a1/a2, g1/g2) are
``a_rank`` and ``g_rank``.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.kv import StateRequest
from ..config.specs import ShortConvSpec
from ..weights.loader import TensorSpec
from .linear import Linear
from .registry import register_mixer
from .short_conv import ShortConv


class ChannelDelta:
    def __init__(self, spec, layer: int, rt):
        from ..kernels import ACTIVATIONS
        p = spec.params
        self.heads, self.kv_heads, self.dim, self.vdim = spec.n_heads, spec.n_kv_heads, spec.head_dim, int(p["v_dim"])
        self.taps, self.eps = int(p["taps"]), float(p["eps"])
        self.a_rank, self.g_rank = int(p["a_rank"]), int(p["g_rank"])
        if min(self.heads, self.kv_heads, self.dim, self.vdim, self.a_rank, self.g_rank) <= 0 or self.dim > 256:
            raise ValueError("channel_delta: heads, key heads, key size (at most 256), value size and ranks must be positive")
        if self.heads % self.kv_heads:
            raise ValueError(f"channel_delta: {self.heads} heads are not a multiple of {self.kv_heads} key heads")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.kd, self.vd, self.gd = self.kv_heads * self.dim, self.heads * self.vdim, self.heads * self.dim
        self.channels = 2 * self.kd + self.vd
        self.conv = ShortConv(ShortConvSpec(channels=self.channels, taps=self.taps), rt)
        self.silu = ACTIVATIONS["silu"]
        self.qkv = self.b = self.a1 = self.a2 = self.g1 = self.g2 = self.out = None
        self.A_log = self.dt_bias = self.norm = None

    @staticmethod
    def _n(prefix, names, key, tail=""):
        return f"{prefix}{names[key]}{tail}{names.get('suffix', '.weight')}"

    def _shapes(self):
        H = self.spec.hidden
        return {"q": (self.kd, H), "k": (self.kd, H), "v": (self.vd, H), "b": (self.heads, H), "a1": (self.a_rank, H),
                "a2": (self.gd, self.a_rank), "g1": (self.g_rank, H), "g2": (self.vd, self.g_rank), "o": (H, self.vd)}

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        p = {self._n(prefix, names, k): TensorSpec(s, std=0.1 if k in ("a2", "g2") else 0.02) for k, s in self._shapes().items()}
        for k, rows in (("q", self.kd), ("k", self.kd), ("v", self.vd)):
            p[self._n(prefix, names, k, ".conv")] = TensorSpec((rows, self.taps), std=0.3)
        p[self._n(prefix, names, "A_log")] = TensorSpec((self.heads,), std=0.5)
        p[self._n(prefix, names, "dt_bias")] = TensorSpec((self.gd,), std=0.5)
        p[self._n(prefix, names, "norm")] = TensorSpec((self.vdim,), init="ones_normal")
        return p

    def load(self, tensors, prefix: str, names: Dict[str, str]) -> None:
        rt = self.rt
        self.qkv = Linear([tensors[self._n(prefix, names, k)] for k in ("q", "k", "v")], None, rt)
        for k in ("b", "a1", "a2", "g1", "g2"):
            setattr(self, k, Linear(tensors[self._n(prefix, names, k)], None, rt))
        self.out = Linear(tensors[self._n(prefix, names, "o")], None, rt)
        taps = torch.cat([tensors[self._n(prefix, names, k, ".conv")].float() for k in ("q", "k", "v")])
        self.conv.load({"w": taps}, "w")
        self.A_log = rt.vector(tensors[self._n(prefix, names, "A_log")])
        self.dt_bias = rt.vector(tensors[self._n(prefix, names, "dt_bias")])
        self.norm = rt.vector(tensors[self._n(prefix, names, "norm")])

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        out, r = {}, 0
        taps = self.conv.weight.t()
        for k, rows in (("q", self.kd), ("k", self.kd), ("v", self.vd)):
            out[self._n(prefix, names, k)] = self.qkv.weight[r:r + rows]
            out[self._n(prefix, names, k, ".conv")] = taps[r:r + rows]
            r += rows
        for k in ("b", "a1", "a2", "g1", "g2"):
            out[self._n(prefix, names, k)] = getattr(self, k).weight
        out[self._n(prefix, names, "o")] = self.out.weight
        out[self._n(prefix, names, "A_log")] = self.A_log
        out[self._n(prefix, names, "dt_bias")] = self.dt_bias
        out[self._n(prefix, names, "norm")] = self.norm
        return out

    def nbytes(self) -> int:
        return (sum(getattr(self, k).nbytes() for k in ("qkv", "b", "a1", "a2", "g1", "g2", "out")) + self.conv.nbytes()
                + (self.A_log.numel() + self.dt_bias.numel() + self.norm.numel()) * 4)

    def scratch_row(self) -> int:
        return 2 * self.channels + 4 * self.kd + 3 * self.gd + 5 * self.vd

    graph_safe = True

    @staticmethod
    def state_name(site: int) -> str:
        return f"channel_delta.{site}"

    def cache_requests(self, site: int) -> List[object]:
        return [StateRequest(self.state_name(site), (self.heads, self.dim, self.vdim), torch.float32)] + self.conv.cache_requests(site)

    def forward(self, h, x: torch.Tensor, batch, cache, site: int, next_norm=None):
        return self.out.accumulate(self._gated(h, batch, cache, site), x, next_norm)

    def produce(self, h, batch, cache, site: int) -> torch.Tensor:
        """The mixer's output as float32 rows of its own (what ``forward`` adds into x)."""
        return self.out.logits(self._gated(h, batch, cache, site))

    def _gated(self, h, batch, cache, site: int) -> torch.Tensor:
        K_, rt = self.rt.kernels, self.rt
        if hasattr(h, "tensor"):
            h = h.tensor()
        rows, kd = h.shape[0], self.kd
        raw = self.qkv.store(h)                                       # [rows, q | k | v]
        c = rt.empty(rows, self.channels)
        conv_state = cache.state[self.conv.state_name(site)] if self.taps > 1 else None
        K_.short_conv(raw, self.conv.weight, conv_state, batch, c, add_input=False, act=self.silu)
        a = self.a2.store(self.a1.store(h))
        b = self.b.store(h)
        f32 = torch.float32
        qn, kn = rt.empty(rows, kd, dtype=f32), rt.empty(rows, kd, dtype=f32)
        g, beta = rt.empty(rows, self.gd, dtype=f32), rt.empty(rows, self.heads, dtype=f32)
        K_.delta_prepare(c, a, b, self.A_log, self.dt_bias, qn, kn, g, beta, self.heads, self.kv_heads, self.dim)
        o = rt.empty(rows, self.vd, dtype=f32)
        K_.recurrence(qn, kn, c[:, 2 * kd:], cache.state[self.state_name(site)], batch, o, self.heads, self.kv_heads, self.dim,
                      self.vdim, g=g, beta=beta)
        gate = self.g2.store(self.g1.store(h))
        gated = rt.empty(rows, self.vd)
        K_.group_rmsnorm_gate(o, self.norm, gate, gated, self.heads, self.eps)
        return gated


register_mixer("channel_delta", ChannelDelta)
