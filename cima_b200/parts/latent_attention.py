"""Causal attention over latents, without position encoding.

Every position keeps ONE vector c of ``kv_rank`` values, c = RMSNorm(W_d u) (its own norm weight); head h's key
and value are k = W_uk[h] c and v = W_uv[h] c, of ``head_dim`` and ``v_dim`` values.  Nothing but c is cached,
and it is cached once (a cache request of one plane): it serves as key and as value.

The step never builds k or v.  Since q.k = q.(W_uk[h] c) = (W_uk[h]^T q).c and sum_s p_s v_s = W_uv[h] (sum_s p_s c_s),

    qa[t, h] = W_uk[h]^T q[t, h]                  the query moved into the latents' space   (kv_rank values)
    ol[t, h] = softmax_s(scale * qa[t, h] . c_s) c_s      attention of all heads over ONE shared "kv head" c
    a[t, h]  = W_uv[h] ol[t, h]                   and out again                               (v_dim values)
    x       += W_o a

so the attention kernels of the grouped-query mixer serve: ``heads`` query heads on one kv head of ``kv_rank``
values whose pages hold one plane.  The step appends its latents first and every row reads the pages, whether
the sequences start or go on.  A layer with ``cache_from`` makes no latents and reads that site's pages with its
own W_uk and W_uv.  Scores and softmax are float32 in every attention kernel; the latent's norm is float32.

Sizes and constants (heads, head_dim, v_dim, kv_rank, scale, the latent norm's eps) are the spec's.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.kv import KVRequest
from ..weights.loader import TensorSpec
from .linear import Linear
from .registry import register_mixer


class LatentAttention:
    def __init__(self, spec, layer: int, rt):
        p = spec.params
        self.heads, self.dim = spec.n_heads, spec.head_dim
        self.vdim, self.rank, self.latent_eps = int(p["v_dim"]), int(p["kv_rank"]), float(p["latent_eps"])
        if min(self.heads, self.dim, self.vdim, self.rank) <= 0:
            raise ValueError(f"latent_attention: heads {self.heads}, head_dim {self.dim}, v_dim {self.vdim} and kv_rank "
                             f"{self.rank} must be positive")
        if spec.window:
            raise ValueError("latent_attention: a window is not implemented")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.own = spec.cache_from is None
        self.qd, self.od = self.heads * self.dim, self.heads * self.vdim
        self.q_latent = None       # W_q (and W_d under it) as one matrix
        self.latent_norm = None    # float32 [kv_rank]
        self.k_up_t = None         # [heads, kv_rank, head_dim]: W_uk's heads, transposed
        self.v_up = None           # [heads, v_dim, kv_rank]
        self.out = None

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _n(prefix, names, key):
        return f"{prefix}{names[key]}{names.get('suffix', '.weight')}"

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        s = self.spec
        p = {self._n(prefix, names, "q"): TensorSpec((self.qd, s.hidden))}
        if self.own:
            p[self._n(prefix, names, "latent")] = TensorSpec((self.rank, s.hidden))
            p[self._n(prefix, names, "latent_norm")] = TensorSpec((self.rank,), init="ones_normal")
        p[self._n(prefix, names, "k_up")] = TensorSpec((self.qd, self.rank), std=self.rank ** -0.5)
        p[self._n(prefix, names, "v_up")] = TensorSpec((self.od, self.rank), std=self.rank ** -0.5)
        p[self._n(prefix, names, "o")] = TensorSpec((s.hidden, self.od))
        return p

    def load(self, tensors, prefix: str, names: Dict[str, str]) -> None:
        rt = self.rt
        mats = [tensors[self._n(prefix, names, "q")]]
        if self.own:
            mats.append(tensors[self._n(prefix, names, "latent")])
            self.latent_norm = rt.vector(tensors[self._n(prefix, names, "latent_norm")])
        self.q_latent = Linear(mats, None, rt)
        del mats
        k_up = rt.matrix(tensors[self._n(prefix, names, "k_up")])
        self.k_up_t = k_up.view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        del k_up
        self.v_up = rt.matrix(tensors[self._n(prefix, names, "v_up")]).view(self.heads, self.vdim, self.rank)
        self.out = Linear(tensors[self._n(prefix, names, "o")], None, rt)
        if len({self.k_up_t.dtype, self.v_up.dtype, rt.dtype}) != 1:
            # a head's projection runs in the activations' dtype (a matrix stored in 32-bit is rounded on the bfloat16 path)
            self.k_up_t, self.v_up = self.k_up_t.to(rt.dtype), self.v_up.to(rt.dtype)

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        out = {self._n(prefix, names, "q"): self.q_latent.weight[:self.qd]}
        if self.own:
            out[self._n(prefix, names, "latent")] = self.q_latent.weight[self.qd:]
            out[self._n(prefix, names, "latent_norm")] = self.latent_norm
        out[self._n(prefix, names, "k_up")] = self.k_up_t.transpose(1, 2).reshape(self.qd, self.rank)
        out[self._n(prefix, names, "v_up")] = self.v_up.reshape(self.od, self.rank)
        out[self._n(prefix, names, "o")] = self.out.weight
        return out

    def nbytes(self) -> int:
        e = self.k_up_t.element_size()
        return (self.q_latent.nbytes() + self.out.nbytes() + (self.k_up_t.numel() + self.v_up.numel()) * e
                + (self.latent_norm.numel() * 4 if self.own else 0))

    def scratch_row(self) -> int:
        return self.qd + self.rank + 2 * self.heads * self.rank + self.od

    graph_safe = True

    @property
    def short_context(self) -> int:
        from ..kernels import short_context
        return short_context(self.rank)

    # ------------------------------------------------------------------ cache
    def cache_requests(self, site: int) -> List[object]:
        if not self.own:
            return []
        return [KVRequest(n_kv_heads=1, head_dim=self.rank, window=0, planes=1)]

    # ------------------------------------------------------------------ step
    def forward(self, u, x: torch.Tensor, batch, cache, site: int, next_norm=None):
        K_, rt = self.rt.kernels, self.rt
        if hasattr(u, "tensor"):
            u = u.tensor()
        rows = u.shape[0]
        kv = cache.layer_kv(site)
        ql = self.q_latent.store(u)                                  # [rows, heads * head_dim (+ kv_rank)]
        qa = rt.empty(rows, self.heads * self.rank)
        # (the step's latents go into the pages before the attention reads them: in the same launch for the few rows
        # of a decode step, in one of their own before it otherwise)
        K_.head_linear(ql[:, :self.qd], self.k_up_t, qa,
                       append=(ql[:, self.qd:], self.latent_norm, self.latent_eps, kv, batch) if self.own else None)
        ol = rt.empty(rows, self.heads * self.rank)
        K_.attention(qa, kv, batch, ol, self.heads, 1, self.rank, self.spec.scale, 0, True)
        att = rt.empty(rows, self.od)
        K_.head_linear(ol, self.v_up, att)
        return self.out.accumulate(att, x, next_norm)


register_mixer("latent_attention", LatentAttention)
