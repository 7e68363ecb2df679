"""Plain, slow implementation of the Vunovik decoder: the oracle of its tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 by default.  It shares no
code with the ``cima_b200`` package: the configuration is a plain dict with config.json's own keys, the
weights a plain dict name -> tensor.

The design in this file's notation (T tokens, width W, layer i, all sums over the visible past only):

  x_0       = s_e * E[token]                                   embedding, s_e = embedding.scale
  h         = x / sqrt(mean(x^2) + eps) * g                    the layer's one norm
  u_t       = h_t + sum_{j<taps} A[:, j] * h_{t-taps+1+j}      causal per-channel convolution, zeros before position 0
  c_t       = rms(Wd u_t) * g_c                                the latent (kv_rank values), the only thing kept per position
  q_t       = Wq u_t;  k_s = Wuk c_s;  v_s = Wuv c_s           per head slices of dim / dim / vdim values
  a_t       = sum_{s<=t} softmax_s(scale * q_t . k_s) v_s      per head, ordinary softmax, no positions
  m_t       = Wo a_t
  f_t       = Wdown (relu(Wgate h_t) * (Wup h_t))              reads h, not u
  X_{i+1}   = x + (m + f)                                      both sublayers read the same norm
  x         = sum_{j<=i+1} d_i[j] * X_j                        depth average: what the next layer (or the output) reads
  logits    = E (x / sqrt(mean(x^2) + eps) * g_f)              the table itself, unscaled

A layer with ``kv_from = j`` has no Wd: it reads layer j's latents.
"""
from __future__ import annotations

import torch


def plain_embed(table: torch.Tensor, ids, scale: float) -> torch.Tensor:
    return table[torch.as_tensor(ids, dtype=torch.long)] * scale


def plain_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return plain_rms(x, eps) * w


def plain_canon(h: torch.Tensor, taps_w: torch.Tensor) -> torch.Tensor:
    """h [T, W], taps_w [W, taps]: u_t = h_t + sum_j taps_w[:, j] * h_{t - taps + 1 + j} (zeros before the start)."""
    T, W = h.shape
    taps = taps_w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += taps_w[:, j] * h[s]
    return out


def plain_latent(u: torch.Tensor, w_dkv: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return plain_rmsnorm(u @ w_dkv.T, g, eps)


def plain_latent_attention(u: torch.Tensor, c: torch.Tensor, w_q, w_uk, w_uv, w_o, heads: int, dim: int,
                           vdim: int, scale: float) -> torch.Tensor:
    """u [T, W] the mixer's input, c [T, R] the latents (own or another layer's)."""
    T = u.shape[0]
    q = (u @ w_q.T).view(T, heads, dim)
    k = (c @ w_uk.T).view(T, heads, dim)
    v = (c @ w_uv.T).view(T, heads, vdim)
    att = torch.zeros(T, heads, vdim, dtype=u.dtype)
    hidden = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)        # [query, key]: key after query
    for hd in range(heads):
        s = (q[:, hd] @ k[:, hd].T) * scale
        p = torch.softmax(s.masked_fill(hidden, float("-inf")), dim=1)
        att[:, hd] = p @ v[:, hd]
    return att.reshape(T, heads * vdim) @ w_o.T


def plain_latent_attention_one(u_t: torch.Tensor, c_past: torch.Tensor, w_q, w_uk, w_uv, w_o, heads: int, dim: int,
                               vdim: int, scale: float) -> torch.Tensor:
    """One position on its own, key by key: u_t [W] its input, c_past [n, R] the latents of positions 0 .. t."""
    q = (w_q @ u_t).view(heads, dim)
    out = torch.zeros(heads, vdim, dtype=u_t.dtype)
    for hd in range(heads):
        ks = [w_uk[hd * dim:(hd + 1) * dim] @ c for c in c_past]
        vs = [w_uv[hd * vdim:(hd + 1) * vdim] @ c for c in c_past]
        s = torch.stack([(kk * q[hd]).sum() * scale for kk in ks])
        p = torch.exp(s - s.max())
        p = p / p.sum()
        for pj, vj in zip(p, vs):
            out[hd] += pj * vj
    return w_o @ out.reshape(heads * vdim)


def plain_gated(h: torch.Tensor, w_gate, w_up, w_down) -> torch.Tensor:
    return (torch.relu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def plain_depth_average(streams, weights: torch.Tensor) -> torch.Tensor:
    assert len(streams) == weights.numel()
    out = torch.zeros_like(streams[0])
    for j, X in enumerate(streams):
        out = out + weights[j] * X
    return out


# --------------------------------------------------------------------------- the model

def plain_forward(config: dict, tensors: dict, ids, dtype=torch.float64):
    """Logits [T, vocab] of one whole sequence, and the stream after every layer [layers, T, W]."""
    w = {k: v.to(dtype) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = plain_embed(w["embed"], ids, float(config["embedding"]["scale"]))
    streams = [x]
    latents = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        assert layer["type"] == "latent_attention"
        m = layer["mixer"]
        h = plain_rmsnorm(x, w[p + "norm1"], eps)
        u = plain_canon(h, w[p + "canon1"])
        src = m.get("kv_from")
        if src is None:
            latents[i] = plain_latent(u, w[p + "mix.dkv"], w[p + "mix.dkv.norm"], eps)
            src = i
        y = plain_latent_attention(u, latents[src], w[p + "mix.q"], w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.o"],
                                   m["heads"], m["dim"], m["vdim"], float(m["scale"]))
        if layer.get("mlp") is not None:
            assert layer["mlp"]["kind"] == "dense"
            y = y + plain_gated(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
        streams.append(x + y)
        x = plain_depth_average(streams, w[p + "dwa"])
        after.append(x)
    logits = plain_rmsnorm(x, w["final.norm"], eps) @ w["embed"].T
    return logits, torch.stack(after)
