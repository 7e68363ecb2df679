"""Plain, slow implementation of the Gisirax decoder: the oracle of its tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 by default.  It shares no code
with the ``cima_b200`` package: the configuration is a plain dict with config.json's own keys, the weights a
plain dict name -> tensor (``read_folder`` reads both from a model folder with nothing but the standard library
and torch).

The design in this file's notation (T tokens of one sequence, width W, t a position counted from 0):

  x_t        = s_e E[tok_t] + B[(tok_(t-1) a_p + tok_t a_c) mod n]      B's last row (number n) for t = 0
  N(x)       = tanh(alpha x) * w + b                                     every norm of a layer, and the last one
  x         <- x + m N1b(mixer(N1(x)));   x <- x + m N2b(ff(N2(x)))      m = residual_mult
  logits     = H N_f(x)

  mixer "parallel":  (rms(L(h)) * w_l + rms(R(h)) * w_r) / 2, rms over the width, with
     L  softmax attention: q, k rotated on their first r dims (pairs (i, i + r/2), frequencies base^(-2i/r) rescaled by
        the wavelength rule below), grouped heads, scores q.k * scale, causal, and a denominator 1 + sum exp(s)
     R  linear attention: q, k, v through silu; per head S <- d_h S + k v^T, o = S^T q; all heads' o normed together
        (rms * w), times sigmoid(Wg h), then Wo
  mixer "channel_delta":  q, k, v = silu(conv(W h)) (causal per-channel taps); q, k to unit length per head, q also
        times dim^(-1/2); beta = sigmoid(Wb h); g = exp(-exp(A_h) softplus(Wa2 Wa1 h + dt)) per head and key channel;
        S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;  rms(o) * w per head, times
        sigmoid(Wg2 Wg1 h), then Wo
  ff "moe":  scores sigmoid(Wr h); groups of neighbouring experts scored by their two best; the best `keep` groups
        stay; the `top` best experts among them, weights s / (sum s + 1e-20) * scale; experts Wd(silu(Wg h) * Wu h)

rms(x) = x / sqrt(mean(x^2) + eps).
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch


# ---------------------------------------------------------------------------------------------- files
def read_folder(folder: str, dtype=torch.float64):
    """(config dict, {name: tensor}) of a model folder; floating tensors in ``dtype``, integer ones as they are."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64, "I32": torch.int32,
             "I64": torch.int64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, out


# ---------------------------------------------------------------------------------------------- small pieces
def plain_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def plain_dyt(x, w, b, alpha):
    return torch.tanh(alpha * x) * w + b


def plain_silu(z):
    return z * torch.sigmoid(z)


def plain_embedding(ids, table, bigram, scale: float, buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    rows = []
    for t, tok in enumerate(ids):
        r = buckets if t == 0 else (int(ids[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets
        rows.append(table[int(tok)] * scale + bigram[r])
    return torch.stack(rows)


# ---------------------------------------------------------------------------------------------- rotary positions
def plain_rotary_frequencies(dims: int, base: float, scaling=None) -> torch.Tensor:
    """f_i = base^(-2i/dims), i < dims/2, then the wavelength rule: short waves stay, long ones are divided by
    ``factor``, those between are blended."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < orig / hi:
                out.append(fi)
            elif wave > orig / lo:
                out.append(fi / fac)
            else:
                s = (orig / wave - lo) / (hi - lo)
                out.append((1.0 - s) * fi / fac + s * fi)
        f = out
    return torch.tensor(f, dtype=torch.float64)


def plain_rotate(x: torch.Tensor, freqs: torch.Tensor, first: int = 0) -> torch.Tensor:
    """x [T, heads, dim]; the first 2 * len(freqs) dims of every head turn by (first + t) * f_i in pairs (i, i + half)."""
    T = x.shape[0]
    half = freqs.numel()
    ang = (torch.arange(first, first + T, dtype=torch.float64)[:, None] * freqs[None, :]).to(x.dtype)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


# ---------------------------------------------------------------------------------------------- the three mixers
def plain_sink_attention(h, w_q, w_k, w_v, w_o, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                         freqs: torch.Tensor, return_weights: bool = False):
    T = h.shape[0]
    q = plain_rotate((h @ w_q.T).view(T, heads, dim), freqs)
    k = plain_rotate((h @ w_k.T).view(T, kv_heads, dim), freqs)
    v = (h @ w_v.T).view(T, kv_heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    weights = torch.zeros(heads, T, T, dtype=h.dtype)
    share = heads // kv_heads
    for hd in range(heads):
        g = hd // share
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, hd]) * scale
            m = torch.clamp(s.max(), min=0.0)                     # the sink's score is 0
            e = torch.exp(s - m)
            p = e / (torch.exp(-m) + e.sum())
            weights[hd, t, :t + 1] = p
            out[t, hd] = p @ v[:t + 1, g]
    y = out.reshape(T, heads * vdim) @ w_o.T
    return (y, weights) if return_weights else y


def plain_decay_attention(h, w_q, w_k, w_v, w_g, w_o, norm_w, decay, heads: int, dim: int, vdim: int, eps: float):
    T = h.shape[0]
    q = plain_silu(h @ w_q.T).view(T, heads, dim)
    k = plain_silu(h @ w_k.T).view(T, heads, dim)
    v = plain_silu(h @ w_v.T).view(T, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for hd in range(heads):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(T):
            S = float(decay[hd]) * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    o = plain_rms(out.reshape(T, heads * vdim), eps) * norm_w
    return (o * torch.sigmoid(h @ w_g.T)) @ w_o.T


def plain_causal_taps(z: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """z [T, C], w [C, taps]: y_t = sum_j w[:, j] z_(t - taps + 1 + j), zeros before the start."""
    T, taps = z.shape[0], w.shape[1]
    out = torch.zeros_like(z)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * z[s]
    return out


def plain_channel_delta(h, W: dict, heads: int, kv_heads: int, dim: int, vdim: int, eps: float):
    """``W``: the mixer's tensors by their short names (q, q.conv, k, k.conv, v, v.conv, b, A_log, norm, a1, a2,
    dt_bias, g1, g2, o)."""
    T = h.shape[0]
    q = plain_silu(plain_causal_taps(h @ W["q"].T, W["q.conv"])).view(T, kv_heads, dim)
    k = plain_silu(plain_causal_taps(h @ W["k"].T, W["k.conv"])).view(T, kv_heads, dim)
    v = plain_silu(plain_causal_taps(h @ W["v"].T, W["v.conv"])).view(T, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W["b"].T)                                            # [T, heads]
    step = torch.nn.functional.softplus((h @ W["a1"].T) @ W["a2"].T + W["dt_bias"]).view(T, heads, dim)
    g = torch.exp(-torch.exp(W["A_log"])[None, :, None] * step)                   # [T, heads, dim]
    gate = torch.sigmoid((h @ W["g1"].T) @ W["g2"].T).view(T, heads, vdim)
    share = heads // kv_heads
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for hd in range(heads):
        c = hd // share
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(T):
            S = g[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, c])
            S = S + torch.outer(k[t, c], u)
            out[t, hd] = S.T @ q[t, c]
    o = plain_rms(out, eps) * W["norm"] * gate
    return o.reshape(T, heads * vdim) @ W["o"].T


# ---------------------------------------------------------------------------------------------- feed-forward
def plain_route(h, w_router, top: int, groups: int, keep: int, scale: float):
    """(expert ids [T, top], weights [T, top]) of every row."""
    s = torch.sigmoid(h @ w_router.T)                                             # [T, E]
    T, E = s.shape
    per = E // groups
    ids, ws = [], []
    for t in range(T):
        gs = [s[t, g * per:(g + 1) * per].topk(min(2, per)).values.sum() for g in range(groups)]
        best = sorted(range(groups), key=lambda g: (-float(gs[g]), g))[:keep]
        allowed = [e for g in best for e in range(g * per, (g + 1) * per)]
        chosen = sorted(allowed, key=lambda e: (-float(s[t, e]), e))[:top]
        w = torch.stack([s[t, e] for e in chosen])
        ids.append(chosen)
        ws.append(w / (w.sum() + 1e-20) * scale)
    return ids, torch.stack(ws)


def plain_moe(h, W: dict, experts: int, top: int, groups: int, keep: int, scale: float):
    ids, ws = plain_route(h, W["router"], top, groups, keep, scale)
    out = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], ws[t]):
            z = plain_silu(W[f"e{e}.gate"] @ h[t]) * (W[f"e{e}.up"] @ h[t])
            out[t] += w * (W[f"e{e}.down"] @ z)
    return out


# ---------------------------------------------------------------------------------------------- the model
def _sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def plain_mixer(h, layer: dict, W: dict, eps: float):
    kind, m = layer["type"], layer["mixer"]
    if kind == "channel_delta":
        return plain_channel_delta(h, W, m["heads"], m["kv_heads"], m["dim"], m["vdim"], eps)
    if kind == "parallel":
        L, R = m["left"], m["right"]
        rot = L.get("rot") or {}
        freqs = plain_rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot.get("dims") else torch.zeros(0, dtype=torch.float64)
        a = plain_sink_attention(h, W["left.q"], W["left.k"], W["left.v"], W["left.o"], L["heads"], L["kv_heads"], L["dim"],
                                 L["vdim"], L["scale"], freqs)
        b = plain_decay_attention(h, W["right.q"], W["right.k"], W["right.v"], W["right.g"], W["right.o"], W["right.norm"],
                                  R["decay"], R["heads"], R["dim"], R["vdim"], eps)
        return 0.5 * (plain_rms(a, eps) * W["left.out"] + plain_rms(b, eps) * W["right.out"])
    raise ValueError(f"unknown layer type {kind!r}")


def plain_forward(cfg: dict, weights: dict, ids, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    big = cfg["embedding"].get("bigram")
    if big is not None:
        x = plain_embedding(ids, weights["embed"], weights["bigram"], cfg["embedding"]["scale"], big["buckets"], big["mul_prev"],
                            big["mul_cur"])
    else:
        x = weights["embed"][torch.as_tensor(ids, dtype=torch.long)] * cfg["embedding"]["scale"]
    streams = []

    def norm(name, z):
        return plain_dyt(z, weights[name], weights[name + ".b"], weights[name + ".alpha"])

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = plain_mixer(norm(p + "norm1", x), layer, _sub(weights, p + "mix."), eps)
        x = x + m * norm(p + "norm1b", y)
        if layer.get("mlp") is not None:
            r = layer["mlp"]["router"]
            groups = r.get("groups") or {"count": 1, "keep": 1}
            y = plain_moe(norm(p + "norm2", x), _sub(weights, p + "mlp."), r["experts"], r["top"], groups["count"],
                          groups["keep"], r.get("scale", 1.0))
            x = x + m * norm(p + "norm2b", y)
        streams.append(x)
    logits = norm("final.norm", x) @ weights["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
