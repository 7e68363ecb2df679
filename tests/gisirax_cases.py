"""Small Gisirax configurations, their weights and helpers shared by the tests of that design.

The weights are drawn by ``cima_b200.write_random_model`` and then scaled by tensor name, so that activations are of
order one, attention scores spread over tens (single keys then carry rows, near or far), decays range from fast to
slow and the router's scores lie apart."""
from __future__ import annotations

import json
import os
import tempfile

import torch

import cima_b200
from cima_b200.engine import load_model


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def parallel(heads, kv_heads, dim, vdim, scale, rotary, r_heads, r_dim, r_vdim, decay, mlp):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rotary is not None:
        left["rot"] = rotary
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": decay}},
            "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv, a_rank, g_rank, mlp):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "a_rank": a_rank, "g_rank": g_rank}, "mlp": mlp}


def moe(ff, experts, top, scale, groups=None, keep=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def config(vocab, width, eps, mult, embed_scale, bigram, layers):
    emb = {"scale": embed_scale}
    if bigram is not None:
        emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    return {"architecture": "Gisirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": emb, "layers": layers}


# value size below and above the key size, a partial rotation with rescaled frequencies, grouped heads down to one
# key head, a layer without feed-forward, three and two taps, groups of experts of which one stays
G_A = config(300, 96, 1e-6, 1.3, 2.0, (61, 5, 3), [
    delta(4, 2, 16, 24, 3, 8, 12, moe(40, 8, 2, 2.0, groups=2, keep=1)),
    parallel(4, 1, 32, 16, 0.18, rot(16, 10000.0, (8.0, 1.0, 4.0, 64)), 2, 16, 40, [0.5, 0.97], None),
    parallel(2, 2, 16, 48, 0.25, rot(16, 500.0), 3, 24, 8, [0.9, 0.99, 0.7], moe(24, 6, 3, 1.0, groups=3, keep=2)),
    delta(2, 1, 40, 8, 2, 16, 4, moe(56, 4, 1, 0.5))])
# the layers in another order; one tap (no convolution state); no groups; every expert chosen; no rotation in one layer;
# a width that is no multiple of 8; one head
G_B = config(513, 100, 1e-5, 0.6, 5.0, (127, 29, 5), [
    parallel(3, 3, 16, 16, 0.25, None, 1, 8, 8, [0.8], moe(20, 3, 3, 1.5)),
    delta(1, 1, 24, 24, 1, 4, 4, None),
    delta(3, 3, 8, 16, 4, 24, 8, moe(32, 10, 3, 1.25, groups=5, keep=3))])
# the sizes of the tensor-core attention kernels (heads of 64 and of 128) and a recurrence over 128 key channels
G_C = config(640, 256, 1e-5, 0.85, 1.0, (509, 3, 11), [
    parallel(4, 2, 64, 64, 0.125, rot(64, 200000.0, (3.0, 1.0, 8.0, 1024)), 4, 32, 64, [0.6, 0.9, 0.97, 0.995],
             moe(96, 8, 2, 1.0, groups=4, keep=2)),
    delta(2, 2, 128, 64, 4, 16, 16, moe(64, 4, 2, 2.5, groups=2, keep=2)),
    parallel(2, 1, 128, 128, 0.09, rot(32, 10000.0), 2, 64, 32, [0.95, 0.99], None)])
CONFIGS = {"A": G_A, "B": G_B, "C": G_C}

# factor by the last part of a tensor's name (after the scaling, a matrix of fan-in K has entries of about f * 0.02)
_BOOST = {"embed": 25.0, "bigram": 25.0, "head": 10.0, "router": 2.0, "left.q": 14.0, "left.k": 14.0, "a2": 2.0, "g2": 2.0}
_DEFAULT_BOOST = 5.0


def _boost(name: str, t: torch.Tensor, sharp: bool = True) -> torch.Tensor:
    """``sharp`` False leaves the attention's scores of order one: bfloat16 runs are compared on such weights, since with
    scores of tens the rounding of a query decides which key carries a row."""
    if t.dim() < 2 or name.endswith(".conv"):
        return t
    for key, f in _BOOST.items():
        if name == key or name.endswith("." + key):
            if not sharp and key in ("left.q", "left.k"):
                f = 3.0
            return (t.float() * f).to(t.dtype)
    return (t.float() * _DEFAULT_BOOST).to(t.dtype)


_FOLDERS = {}


def folder(name: str, seed: int = 0, drop_ranks: bool = False) -> str:
    """A model folder of configuration ``name``; ``drop_ranks`` leaves the low-rank sizes out of config.json, so that
    only the stored tensors' shapes give them."""
    key = (name, seed, drop_ranks)
    if key not in _FOLDERS:
        from safetensors.torch import load_file, save_file
        d = tempfile.mkdtemp(prefix=f"cima_gisirax_{name}_")
        cima_b200.write_random_model(d, CONFIGS[name], seed=seed)
        path = os.path.join(d, "model.safetensors")
        save_file({n: _boost(n, t).contiguous() for n, t in load_file(path).items()}, path)
        if drop_ranks:
            with open(os.path.join(d, "config.json")) as f:
                cfg = json.load(f)
            for L in cfg["layers"]:
                L["mixer"].pop("a_rank", None)
                L["mixer"].pop("g_rank", None)
            with open(os.path.join(d, "config.json"), "w") as f:
                json.dump(cfg, f)
        _FOLDERS[key] = d
    return _FOLDERS[key]


def plain_weights(name: str, seed: int = 0):
    """(config dict, tensors in float64) of a folder, read without the package."""
    from gisirax_plain import read_folder
    return read_folder(folder(name, seed))


def cpu_model(name, dtype="float32", max_tokens=1024, seed=0, **kw):
    from reference_kernels import ReferenceKernels
    return load_model(folder(name, seed), dtype=dtype, max_tokens=max_tokens, device="cpu", kernels=ReferenceKernels(),
                      verbose=False, **kw)


def gpu_model(name, dtype="float32", max_tokens=1024, seed=0, **kw):
    return load_model(folder(name, seed), dtype=dtype, max_tokens=max_tokens, device="cuda:0", verbose=False, **kw)


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference (its mean taken off) over that of the wanted row."""
    d = got.double() - want.double()
    d = d - d.mean(dim=1, keepdim=True)
    w = want.double() - want.double().mean(dim=1, keepdim=True)
    return d.pow(2).mean(dim=1).sqrt() / w.pow(2).mean(dim=1).sqrt().clamp_min(1e-30)
