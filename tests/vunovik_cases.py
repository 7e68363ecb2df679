"""Small Vunovik configurations and helpers shared by the tests of that design."""
from __future__ import annotations

import json
import os
import tempfile

import torch

import cima_b200
from cima_b200.engine import load_model


def layer(heads, dim, vdim, rank, scale, ff, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(vocab, width, taps, embed_scale, eps, layers):
    return {"architecture": "Vunovik", "vocab": vocab, "width": width, "canon": {"taps": taps},
            "embedding": {"scale": embed_scale}, "norm": {"eps": eps}, "layers": layers}


# sizes that differ from layer to layer; a layer without feed-forward; one head; values wider than keys
V_A = config(300, 96, 2, 1.0, 1e-6, [layer(2, 16, 16, 32, 0.25, 128), layer(3, 32, 8, 32, 0.5, 0, kv_from=0),
                                     layer(1, 24, 40, 16, 1.0, 64)])
# a latent whose size no fast kernel takes, two layers that read one layer's latents, four taps, a scaled embedding
V_B = config(513, 72, 4, 3.0, 1e-5, [layer(2, 8, 8, 24, 0.35, 40), layer(4, 16, 8, 24, 0.2, 96, kv_from=0),
                                     layer(2, 8, 16, 24, 0.3, 0, kv_from=0), layer(5, 8, 24, 48, 0.4, 56)])
# the sizes of the tensor-core kernels: latents of 128 and of 64 values
V_C = config(640, 256, 3, 0.5, 1e-5, [layer(4, 64, 64, 128, 0.125, 512), layer(8, 32, 48, 128, 0.2, 384, kv_from=0),
                                      layer(4, 48, 32, 64, 0.15, 256)])
# no convolution state at all (one tap), a width that is no multiple of 8, odd sizes everywhere
V_D = config(101, 100, 1, 2.0, 1e-6, [layer(3, 10, 6, 20, 0.3, 50), layer(2, 14, 22, 20, 0.25, 30, kv_from=0)])
# sharp attention: a large score factor makes single keys carry a row, wherever they stand
V_SHARP = config(257, 128, 3, 1.0, 1e-6, [layer(4, 32, 32, 64, 6.0, 192), layer(2, 64, 16, 64, 4.0, 0, kv_from=0),
                                          layer(4, 16, 16, 32, 8.0, 128)])
CONFIGS = {"A": V_A, "B": V_B, "C": V_C, "D": V_D, "SHARP": V_SHARP}

_FOLDERS = {}


def folder(name: str, seed: int = 0) -> str:
    key = (name, seed)
    if key not in _FOLDERS:
        d = tempfile.mkdtemp(prefix=f"cima_vunovik_{name}_")
        cima_b200.write_random_model(d, CONFIGS[name], seed=seed)
        _FOLDERS[key] = d
    return _FOLDERS[key]


def plain_weights(name: str, seed: int = 0):
    """(config dict, tensors) of a folder, read without the package: json and the safetensors package."""
    from safetensors.torch import load_file
    d = folder(name, seed)
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(d, "model.safetensors"))


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


# float32: sums of a few hundred float32 terms through a few layers.  bfloat16: activations rounded to 8 bits several
# times a layer; sharp attention multiplies the rounding of a score by the score factor.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}
