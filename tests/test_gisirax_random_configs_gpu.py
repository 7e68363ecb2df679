"""Gisirax configurations drawn at random (every size and constant that config.json gives, layer by layer, in any order
of the two layer kinds) in cuttings drawn at random too (whole, a tail one by one, pieces, unequal batches): in 32-bit
against the plain implementation on weights that make attention sharp, and in bfloat16 against the 32-bit engine on
milder weights of the same configuration."""
import os
import random

import pytest
import torch
from safetensors.torch import load_file, save_file

import cima_b200
from cima_b200.engine import load_model
from gisirax_cases import _boost, config, delta, moe, parallel, rot, row_errors
from gisirax_plain import plain_forward, read_folder
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole

pytestmark = pytest.mark.gpu

SEEDS = list(range(int(os.environ.get("CIMA_RANDOM_CONFIGS", "6"))))


def draw_moe(rng: random.Random):
    if rng.random() < 0.2:
        return None
    groups = rng.choice([1, 1, 2, 3, 4, 6])
    per = rng.choice([1, 2, 3, 4])
    keep = rng.randint(1, groups)
    top = rng.randint(1, min(keep * per, 6))
    return moe(rng.choice([8, 20, 33, 64, 96, 130]), groups * per, top, rng.choice([0.5, 1.0, 1.5, 2.5]),
               groups=groups if (groups > 1 or rng.random() < 0.5) else None, keep=keep)


def draw_config(rng: random.Random) -> dict:
    width = rng.choice([64, 72, 100, 128, 136, 192, 256, 320])                  # some are no multiple of 8
    layers = []
    for _ in range(rng.randint(1, 5)):
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            heads = kv * rng.choice([1, 2, 4])
            dim = rng.choice([8, 16, 24, 32, 48, 64, 80, 128])
            rotary = None
            if rng.random() < 0.85:
                dims = rng.choice([d for d in (4, 8, 16, 32, 64, 128, dim, dim) if d <= dim])      # a part of the head, or all of it
                sc = (rng.choice([2.0, 4.0, 8.0]), rng.choice([0.5, 1.0]), rng.choice([2.0, 4.0, 16.0]), rng.choice([16, 64, 512, 4096]))
                rotary = rot(dims, rng.choice([100.0, 10000.0, 500000.0]), sc if rng.random() < 0.7 else None)
            r_heads = rng.randint(1, 5)
            layers.append(parallel(heads, kv, dim, rng.choice([8, 16, 24, 32, 48, 64, 96]), rng.choice([0.05, 0.125, 0.25]), rotary,
                                   r_heads, rng.choice([8, 16, 40, 64, 128]), rng.choice([8, 16, 24, 64, 100]),
                                   [rng.choice([0.3, 0.8, 0.95, 0.99, 0.998]) for _ in range(r_heads)], draw_moe(rng)))
        else:
            kv = rng.choice([1, 2, 3])
            layers.append(delta(kv * rng.choice([1, 2, 3]), kv, rng.choice([8, 16, 24, 40, 64, 128, 160]), rng.choice([8, 16, 24, 48, 64, 100]),
                                rng.randint(1, 5), rng.choice([4, 8, 12, 24]), rng.choice([4, 8, 20]), draw_moe(rng)))
    bigram = (rng.choice([13, 127, 509]), rng.randint(0, 40), rng.randint(1, 40)) if rng.random() < 0.85 else None
    return config(rng.choice([129, 333, 512, 1001]), width, rng.choice([1e-6, 1e-5, 3e-4]), rng.choice([0.5, 0.7, 1.0, 1.4]),
                  rng.choice([0.5, 1.0, 4.0, 12.0]), bigram, layers)


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(seed, tmp_path):
    rng = random.Random(9000 + seed)
    cfg = draw_config(rng)
    folders = {}
    for kind in ("sharp", "mild"):
        folders[kind] = str(tmp_path / kind)
        cima_b200.write_random_model(folders[kind], cfg, seed=seed)
        path = os.path.join(folders[kind], "model.safetensors")
        save_file({n: _boost(n, t, sharp=kind == "sharp").contiguous() for n, t in load_file(path).items()}, path)
    c, W = read_folder(folders["sharp"])
    n = rng.choice([40, 130, 200])
    toks = random_tokens(cfg["vocab"], n, seed)
    want = plain_forward(c, W, toks)
    cuts = sorted(rng.sample(range(1, n), 3))
    lens = [n, rng.randint(1, n), rng.randint(1, n)]
    starts = [rng.randint(1, l) for l in lens]
    others = [random_tokens(cfg["vocab"], l, seed + 100 + i) for i, l in enumerate(lens[1:])]
    exact = {}
    tail = min(n - 1, rng.randint(1, 70))
    for kind, dtype in (("sharp", "float32"), ("mild", "float32"), ("mild", "bfloat16")):
        m = load_model(folders[kind], dtype=dtype, max_tokens=2048, device="cuda:0", verbose=False)
        runs = {"whole": run_whole(m, toks), "tail": run_tail_one_by_one(m, toks, tail),
                "pieces": run_in_pieces(m, [toks], [cuts])[0], "batch": run_batched(m, [toks] + others, starts)[0]}
        for what, got in runs.items():
            if kind == "sharp":
                e = row_errors(got, want)
                assert e.max() < 2e-4, (cfg, what, float(e.max()))      # sums of float32 through sharp softmaxes; a fault shows at 1e-2
            elif dtype == "float32":
                exact[what] = got
            else:
                e = row_errors(got, exact[what])
                assert torch.isfinite(got).all() and e.median() < 4e-2, (cfg, what, float(e.median()), float(e.max()))
        m.cache.check()
        assert m.cache.slots.held == 0
        del m
        torch.cuda.empty_cache()
