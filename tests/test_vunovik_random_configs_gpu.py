"""Vunovik configurations drawn at random (every size and constant that config.json gives, layer by layer) against
the plain implementation, in both precisions and in cuttings drawn at random too: whole, a tail one by one, pieces,
unequal batches; and generation through the entry point, greedy and sampled, against the plain loop."""
import json
import os
import random

import pytest
import torch
from safetensors.torch import load_file

import cima_b200
from cima_b200.engine import load_model
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole
from vunovik_cases import config, layer, row_errors
from vunovik_plain import plain_forward

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 4e-2}
SEEDS = list(range(int(os.environ.get("CIMA_RANDOM_CONFIGS", "8"))))


def draw_config(rng: random.Random) -> dict:
    width = rng.choice([64, 72, 100, 128, 136, 192, 256, 320, 384])           # some are no multiple of 8
    n = rng.randint(1, 5)
    layers, owners = [], []
    for i in range(n):
        src = rng.choice(owners) if owners and rng.random() < 0.45 else None
        rank = layers[src]["mixer"]["kv_rank"] if src is not None else rng.choice([8, 16, 24, 32, 48, 64, 80, 96, 128, 144])
        ff = 0 if rng.random() < 0.2 else rng.choice([48, 99, 128, 130, 264, 328])
        layers.append(layer(rng.randint(1, 7), rng.choice([8, 12, 16, 24, 32, 40, 64, 96]), rng.choice([8, 10, 16, 24, 48, 64, 80]),
                            rank, rng.choice([0.08, 0.125, 0.25, 0.5, 1.0]), ff, kv_from=src))
        if src is None:
            owners.append(i)
    return config(rng.choice([129, 333, 512, 640, 1001]), width, rng.randint(1, 5), rng.choice([0.5, 1.0, 2.5, 12.0]),
                  rng.choice([1e-6, 1e-5, 3e-4]), layers)


def plain_of(folder):
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f), load_file(os.path.join(folder, "model.safetensors"))


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(seed, tmp_path):
    rng = random.Random(7000 + seed)
    cfg = draw_config(rng)
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=seed)
    c, W = plain_of(folder)
    n = rng.choice([40, 130, 300])
    toks = random_tokens(cfg["vocab"], n, seed)
    want = plain_forward(c, W, toks)[0]
    cuts = sorted(rng.sample(range(1, n), 3))
    lens = [n, rng.randint(1, n), rng.randint(1, n)]
    starts = [rng.randint(1, l) for l in lens]
    for dtype in ("float32", "bfloat16"):
        m = load_model(folder, dtype=dtype, max_tokens=2048, device="cuda:0", verbose=False)
        tol = TOL[dtype]
        what = (seed, dtype, cfg)
        assert row_errors(run_whole(m, toks), want).max() <= tol, what
        assert row_errors(run_tail_one_by_one(m, toks, min(32, n - 1)), want).max() <= tol, what
        assert row_errors(run_in_pieces(m, [toks], [cuts])[0], want).max() <= tol, (what, cuts)
        for got, l in zip(run_batched(m, [toks[:l] for l in lens], starts), lens):
            assert row_errors(got, want[:l]).max() <= tol, (what, lens, starts)
        m.cache.check()
        assert m.cache.slots.held == 0
        m.check_device()


@pytest.mark.parametrize("seed", SEEDS[:4])
def test_random_configuration_generates_as_the_plain_loop(seed, tmp_path):
    """Through the entry point in 32-bit: several prompts of random lengths, greedy or through the default sampling
    chain, with stop tokens taken from a first run; twice over, so that slots, pages, convolution state and recorded
    steps are used again.  Token for token what the plain loop generates."""
    from qwen2_plain import PlainXorshift, plain_sample
    rng = random.Random(9000 + seed)
    cfg = draw_config(rng)
    folder = str(tmp_path / "m")
    cima_b200.write_random_model(folder, cfg, seed=seed)
    c, W = plain_of(folder)
    prompts = [random_tokens(cfg["vocab"], rng.choice([1, 2, 15, 17, 40, 64, 65, 70, 129]), seed * 100 + i)
               for i in range(rng.choice([1, 2, 5, 9]))]
    opts = rng.choice([dict(temperature=0.0, repeat_penalty=1.0), dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=seed + 1)])
    steps = 5

    def plain_generate(p, stops):
        gen, seq, out = PlainXorshift(opts.get("seed", 0)), list(p), []
        for _ in range(steps):
            t = plain_sample(plain_forward(c, W, seq)[0][-1].float().tolist(), seq, opts, gen)
            if t in stops:
                break
            out.append(t)
            seq.append(t)
        return out

    lm = cima_b200.load(folder, dtype="float32", max_tokens=4096, verbose=False, retain=rng.choice([0, 0, 2]))
    free = [plain_generate(p, ()) for p in prompts]
    what = (seed, cfg, [len(p) for p in prompts], opts)
    assert [r.tokens for r in lm.generate(prompts, max_tokens=steps, **opts)] == free, what
    stops = tuple({free[0][min(2, len(free[0]) - 1)], free[-1][0]})
    want = [plain_generate(p, stops) for p in prompts]
    for _ in range(2):
        got = lm.generate(prompts, max_tokens=steps, stop=stops, **opts)
        assert [r.tokens for r in got] == want, (what, stops)
    lm.stepper.drop_retained()
    lm.model.cache.check()
    assert lm.model.cache.slots.held == 0
    lm.model.check_device()
