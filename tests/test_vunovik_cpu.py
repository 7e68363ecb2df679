"""The Vunovik design without a GPU: its configuration, the plain implementation against independent statements of
the same mechanisms, and the package's host logic (cache, state, step function, generation loop) driven on the CPU
through the plain PyTorch stand-ins of the kernels."""
import copy

import pytest
import torch

import cima_b200
from cima_b200.config import ConfigError, VunovikConfig, lookup_architecture
from cima_b200.engine import StepEntry, build_plan
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole
from vunovik_cases import CONFIGS, TOL, V_A, V_B, cpu_model, plain_weights, row_errors
from vunovik_plain import (plain_canon, plain_depth_average, plain_forward, plain_latent, plain_latent_attention,
                           plain_latent_attention_one)


# ------------------------------------------------------------------------------------------- configuration
def test_configuration_round_trip_and_plan():
    entry = lookup_architecture(V_B)
    cfg = entry.parse(V_B)
    assert isinstance(cfg, VunovikConfig) and cfg.to_dict() == V_B
    spec = entry.spec(cfg)
    assert spec.stream == "depth_average" and spec.tie_head and spec.embed_scale == 3.0
    assert [b.mixer.cache_from for b in spec.layers] == [None, 0, 0, None]
    plan = build_plan(spec)
    assert plan["l0.mix.dkv"].shape == (24, 72) and "l1.mix.dkv" not in plan and "l1.mix.dkv.norm" not in plan
    assert plan["l3.mix.uv"].shape == (5 * 24, 48) and plan["l3.mix.uk"].shape == (5 * 8, 48)
    assert plan["l2.dwa"].shape == (4,) and plan["l0.canon1"].shape == (72, 4)
    assert "l2.mlp.gate" not in plan and plan["l1.mlp.down"].shape == (72, 96)
    assert "embed" in plan and "final.norm" in plan and len(plan) == 2 + 4 * 3 + 4 * 4 + 2 * 2 + 3 * 3


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=16), "kv_rank"),
    (lambda c: c["layers"][0].update(type="attention"), "latent_attention"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "dense"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c["canon"].pop("taps"), "taps"),
    (lambda c: c.update(width=0), "width"),
    (lambda c: c["layers"][2]["mixer"].pop("scale"), "scale"),
])
def test_configuration_refuses(change, word):
    cfg = copy.deepcopy(V_A)
    change(cfg)
    with pytest.raises(ConfigError, match=word):
        VunovikConfig.from_dict(cfg)


# ------------------------------------------------------------------------------------------- the plain side
def test_plain_attention_row_by_row_and_moved_into_the_latents_space():
    torch.manual_seed(0)
    T, W, H, D, Dv, R = 9, 12, 3, 4, 5, 6
    u, c = torch.randn(T, W, dtype=torch.float64), torch.randn(T, R, dtype=torch.float64)
    wq, wuk, wuv, wo = (torch.randn(*s, dtype=torch.float64) for s in ((H * D, W), (H * D, R), (H * Dv, R), (W, H * Dv)))
    whole = plain_latent_attention(u, c, wq, wuk, wuv, wo, H, D, Dv, 0.7)
    for t in range(T):
        one = plain_latent_attention_one(u[t], c[:t + 1], wq, wuk, wuv, wo, H, D, Dv, 0.7)
        assert torch.allclose(whole[t], one, atol=1e-12)
    # q.(Wuk c) = (Wuk^T q).c and sum p (Wuv c) = Wuv (sum p c)
    q = (u @ wq.T).view(T, H, D)
    for h in range(H):
        qa = q[:, h] @ wuk[h * D:(h + 1) * D]                          # [T, R]
        s = (qa @ c.T) * 0.7
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        ol = torch.softmax(s, 1) @ c
        a = ol @ wuv[h * Dv:(h + 1) * Dv].T
        k, v = c @ wuk[h * D:(h + 1) * D].T, c @ wuv[h * Dv:(h + 1) * Dv].T
        s2 = ((q[:, h] @ k.T) * 0.7).masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        assert torch.allclose(a, torch.softmax(s2, 1) @ v, atol=1e-12)


def test_plain_convolution_is_a_causal_filter_with_the_input_added():
    torch.manual_seed(1)
    h, w = torch.randn(7, 5, dtype=torch.float64), torch.randn(5, 3, dtype=torch.float64)
    u = plain_canon(h, w)
    padded = torch.cat([torch.zeros(2, 5, dtype=torch.float64), h])
    conv = torch.nn.functional.conv1d(padded.T[None], w[:, None, :], groups=5)[0].T
    assert torch.allclose(u, h + conv, atol=1e-12)
    assert torch.allclose(plain_canon(h, torch.randn(5, 1, dtype=torch.float64) * 0 + 2.0), 3.0 * h)      # one tap: no past


def test_plain_depth_average_and_latent():
    X = [torch.full((2, 3), float(j + 1), dtype=torch.float64) for j in range(3)]
    assert torch.allclose(plain_depth_average(X, torch.tensor([0.5, 0.25, 2.0], dtype=torch.float64)),
                          torch.full((2, 3), 0.5 + 0.5 + 6.0, dtype=torch.float64))
    u, wd, g = torch.randn(4, 6, dtype=torch.float64), torch.randn(3, 6, dtype=torch.float64), torch.tensor([1.0, 2.0, 0.5], dtype=torch.float64)
    c = plain_latent(u, wd, g, 1e-6)
    r = u @ wd.T
    assert torch.allclose(c / g, r / r.pow(2).mean(1, keepdim=True).add(1e-6).sqrt())


# ------------------------------------------------------------------------------------------- the host logic
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_every_cutting_matches_the_plain_model(name):
    cfg, W = plain_weights(name)
    toks = random_tokens(cfg["vocab"], 75, seed=11)
    want, _ = plain_forward(cfg, W, toks)
    m = cpu_model(name)
    assert row_errors(run_whole(m, toks), want).max() < TOL["float32"]
    assert row_errors(run_tail_one_by_one(m, toks, 70), want).max() < TOL["float32"]
    (got,) = run_in_pieces(m, [toks], [[2, 4, 5, 36, 64, 66]])
    assert row_errors(got, want).max() < TOL["float32"]
    m.cache.check()
    assert m.cache.slots.held == 0


def test_unequal_batches_on_reused_slots_and_pages():
    cfg, W = plain_weights("B")
    m = cpu_model("B", max_tokens=64 * 6, max_seqs=3)
    for rnd in range(3):
        lens = [[5, 1, 70], [66, 3, 9], [1, 1, 64]][rnd]
        seqs = [random_tokens(cfg["vocab"], n + 6, seed=10 * rnd + i) for i, n in enumerate(lens)]
        got = run_batched(m, seqs, lens)
        for q, g in zip(seqs, got):
            assert row_errors(g, plain_forward(cfg, W, q)[0]).max() < TOL["float32"], (rnd, len(q))
        m.cache.check()
        assert m.cache.slots.held == 0


def test_bfloat16_plumbing():
    cfg, W = plain_weights("A")
    toks = random_tokens(cfg["vocab"], 40, seed=2)
    got = run_tail_one_by_one(cpu_model("A", "bfloat16"), toks, 8)
    assert row_errors(got, plain_forward(cfg, W, toks)[0]).max() < TOL["bfloat16"]


def test_greedy_generation_through_the_entry_point():
    cfg, W = plain_weights("A")
    lm = cima_b200.LM(cpu_model("A"), pipeline=False)
    prompts = [random_tokens(cfg["vocab"], n, seed=n) for n in (3, 17, 1)]
    got = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=6)
    for p, r in zip(prompts, got):
        seq = list(p)
        for t in r.tokens:
            lg = plain_forward(cfg, W, seq)[0][-1]
            assert lg[t] >= lg.max() - 1e-5
            seq.append(t)
        assert len(r.tokens) == 6
    assert lm.model.cache.slots.held == 0


def test_state_dict_gives_the_checkpoint_back():
    cfg, W = plain_weights("B")
    sd = cpu_model("B").state_dict()
    assert sorted(sd) == sorted(W)
    for n, t in W.items():
        assert torch.equal(sd[n].float().cpu(), t.float()), n
