"""The Gisirax design without a GPU: its configuration, the plain implementation against independent statements of the
same mechanisms, and the package's host logic (cache, state, step function, generation loop) driven on the CPU through
the plain PyTorch stand-ins of the kernels."""
import copy
import math

import pytest
import torch

import cima_b200
from cima_b200.config import ConfigError, GisiraxConfig, lookup_architecture
from cima_b200.engine import build_plan
from gisirax_cases import CONFIGS, G_A, G_B, cpu_model, folder, plain_weights, row_errors
from gisirax_plain import (plain_causal_taps, plain_channel_delta, plain_decay_attention, plain_forward, plain_rms,
                           plain_rotary_frequencies, plain_rotate, plain_route, plain_silu, plain_sink_attention)
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole

TOL = 3e-5


# ------------------------------------------------------------------------------------------- configuration
def test_configuration_round_trip_and_plan():
    entry = lookup_architecture(G_A)
    cfg = entry.parse(G_A)
    assert isinstance(cfg, GisiraxConfig) and GisiraxConfig.from_dict(cfg.to_dict()) == cfg
    spec = entry.spec(cfg)
    assert not spec.tie_head and spec.embed_scale == 2.0 and spec.embed_bigram.buckets == 61
    assert [b.kind for b in spec.layers] == ["sandwich"] * 4 and spec.layers[1].feed_forward is None
    assert [b.mixer.kind for b in spec.layers] == ["channel_delta", "side_by_side", "side_by_side", "channel_delta"]
    plan = build_plan(spec)
    assert plan["bigram"].shape == (62, 96) and plan["head"].shape == (300, 96) and plan["l0.norm1.alpha"].shape == ()
    assert plan["l0.mix.q"].shape == (32, 96) and plan["l0.mix.v"].shape == (96, 96) and plan["l0.mix.k.conv"].shape == (32, 3)
    assert plan["l0.mix.a1"].shape == (8, 96) and plan["l0.mix.a2"].shape == (64, 8) and plan["l0.mix.g2"].shape == (96, 12)
    assert plan["l0.mix.norm"].shape == (24,) and plan["l0.mix.b"].shape == (4, 96) and plan["l0.mix.dt_bias"].shape == (64,)
    assert plan["l1.mix.left.q"].shape == (128, 96) and plan["l1.mix.left.k"].shape == (32, 96)
    assert plan["l1.mix.left.v"].shape == (16, 96) and plan["l1.mix.left.o"].shape == (96, 64)
    assert plan["l1.mix.right.g"].shape == (80, 96) and plan["l1.mix.right.norm"].shape == (80,) and plan["l1.mix.left.out"].shape == (96,)
    assert "l1.norm2" not in plan and "l1.mlp.router" not in plan and plan["l2.mlp.e5.down"].shape == (96, 24)
    assert plan["l3.mlp.router"].shape == (4, 96)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="attention"), "channel_delta"),
    (lambda c: c["layers"][0]["mixer"].pop("a_rank"), "a_rank"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"]["scaling"].update(high=1.0), "scaling"),
    (lambda c: c["layers"][1]["mixer"].pop("left"), "left"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "router"),
    (lambda c: c["layers"][2]["mlp"]["router"]["groups"].update(count=4), "router"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
])
def test_configuration_refuses(change, word):
    cfg = copy.deepcopy(G_A)
    change(cfg)
    with pytest.raises(ConfigError, match=word):
        GisiraxConfig.from_dict(cfg)


def test_ranks_come_from_the_stored_shapes_where_the_configuration_is_silent():
    from cima_b200.weights.loader import tensor_shapes
    d = folder("A", drop_ranks=True)
    raw = cima_b200.read_config_json(d)
    assert "a_rank" not in raw["layers"][0]["mixer"]
    cfg = GisiraxConfig.from_dict(raw, tensor_shapes(d))
    assert (cfg.layers[0].delta.a_rank, cfg.layers[0].delta.g_rank, cfg.layers[3].delta.a_rank) == (8, 12, 16)


# ------------------------------------------------------------------------------------------- the plain side
def test_plain_sink_attention_against_a_softmax_with_one_more_key():
    """A sink is a key of score 0 whose value is zero: the ordinary softmax over the keys and that one."""
    torch.manual_seed(0)
    T, W, H, G, D, Dv = 7, 10, 4, 2, 6, 3
    h = torch.randn(T, W, dtype=torch.float64)
    wq, wk, wv, wo = (torch.randn(*s, dtype=torch.float64) for s in ((H * D, W), (G * D, W), (G * Dv, W), (W, H * Dv)))
    fr = plain_rotary_frequencies(4, 100.0)
    got = plain_sink_attention(h, wq, wk, wv, wo, H, G, D, Dv, 0.4, fr)
    q = plain_rotate((h @ wq.T).view(T, H, D), fr)
    k = plain_rotate((h @ wk.T).view(T, G, D), fr)
    v = (h @ wv.T).view(T, G, Dv)
    out = torch.zeros(T, H, Dv, dtype=torch.float64)
    for t in range(T):
        for hd in range(H):
            s = torch.cat([(k[:t + 1, hd // 2] @ q[t, hd]) * 0.4, torch.zeros(1, dtype=torch.float64)])
            p = torch.softmax(s, dim=0)
            out[t, hd] = p[:-1] @ v[:t + 1, hd // 2]
    assert torch.allclose(got, out.view(T, -1) @ wo.T, atol=1e-12)


def test_plain_rotation_depends_on_the_distance_only_and_leaves_the_rest():
    fr = plain_rotary_frequencies(8, 50.0, {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 20})
    torch.manual_seed(1)
    x, y = torch.randn(1, 1, 12, dtype=torch.float64), torch.randn(1, 1, 12, dtype=torch.float64)
    dots = [float((plain_rotate(x, fr, first=a)[0, 0, :8] * plain_rotate(y, fr, first=a + 3)[0, 0, :8]).sum()) for a in (0, 5, 40)]
    assert max(dots) - min(dots) < 1e-9
    assert torch.equal(plain_rotate(x, fr, first=9)[..., 8:], x[..., 8:])
    plain = plain_rotary_frequencies(8, 50.0)
    assert fr[0] == plain[0] and math.isclose(float(fr[-1]), float(plain[-1]) / 4.0) and plain[1] / 4.0 < fr[1] < plain[1]


def test_plain_decay_attention_as_a_weighted_sum_over_the_past():
    """o_t = sum_(s <= t) d^(t - s) (q_t . k_s) v_s: the recurrence unrolled."""
    torch.manual_seed(2)
    T, W, H, D, Dv = 6, 8, 2, 3, 4
    h = torch.randn(T, W, dtype=torch.float64)
    wq, wk, wv, wg, wo = (torch.randn(*s, dtype=torch.float64) for s in ((H * D, W), (H * D, W), (H * Dv, W), (H * Dv, W), (W, H * Dv)))
    nw, decay = torch.randn(H * Dv, dtype=torch.float64), [0.5, 0.9]
    got = plain_decay_attention(h, wq, wk, wv, wg, wo, nw, decay, H, D, Dv, 1e-5)
    q, k, v = (plain_silu(h @ w.T).view(T, H, -1) for w in (wq, wk, wv))
    o = torch.zeros(T, H, Dv, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            for hd in range(H):
                o[t, hd] += decay[hd] ** (t - s) * (q[t, hd] @ k[s, hd]) * v[s, hd]
    want = (plain_rms(o.view(T, -1), 1e-5) * nw * torch.sigmoid(h @ wg.T)) @ wo.T
    assert torch.allclose(got, want, atol=1e-12)


def test_plain_delta_rule_writes_what_it_then_reads():
    """With beta = 1 and no decay, reading the state with the key just written returns that token's value."""
    torch.manual_seed(3)
    T, W, H, D, Dv = 5, 8, 1, 4, 3
    Wt = {"q": torch.randn(D, W), "k": torch.randn(D, W), "v": torch.randn(Dv, W), "q.conv": torch.zeros(D, 2), "k.conv": torch.zeros(D, 2),
          "v.conv": torch.zeros(Dv, 2), "b": torch.zeros(H, W), "A_log": torch.zeros(H), "norm": torch.ones(Dv), "a1": torch.zeros(2, W),
          "a2": torch.zeros(D, 2), "dt_bias": torch.full((D,), -60.0), "g1": torch.zeros(2, W), "g2": torch.zeros(Dv, 2), "o": torch.eye(Dv)}
    for k in ("q.conv", "k.conv", "v.conv"):
        Wt[k][:, -1] = 1.0                                             # the convolution passes the current token on
    Wt["q"] = Wt["k"].clone()                                          # the query is the key
    Wt = {k: v.double() for k, v in Wt.items()}
    Wt["b"] = Wt["b"] + 0.0
    h = torch.randn(T, W, dtype=torch.float64)
    # beta = sigmoid(0) = 1/2: u = (v - S^T k) / 2, so the read-out moves half of the way from the old answer to v
    got = plain_channel_delta(h, Wt, H, H, D, Dv, 1e-12)
    v0 = plain_silu(h[0] @ Wt["v"].T)
    first = 0.5 * v0 * D ** -0.5                                       # S was zero; q = k / |k| * D^-1/2, k . k / |k|^2 = 1
    want0 = first / torch.sqrt((first * first).mean() + 1e-12) * 0.5   # the norm, then sigmoid(0) of the gate
    assert torch.allclose(got[0], want0, atol=1e-6)


def test_plain_causal_taps_against_conv1d():
    torch.manual_seed(4)
    z, w = torch.randn(9, 5, dtype=torch.float64), torch.randn(5, 3, dtype=torch.float64)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(z.T[None], (2, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(plain_causal_taps(z, w), want, atol=1e-12)


def test_plain_route_keeps_to_the_best_groups():
    torch.manual_seed(5)
    h, wr = torch.randn(40, 16, dtype=torch.float64), torch.randn(15, 16, dtype=torch.float64)
    ids, ws = plain_route(h, wr, top=4, groups=5, keep=2, scale=1.25)
    s = torch.sigmoid(h @ wr.T)
    for t in range(40):
        groups = sorted({e // 3 for e in ids[t]})
        score = [s[t, g * 3:(g + 1) * 3].topk(2).values.sum() for g in range(5)]
        assert len(groups) <= 2 and set(groups) <= set(sorted(range(5), key=lambda g: -score[g])[:2])
        assert math.isclose(float(ws[t].sum()), 1.25, rel_tol=1e-9) and len(set(ids[t])) == 4
    free, _ = plain_route(h, wr, top=4, groups=1, keep=1, scale=1.0)
    assert all(sorted(free[t]) == sorted(s[t].topk(4).indices.tolist()) for t in range(40))


# ------------------------------------------------------------------------------------------- host logic on the stand-ins
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_on_the_cpu(name):
    cfg, W = plain_weights(name)
    toks, other = random_tokens(cfg["vocab"], 80, seed=3), random_tokens(cfg["vocab"], 70, seed=4)
    want, want2 = plain_forward(cfg, W, toks), plain_forward(cfg, W, other)
    m = cpu_model(name)
    assert row_errors(run_whole(m, toks), want).max() < TOL
    assert row_errors(run_tail_one_by_one(m, toks, 20), want).max() < TOL
    got = run_in_pieces(m, [toks, other], [[2, 4, 7, 64, 66], [63, 65]])
    assert row_errors(got[0], want).max() < TOL and row_errors(got[1], want2).max() < TOL
    got = run_batched(m, [toks, other[:9], other], [70, 3, 64])
    assert row_errors(got[0], want).max() < TOL and row_errors(got[1], want2[:9]).max() < TOL and row_errors(got[2], want2).max() < TOL
    m.cache.check()
    assert m.cache.slots.held == 0


def test_reused_slots_start_from_nothing():
    """A slot that held a sequence is handed to the next one with its recurrent state, the convolution's inputs and
    the last token zeroed."""
    cfg, W = plain_weights("A")
    m = cpu_model("A", max_tokens=128, max_seqs=1)
    for seed in (1, 2, 3):
        toks = random_tokens(cfg["vocab"], 30, seed=seed)
        assert row_errors(run_tail_one_by_one(m, toks, 10), plain_forward(cfg, W, toks)).max() < TOL
    assert m.cache.has_mixer_state


def test_greedy_generation_on_the_cpu():
    from cima_b200 import LM
    cfg, W = plain_weights("B")
    lm = LM(cpu_model("B"), [], max_batch=4, pipeline=False, use_graphs=False)
    prompts = [random_tokens(cfg["vocab"], n, seed=20 + n) for n in (5, 1, 12)]
    got = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=6)
    for p, r in zip(prompts, got):
        seq = list(p)
        for t in r.tokens:
            lg = plain_forward(cfg, W, seq)[-1]
            assert lg[t] >= lg.max() - 1e-4
            seq.append(t)


def test_tensors_by_name_round_trip():
    m = cpu_model("A")
    sd = m.state_dict()
    cfg, W = plain_weights("A")
    assert set(sd) == set(W)
    for n, t in W.items():
        assert torch.allclose(sd[n].double().reshape(t.shape), t, atol=0, rtol=0), n
