"""The Vunovik design on the GPU: each new kernel alone against the plain functions, then the model in every cutting
(whole, token by token, pieces down to two tokens, unequal batches, reused slots and pages, long decoding), in 32-bit
and in bfloat16, on configurations that differ in every size, and generation through the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import cima_b200
from cima_b200.cache.kv import KVCache, KVRequest
from cima_b200.engine import StepEntry
from cima_b200.engine.batch import build_batch
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole
from vunovik_cases import CONFIGS, TOL, folder, gpu_model, plain_weights, row_errors
from vunovik_plain import (plain_canon, plain_depth_average, plain_embed, plain_forward, plain_latent, plain_rmsnorm)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda:0"

_kernels = []


def K():
    if not _kernels:
        from cima_b200.kernels import Kernels
        _kernels.append(Kernels(verbose=False))
    return _kernels[0]


def entries_batch(counts, starts, slots=None):
    slots = slots or list(range(len(counts)))
    return build_batch([StepEntry(s, [0] * c, []) for s, c in zip(slots, counts)], starts, 1, DEV)


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows_per_thread", [0, 2, 8])
@pytest.mark.parametrize("taps,C", [(1, 40), (2, 300), (3, 64), (4, 512), (5, 257)])
def test_short_conv_in_pieces(taps, C, rows_per_thread, dtype):
    """Three sequences fed in three steps (many rows, a few, one each): every piece finds its past in the state."""
    g = torch.Generator().manual_seed(taps * 1000 + C)
    lens = [11, 2, 7]
    w = torch.randn(C, taps, generator=g)
    hs = [torch.randn(n + 4 + 1, C, generator=g).to(DT[dtype]) for n in lens]
    want = [plain_canon(h.double(), w.double()) for h in hs]
    state = torch.zeros(5, max(taps - 1, 1), C, dtype=DT[dtype], device=DEV)[:, :taps - 1]
    slots = [4, 0, 2]
    state[slots] = 7.0                                                     # a slot's state is zeroed when it opens
    state[slots] = 0.0
    got = [[] for _ in lens]
    pos = [0, 0, 0]
    for counts in (lens, [4, 4, 4], [1, 1, 1]):
        b = entries_batch(counts, pos, slots)
        h = torch.cat([hs[i][pos[i]:pos[i] + c] for i, c in enumerate(counts)]).to(DEV)
        out = torch.empty_like(h)
        K().short_conv(h, w.t().contiguous().to(DEV), state if taps > 1 else None, b, out, rows_per_thread)
        r = 0
        for i, c in enumerate(counts):
            got[i].append(out[r:r + c].float().cpu()); r += c; pos[i] += c
    tol = 1e-5 if dtype == "float32" else 3e-2
    for i in range(3):
        assert (torch.cat(got[i]).double() - want[i]).abs().max().item() < tol * (1 + want[i].abs().max().item())
    if taps > 1:                                                          # what the state holds: the newest inputs
        for i, s in enumerate(slots):
            assert torch.equal(state[s].cpu(), hs[i][-(taps - 1):])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,T,H", [(1, 3, 40), (2, 9, 96), (5, 70, 257), (9, 4, 1024)])
def test_depth_average_with_and_without_the_norm(n, T, H, dtype):
    g = torch.Generator().manual_seed(n)
    stack = torch.randn(n + 2, T, H, generator=g)
    a, w = torch.randn(n, generator=g), 1 + 0.1 * torch.randn(H, generator=g)
    want = plain_depth_average(list(stack[:n].double()), a.double())
    sd = stack.to(DEV)
    y = torch.empty(T, H, dtype=DT[dtype], device=DEV)
    K().depth_average(sd, n, a.to(DEV), sd[n], w.to(DEV), 1e-5, y)       # into the plane after the summed ones
    assert (sd[n].cpu().double() - want).abs().max().item() < 1e-5
    assert torch.equal(sd[:n].cpu(), stack[:n])
    wy = plain_rmsnorm(want, w.double(), 1e-5)
    assert (y.cpu().double() - wy).abs().max().item() < (1e-5 if dtype == "float32" else 4e-2)
    K().depth_average(sd, n, a.to(DEV), sd[n + 1])
    assert torch.equal(sd[n + 1], sd[n])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,H", [(1, 40), (2, 96), (4, 1536)])
def test_depth_average_with_the_convolution_of_a_decode_step(taps, H, dtype):
    """One row a sequence: average, norm, convolution and the state's update as one launch give what the three give."""
    g = torch.Generator().manual_seed(taps)
    n, T = 3, 5
    stack = torch.randn(n + 1, T, H, generator=g).to(DEV)
    a, w, cw = torch.randn(n, generator=g).to(DEV), (1 + 0.1 * torch.randn(H, generator=g)).to(DEV), torch.randn(taps, H, generator=g).to(DEV)
    slots = [3, 0, 6, 1, 4]
    state = torch.randn(7, max(taps - 1, 1), H, generator=g).to(DT[dtype]).to(DEV)[:, :taps - 1].contiguous()
    b = entries_batch([1] * T, [9] * T, slots)
    y1, u1, s1 = torch.empty(T, H, dtype=DT[dtype], device=DEV), torch.empty(T, H, dtype=DT[dtype], device=DEV), state.clone()
    K().depth_average(stack, n, a, stack[n], w, 1e-5, y1)
    K().short_conv(y1, cw, s1 if taps > 1 else None, b, u1)
    y2, u2, s2 = torch.empty_like(y1), torch.empty_like(u1), state.clone()
    K().depth_average(stack, n, a, stack[n], w, 1e-5, y2, conv=(cw, s2 if taps > 1 else None, b.seq_slot, u2))
    assert torch.equal(y1, y2) and torch.equal(u1, u2) and torch.equal(s1, s2)
    if taps > 1:
        assert not torch.equal(s1, state) and torch.equal(s1[2], state[2])      # slots 2 and 5 belong to nobody in the step


def latent_cache(R, dtype, n_pages=12, slots=4):
    return KVCache([[KVRequest(1, R, 0, planes=1)]], n_pages * 64, 1 << 20, DT[dtype], DEV, max_seqs=slots)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("R", [16, 24, 64, 200])
def test_latent_append_writes_the_normed_vector_once(R, dtype):
    g = torch.Generator().manual_seed(R)
    cache = latent_cache(R, dtype)
    s0, s1 = cache.open(2)
    counts, starts = [70, 3], [0, 0]
    for s, c in zip((s0, s1), counts):
        cache.reserve(s, c)
    cache.flush()
    wide = torch.randn(sum(counts), R + 5, generator=g).to(DT[dtype]).to(DEV)
    gw = (1 + 0.1 * torch.randn(R, generator=g)).to(DEV)
    kv = cache.layer_kv(0)
    assert kv.planes == 1 and tuple(kv.storage.shape[1:]) == (1, 1, 64, R)
    b = entries_batch(counts, starts, [s0, s1])
    K().latent_append(wide[:, 5:], gw, 1e-5, kv, b)
    r = wide[:, 5:].double().cpu()
    want = r / r.pow(2).mean(1, keepdim=True).add(1e-5).sqrt() * gw.double().cpu()
    table = kv.block_table.cpu()
    row = 0
    for s, c in zip((s0, s1), counts):
        for p in range(c):
            got = kv.storage[int(table[s, p // 64]), 0, 0, p % 64].double().cpu()
            assert (got - want[row]).abs().max().item() < (1e-5 if dtype == "float32" else 3e-2), (s, p)
            row += 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,heads,N,K_", [(1, 3, 24, 10), (8, 2, 64, 64), (9, 5, 17, 33), (70, 4, 128, 64), (300, 6, 48, 128)])
def test_head_linear(T, heads, N, K_, dtype):
    g = torch.Generator().manual_seed(T + N)
    wide = torch.randn(T, heads * K_ + 3, generator=g).to(DT[dtype])
    w = (torch.randn(heads, N, K_, generator=g) / K_ ** 0.5).to(DT[dtype])
    want = torch.einsum("thk,hnk->thn", wide[:, :heads * K_].double().view(T, heads, K_), w.double()).reshape(T, heads * N)
    out = torch.empty(T, heads * N, dtype=DT[dtype], device=DEV)
    K().head_linear(wide.to(DEV)[:, :heads * K_], w.to(DEV), out)
    assert (out.cpu().double() - want).abs().max().item() < (2e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,R", [(1, 24), (5, 64), (8, 200), (12, 32)])
def test_head_linear_appends_the_latents_of_a_decode_step(rows, R, dtype):
    """The first head product of a decode step writes the step's latents in its own launch (more rows: in one before
    it): the pages and the product are what the two kernels give apart."""
    g = torch.Generator().manual_seed(rows + R)
    heads, N, K_ = 3, 40, 16
    wide = torch.randn(rows, heads * K_ + R, generator=g).to(DT[dtype]).to(DEV)          # q heads | compressed vector
    w = (torch.randn(heads, N, K_, generator=g) / 4).to(DT[dtype]).to(DEV)
    gw = (1 + 0.1 * torch.randn(R, generator=g)).to(DEV)
    pages, outs = [], []
    for fused in (False, True):
        cache = latent_cache(R, dtype, n_pages=rows + 3, slots=rows)
        slots = cache.open(rows)
        starts = [(7 * i) % 70 for i in range(rows)]
        for s_, n in zip(slots, starts):
            cache.reserve(s_, n + 1)
        cache.flush()
        kv = cache.layer_kv(0)
        b = entries_batch([1] * rows, starts, slots)
        out = torch.empty(rows, heads * N, dtype=DT[dtype], device=DEV)
        if fused:
            K().head_linear(wide[:, :heads * K_], w, out, append=(wide[:, heads * K_:], gw, 1e-5, kv, b))
        else:
            K().latent_append(wide[:, heads * K_:], gw, 1e-5, kv, b)
            K().head_linear(wide[:, :heads * K_], w, out)
        pages.append(kv.storage.float().cpu()); outs.append(out.float().cpu())
    assert torch.equal(outs[0], outs[1])
    assert pages[0].abs().sum() > 0 and (pages[0] - pages[1]).abs().max().item() < (1e-6 if dtype == "float32" else 2e-2)


def fill_latents(cache, slots, lens, R, dtype, g):
    """Random latents for ``lens`` positions of each slot, written through the block table; returns them."""
    kv = cache.layer_kv(0)
    out = []
    for s, n in zip(slots, lens):
        cache.reserve(s, n)
    cache.flush()
    table = kv.block_table.cpu()
    for s, n in zip(slots, lens):
        c = torch.randn(n, R, generator=g).to(DT[dtype])
        for p0 in range(0, n, 64):
            m = min(64, n - p0)
            kv.storage[int(table[s, p0 // 64]), 0, 0, :m] = c[p0:p0 + m].to(DEV)
        cache.commit(s, n)
        out.append(c)
    return out


def shared_attention(qa, c, heads, R, scale, first_pos):
    """Plain: rows of one sequence at positions first_pos ..., all heads on the one latent as key and value."""
    out = torch.zeros(qa.shape[0], heads, R, dtype=torch.float64)
    q = qa.double().view(-1, heads, R)
    for t in range(qa.shape[0]):
        keys = c[:first_pos + t + 1].double()
        for h in range(heads):
            s = (keys @ q[t, h]) * scale
            out[t, h] = torch.softmax(s, 0) @ keys
    return out.reshape(qa.shape[0], heads * R)


@pytest.mark.parametrize("dtype,R,heads", [("float32", 24, 3), ("float32", 64, 2), ("bfloat16", 64, 6), ("bfloat16", 128, 20),
                                           ("bfloat16", 48, 1), ("bfloat16", 24, 2), ("bfloat16", 320, 2)])
def test_attention_over_one_plane_decoding(dtype, R, heads):
    """One row a sequence over cached latents: lengths at the pages' borders, and in every sequence one head's query
    made so that a single key (the first, one at a page's border, a far one, the newest) carries the row."""
    g = torch.Generator().manual_seed(R + heads)
    lens = [1, 63, 64, 65, 128, 129, 400]
    cache = latent_cache(R, dtype, n_pages=20, slots=8)
    slots = cache.open(len(lens))
    cs = fill_latents(cache, slots, lens, R, dtype, g)
    qa = (0.3 * torch.randn(len(lens), heads * R, generator=g))
    stand_out = [0, 0, 63, 64, 5, 128, 17]
    for i, j in enumerate(stand_out):
        qa[i, :R] = 40.0 * cs[i][j].float() / R                           # head 0: key j's score is far above the rest
    qa = qa.to(DT[dtype])
    b = entries_batch([1] * len(lens), [n - 1 for n in lens], slots)
    out = torch.empty(len(lens), heads * R, dtype=DT[dtype], device=DEV)
    K().attention(qa.to(DEV), cache.layer_kv(0), b, out, heads, 1, R, 1.0, 0, True)
    tol = 2e-5 if dtype == "float32" else 3e-2
    for i, n in enumerate(lens):
        want = shared_attention(qa[i:i + 1], cs[i], heads, R, 1.0, n - 1)
        assert (out[i:i + 1].cpu().double() - want).abs().max().item() < tol, (i, n)
        assert (want[0, :R] - cs[i][stand_out[i]].double()).abs().max().item() < 0.2      # the row IS that key


@pytest.mark.parametrize("dtype,R,heads,counts,starts", [
    ("bfloat16", 64, 4, [300, 70, 2], [0, 0, 0]),          # from position 0: the tensor-core kernel and the tiled one
    ("bfloat16", 128, 5, [260, 3], [65, 190]),             # sequences that go on
    ("bfloat16", 96, 3, [100, 64, 1], [0, 64, 7]),
    ("float32", 40, 2, [70, 5], [0, 130]),
    ("bfloat16", 288, 2, [70, 5], [0, 130]),               # wider than any tiled kernel takes: the plain one, 9 values a lane
    ("float32", 520, 1, [9, 3], [0, 66]),
])
def test_attention_over_one_plane_many_rows(dtype, R, heads, counts, starts):
    g = torch.Generator().manual_seed(R * heads)
    cache = latent_cache(R, dtype, n_pages=16, slots=4)
    slots = cache.open(len(counts))
    cs = fill_latents(cache, slots, [s + c for s, c in zip(starts, counts)], R, dtype, g)
    qa = (0.3 * torch.randn(sum(counts), heads * R, generator=g))
    qa[counts[0] - 1, :R] = 40.0 * cs[0][1].float() / R                     # the first sequence's last row: key 1 stands out
    qa = qa.to(DT[dtype])
    b = entries_batch(counts, starts, slots)
    out = torch.empty(sum(counts), heads * R, dtype=DT[dtype], device=DEV)
    K().attention(qa.to(DEV), cache.layer_kv(0), b, out, heads, 1, R, 1.0, 0, True)
    r = 0
    for i, c in enumerate(counts):
        want = shared_attention(qa[r:r + c], cs[i], heads, R, 1.0, starts[i])
        assert (out[r:r + c].cpu().double() - want).abs().max().item() < (2e-5 if dtype == "float32" else 3e-2), i
        r += c
    assert K().device_errors() == 0


# ------------------------------------------------------------------------------------------- the model
_models, _plain = {}, {}


def model_of(name, dtype, max_tokens=2048):
    if (name, dtype) not in _models:
        _models[(name, dtype)] = gpu_model(name, dtype, max_tokens=max_tokens)
    return _models[(name, dtype)]


def plain_logits(name, toks):
    key = (name, tuple(toks))
    if key not in _plain:
        cfg, W = plain_weights(name)
        _plain[key] = plain_forward(cfg, W, toks)[0]
    return _plain[key]


def tol_of(name, dtype):
    return TOL[dtype] * (4 if name == "SHARP" else 1)


LENGTHS = {"A": 150, "B": 131, "C": 330, "D": 70, "SHARP": 200}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_and_token_by_token(name, dtype):
    cfg = CONFIGS[name]
    toks = random_tokens(cfg["vocab"], LENGTHS[name], seed=3)
    m = model_of(name, dtype)
    want = plain_logits(name, toks)
    assert row_errors(run_whole(m, toks), want).max() < tol_of(name, dtype)
    assert row_errors(run_tail_one_by_one(m, toks, 70), want).max() < tol_of(name, dtype)      # across a page's border
    assert row_errors(run_tail_one_by_one(m, toks[:5], 5), want[:5]).max() < tol_of(name, dtype)   # the first tokens
    assert row_errors(run_whole(m, toks[:1]), want[:1]).max() < tol_of(name, dtype)
    m.cache.check()
    assert m.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_down_to_two_tokens(name, dtype):
    cfg = CONFIGS[name]
    a, b_ = random_tokens(cfg["vocab"], LENGTHS[name], seed=5), random_tokens(cfg["vocab"], 90, seed=6)
    m = model_of(name, dtype)
    got = run_in_pieces(m, [a, b_], [[2, 4, 7, 64, 66, 128, 129], [63, 65, 67]])
    assert row_errors(got[0], plain_logits(name, a)).max() < tol_of(name, dtype)
    assert row_errors(got[1], plain_logits(name, b_)).max() < tol_of(name, dtype)
    assert m.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "SHARP"])
def test_unequal_batches_on_reused_slots_and_pages(name, dtype):
    """Three rounds on a cache of three slots and six pages: later sequences get the slots, the pages and the
    convolution state of earlier ones, shorter requests end earlier."""
    cfg = CONFIGS[name]
    m = gpu_model(name, dtype, max_tokens=64 * 6, max_seqs=3)
    for rnd in range(3):
        lens = [[5, 1, 130], [66, 3, 64], [1, 1, 63]][rnd]
        seqs = [random_tokens(cfg["vocab"], n + (2 if i == 1 else 9), seed=10 * rnd + i) for i, n in enumerate(lens)]
        got = run_batched(m, seqs, lens)
        for q, g_ in zip(seqs, got):
            assert row_errors(g_, plain_logits(name, q)).max() < tol_of(name, dtype), (rnd, len(q))
        m.cache.check()
        assert m.cache.slots.held == 0


def test_sharp_attention_rests_on_far_keys():
    """The configuration with large score factors does what it is for: in its first layer, many rows put most of
    their weight on one key, often hundreds of positions back, so that a lost or doubled key anywhere shows."""
    cfg, W = plain_weights("SHARP")
    toks = random_tokens(cfg["vocab"], LENGTHS["SHARP"], seed=3)
    w = {k: v.double() for k, v in W.items()}
    x = plain_embed(w["embed"], toks, cfg["embedding"]["scale"])
    u = plain_canon(plain_rmsnorm(x, w["l0.norm1"], cfg["norm"]["eps"]), w["l0.canon1"])
    c = plain_latent(u, w["l0.mix.dkv"], w["l0.mix.dkv.norm"], cfg["norm"]["eps"])
    mx = cfg["layers"][0]["mixer"]
    T = len(toks)
    q = (u @ w["l0.mix.q"].T).view(T, mx["heads"], mx["dim"])
    k = (c @ w["l0.mix.uk"].T).view(T, mx["heads"], mx["dim"])
    s = torch.einsum("thd,shd->hts", q, k) * mx["scale"]
    p = torch.softmax(s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf")), dim=2)
    top, where = p.max(dim=2)
    far = (top > 0.5) & ((torch.arange(T)[None, :] - where) > 64)
    assert far.sum().item() >= 10


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    cfg = CONFIGS["A"]
    toks = random_tokens(cfg["vocab"], 300, seed=9)
    m = model_of("A", dtype)
    assert row_errors(run_tail_one_by_one(m, toks, 297), plain_logits("A", toks)).max() < tol_of("A", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_composition_and_slot_do_not_change_a_row(dtype):
    cfg = CONFIGS["C"]
    m = model_of("C", dtype)
    a, others = random_tokens(cfg["vocab"], 140, seed=1), [random_tokens(cfg["vocab"], n, seed=n) for n in (300, 7)]
    alone = run_batched(m, [a], [130])[0]
    among = run_batched(m, [others[0], a, others[1]], [290, 130, 3])[1]
    assert row_errors(among, alone).max() < (1e-5 if dtype == "float32" else TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype):
    name = "B"
    cfg, W = plain_weights(name)
    lm = cima_b200.load(folder(name), dtype=dtype, max_tokens=1024, verbose=False)
    prompts = [random_tokens(cfg["vocab"], n, seed=40 + n) for n in (7, 1, 70, 64)]
    got = lm.generate(prompts, temperature=0, repeat_penalty=1.0, max_tokens=12)
    for p, r in zip(prompts, got):
        assert r.finish_reason == "length" and len(r.tokens) == 12
        seq = list(p)
        for t in r.tokens:
            lg = plain_forward(cfg, W, seq)[0][-1]
            assert lg[t] >= lg.max() - (1e-5 if dtype == "float32" else 2e-2)
            seq.append(t)
    assert lm.model.cache.slots.held == 0
    # a second call finds slots, pages and state that the first one used
    again = lm.generate(prompts[:2], temperature=0, repeat_penalty=1.0, max_tokens=12)
    if dtype == "float32":
        assert [r.tokens for r in again] == [r.tokens for r in got[:2]]


def test_model_from_a_configuration_in_memory_steps_and_writes_out(tmp_path):
    lm = cima_b200.load(config=CONFIGS["D"], seed=4, dtype="float32", max_tokens=256, verbose=False)
    cima_b200.write_random_model(str(tmp_path / "m"), CONFIGS["D"], seed=4)
    from safetensors.torch import load_file
    W = load_file(str(tmp_path / "m" / "model.safetensors"))
    toks = random_tokens(CONFIGS["D"]["vocab"], 20, seed=1)
    assert row_errors(run_whole(lm.model, toks), plain_forward(CONFIGS["D"], W, toks)[0]).max() < TOL["float32"]


def test_trace_replay_of_this_design(tmp_path):
    name = "A"
    cfg = CONFIGS[name]
    V = cfg["vocab"]
    reqs = {"a": random_tokens(V, 70, seed=1), "b": random_tokens(V, 9, seed=2)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"][:66], "want": [0, 65]},
                                     {"id": "b", "tokens": reqs["b"][:5], "want": [4]}], "end": []}]
    for j in range(4):
        steps.append({"step": j + 1, "entries": [{"id": "a", "tokens": [reqs["a"][66 + j]], "want": [0]},
                                                 {"id": "b", "tokens": [reqs["b"][5 + j]], "want": [0]}],
                      "end": ["a", "b"] if j == 3 else []})
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder(name), "--dtype", "float32",
                        "--out", str(tmp_path), "--max-tokens", "256"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    wa, wb = plain_logits(name, reqs["a"]), plain_logits(name, reqs["b"])
    got = torch.from_numpy(np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(-1, V).copy())
    assert row_errors(got, torch.stack([wa[0], wa[65], wb[4]])).max() < TOL["float32"]
    for j in range(4):
        got = torch.from_numpy(np.fromfile(tmp_path / f"{j + 1}.f32", dtype="<f4").reshape(-1, V).copy())
        assert row_errors(got, torch.stack([wa[66 + j], wb[5 + j]])).max() < TOL["float32"]
