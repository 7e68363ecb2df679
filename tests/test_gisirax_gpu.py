"""The Gisirax design on the GPU: each new kernel alone against a plain statement of it, then the model in every cutting
(whole, token by token, pieces down to two tokens, unequal batches, reused slots, pages and state, long decoding), in
32-bit and in bfloat16, on configurations that differ in every size, and generation through the entry point."""
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
from gisirax_cases import CONFIGS, folder, gpu_model, plain_weights, row_errors
from gisirax_plain import (plain_causal_taps, plain_forward, plain_rotary_frequencies, plain_rotate, plain_route, plain_silu)
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole
from reference_kernels import ReferenceKernels

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda:0"
REF = ReferenceKernels()
_kernels = []


def K():
    if not _kernels:
        from cima_b200.kernels import Kernels
        _kernels.append(Kernels(verbose=False))
    return _kernels[0]


def entries_batch(counts, starts, slots=None, tokens=None, device=DEV):
    slots = slots or list(range(len(counts)))
    tokens = tokens or [[0] * c for c in counts]
    return build_batch([StepEntry(s, t, []) for s, t in zip(slots, tokens)], starts, 1 << 30, device)


def close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H", [(1, 40), (7, 96), (300, 257)])
def test_dynamic_tanh_alone_and_behind_a_sublayer(T, H, dtype):
    g = torch.Generator().manual_seed(T + H)
    x, y = torch.randn(T, H, generator=g) * 3, torch.randn(T, H, generator=g) * 2
    n1 = (torch.tensor([0.7]), torch.randn(H, generator=g), torch.randn(H, generator=g))
    n2 = (torch.tensor([1.9]), torch.randn(H, generator=g), torch.randn(H, generator=g))
    out = torch.empty(T, H, dtype=DT[dtype], device=DEV)
    K().dyt(x.to(DEV), *[t.to(DEV) for t in n1], out)
    want = torch.tanh(0.7 * x.double()) * n1[1].double() + n1[2].double()
    assert close(out, want, 1e-6 if dtype == "float32" else 8e-3)
    for second in (False, True):
        xd, h = x.to(DEV).clone(), torch.empty(T, H, dtype=DT[dtype], device=DEV)
        K().dyt_add(xd, y.to(DEV), tuple(t.to(DEV) for t in n1), 0.6, tuple(t.to(DEV) for t in n2) if second else None,
                    h if second else None)
        wx = x.double() + 0.6 * (torch.tanh(0.7 * y.double()) * n1[1].double() + n1[2].double())
        assert close(xd, wx, 1e-6)
        if second:
            assert close(h, torch.tanh(1.9 * wx) * n2[1].double() + n2[2].double(), 2e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_bigram_embedding_keeps_the_token_before_a_step(dtype):
    """Three sequences in three steps (many rows, a few, one each) on slots that held other tokens before."""
    V, H, buckets, mp, mc = 50, 24, 13, 29, 5
    g = torch.Generator().manual_seed(1)
    table, big = torch.randn(V, H, generator=g).to(DT[dtype]), torch.randn(buckets + 1, H, generator=g).to(DT[dtype])
    seqs = [random_tokens(V, n, seed=n) for n in (9, 4, 6)]
    slots = [3, 0, 2]
    state = torch.full((5,), 17, dtype=torch.int32, device=DEV)
    state[slots] = 0                                                           # a slot's state is zeroed when it opens
    pos = [0, 0, 0]
    for counts in ([6, 1, 3], [2, 2, 2], [1, 1, 1]):
        toks = [q[p:p + c] for q, p, c in zip(seqs, pos, counts)]
        b = entries_batch(counts, pos, slots, toks)
        x = torch.empty(sum(counts), H, dtype=torch.float32, device=DEV)
        K().embed_bigram(b, table.to(DEV), big.to(DEV), x, 2.5, buckets, mp, mc, state)
        r = 0
        for q, p, c in zip(seqs, pos, counts):
            for t in range(p, p + c):
                row = buckets if t == 0 else (q[t - 1] * mp + q[t] * mc) % buckets
                assert close(x[r], table[q[t]].double() * 2.5 + big[row].double(), 1e-6), (counts, t)
                r += 1
        pos = [p + c for p, c in zip(pos, counts)]
    assert state[slots].tolist() == [q[p - 1] for q, p in zip(seqs, pos)] and int(state[1]) == 17


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,C", [(1, 40), (2, 304), (3, 64), (4, 512), (5, 257)])
def test_plain_convolution_with_activation_in_pieces(taps, C, dtype):
    g = torch.Generator().manual_seed(taps * 1000 + C)
    lens = [11, 2, 7]
    w = torch.randn(C, taps, generator=g)
    hs = [torch.randn(n + 5, C, generator=g).to(DT[dtype]) for n in lens]
    want = [plain_silu(plain_causal_taps(h.double(), w.double())) for h in hs]
    state = torch.zeros(5, max(taps - 1, 1), C, dtype=DT[dtype], device=DEV)[:, :taps - 1]
    slots, got, pos = [4, 0, 2], [[] for _ in lens], [0, 0, 0]
    for counts in (lens, [4, 4, 4], [1, 1, 1]):
        b = entries_batch(counts, pos, slots)
        h = torch.cat([hs[i][pos[i]:pos[i] + c] for i, c in enumerate(counts)]).to(DEV)
        out = torch.empty_like(h)
        K().short_conv(h, w.t().contiguous().to(DEV), state if taps > 1 else None, b, out, add_input=False, act=0)
        r = 0
        for i, c in enumerate(counts):
            got[i].append(out[r:r + c].cpu()); r += c
        pos = [p + c for p, c in zip(pos, counts)]
    for gi, wi in zip(got, want):
        assert close(torch.cat(gi), wi, 2e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim", [(2, 1, 16), (3, 3, 40), (4, 2, 128)])
def test_delta_prepare(heads, kv_heads, dim, dtype):
    T = 9
    g = torch.Generator().manual_seed(dim)
    wide = torch.randn(T, 2 * kv_heads * dim + 24, generator=g).to(DT[dtype]).to(DEV)         # q | k | (v)
    a = (torch.randn(T, heads * dim, generator=g) * 2).to(DT[dtype]).to(DEV)
    b = torch.randn(T, heads, generator=g).to(DT[dtype]).to(DEV)
    A_log, dt = torch.randn(heads, generator=g).to(DEV), torch.randn(heads * dim, generator=g).to(DEV)
    outs = [[torch.empty(T, n, dtype=torch.float32, device=d) for n in (kv_heads * dim, kv_heads * dim, heads * dim, heads)]
            for d in (DEV, "cpu")]
    K().delta_prepare(wide, a, b, A_log, dt, *outs[0], heads, kv_heads, dim)
    REF.delta_prepare(wide.cpu(), a.cpu(), b.cpu(), A_log.cpu(), dt.cpu(), *outs[1], heads, kv_heads, dim)
    for got, want in zip(*outs):
        assert close(got, want, 2e-6)
    qn = outs[0][0].view(T, kv_heads, dim)
    assert close((qn * qn).sum(-1) * dim, torch.ones(T, kv_heads), 1e-4)                         # unit length, then dim^-1/2


def _recurrence_case(delta, heads, kv_heads, dim, vdim, dtype, counts_per_step, seed):
    """The same sequences through the kernel in the given pieces and through the plain statement whole."""
    g = torch.Generator().manual_seed(seed)
    n_seqs = len(counts_per_step[0])
    lens = [sum(step[i] for step in counts_per_step) for i in range(n_seqs)]
    qdt = torch.float32 if delta else DT[dtype]
    data = []
    for n in lens:
        q, k = torch.randn(n, kv_heads * dim, generator=g).to(qdt), torch.randn(n, kv_heads * dim, generator=g).to(qdt)
        if delta:
            k = k / k.view(n, kv_heads, dim).norm(dim=-1, keepdim=True).repeat_interleave(dim, dim=-1).view(n, -1)
        v = torch.randn(n, heads * vdim, generator=g).to(DT[dtype])
        gg = torch.rand(n, heads * dim, generator=g) * 0.5 + 0.5
        beta = torch.rand(n, heads, generator=g)
        data.append((q, k, v, gg, beta))
    decay = torch.tensor([0.5 + 0.499 * i / max(1, heads - 1) for i in range(heads)])
    slots = [5, 1, 3, 0][:n_seqs]
    state = torch.randn(7, heads, dim, vdim, generator=g).to(DEV)
    state[slots] = 0
    want_state = torch.zeros(7, heads, dim, vdim)
    wants = []
    for i, (q, k, v, gg, beta) in enumerate(data):
        b = entries_batch([lens[i]], [0], [slots[i]], device="cpu")
        o = torch.zeros(lens[i], heads * vdim)
        REF.recurrence(q, k, v, want_state, b, o, heads, kv_heads, dim, vdim, **(dict(g=gg, beta=beta) if delta else dict(decay=decay)))
        wants.append(o)
    got, pos = [[] for _ in lens], [0] * n_seqs
    for counts in counts_per_step:
        live = [i for i, c in enumerate(counts) if c > 0]
        b = entries_batch([counts[i] for i in live], [pos[i] for i in live], [slots[i] for i in live])
        cat = lambda j: torch.cat([data[i][j][pos[i]:pos[i] + counts[i]] for i in live]).to(DEV)
        o = torch.empty(b.n_rows, heads * vdim, dtype=torch.float32, device=DEV)
        # q, k, v as column slices of one wider matrix, as a mixer hands them over
        if delta:
            K().recurrence(cat(0), cat(1), cat(2), state, b, o, heads, kv_heads, dim, vdim, g=cat(3), beta=cat(4))
        else:
            wide = torch.cat([cat(0), cat(1), cat(2)], dim=1)
            kd = kv_heads * dim
            K().recurrence(wide[:, :kd], wide[:, kd:2 * kd], wide[:, 2 * kd:], state, b, o, heads, kv_heads, dim, vdim, decay=decay.to(DEV))
        r = 0
        for i in live:
            got[i].append(o[r:r + counts[i]].cpu()); r += counts[i]
            pos[i] += counts[i]
    for gi, wi in zip(got, wants):
        assert close(torch.cat(gi), wi, 3e-5)
    assert close(state[slots], want_state[slots], 3e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("delta", [True, False])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(2, 1, 16, 24), (3, 3, 40, 8), (2, 2, 128, 64), (1, 1, 8, 100), (2, 1, 200, 16)])
def test_recurrence_whole_in_pieces_and_token_by_token(heads, kv_heads, dim, vdim, delta, dtype):
    if not delta:
        kv_heads = heads
    steps = [[20, 3, 9], [2, 2, 2], [1, 1, 1], [1, 0, 1], [17, 0, 1]]
    _recurrence_case(delta, heads, kv_heads, dim, vdim, dtype, steps, seed=dim + vdim)


def test_recurrence_long_decoding_holds_its_state():
    _recurrence_case(True, 2, 1, 32, 32, "float32", [[3, 1]] + [[1, 1]] * 150, seed=5)
    _recurrence_case(False, 2, 2, 32, 32, "bfloat16", [[3, 1]] + [[1, 1]] * 150, seed=6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,groups,n,shared,gated", [(5, 3, 24, True, True), (9, 1, 200, False, True), (70, 4, 64, True, False),
                                                      (3, 2, 33, False, True)])
def test_group_rmsnorm_gate(T, groups, n, shared, gated, dtype):
    g = torch.Generator().manual_seed(T * n)
    o = torch.randn(T, groups * n, generator=g) * 3
    w = torch.randn(n if shared else groups * n, generator=g)
    wide = torch.randn(T, groups * n + 8, generator=g).to(DT[dtype])
    out = torch.empty(T, groups * n, dtype=DT[dtype], device=DEV)
    K().group_rmsnorm_gate(o.to(DEV), w.to(DEV), wide.to(DEV)[:, 8:] if gated else None, out, groups, 1e-5)
    z = o.double().view(T, groups, n)
    z = z / torch.sqrt((z * z).mean(-1, keepdim=True) + 1e-5) * (w.double().view(1, 1, n) if shared else w.double().view(1, groups, n))
    if gated:
        z = z * torch.sigmoid(wide[:, 8:].double().view(T, groups, n))
    assert close(out, z.view(T, -1), 2e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("T,H,n", [(1, 40, 2), (9, 257, 1), (70, 1024, 3)])
def test_rms_mean_of_branches(T, H, n):
    g = torch.Generator().manual_seed(T + H)
    ys, ws = [torch.randn(T, H, generator=g) * (i + 1) for i in range(n)], [torch.randn(H, generator=g) for _ in range(n)]
    x = torch.randn(T, H, generator=g)
    xd = x.to(DEV).clone()
    K().rms_mean([y.to(DEV) for y in ys], [w.to(DEV) for w in ws], xd, 1e-6)
    want = x.double() + sum(y.double() / torch.sqrt((y.double() ** 2).mean(-1, keepdim=True) + 1e-6) * w.double() for y, w in zip(ys, ws)) / n
    assert close(xd, want, 2e-6)


@pytest.mark.parametrize("E,top,groups,keep", [(15, 4, 5, 3), (8, 2, 2, 1), (6, 3, 3, 2), (4, 1, 1, 1), (3, 3, 1, 1), (64, 6, 8, 4),
                                                (5, 2, 5, 3)])
def test_router_choice_and_weights(E, top, groups, keep):
    T, H = 50, 32
    g = torch.Generator().manual_seed(E * 7 + top)
    h, wr = torch.randn(T, H, generator=g).double(), torch.randn(E, H, generator=g).double() * 0.3
    scores = (h @ wr.T).float().to(DEV)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wgt = torch.empty(T, top, dtype=torch.float32, device=DEV)
    K().moe_route(scores.clone(), top, groups, keep, 1.25, idx, wgt)
    ids, ws = plain_route(h, wr, top, groups, keep, 1.25)
    assert idx.cpu().tolist() == ids
    assert close(wgt, ws, 2e-6)
    # the same launch can order the pairs by expert (a decode step's few rows)
    idx2, wgt2 = torch.empty_like(idx), torch.empty_like(wgt)
    meta = K().moe_route(scores.clone(), top, groups, keep, 1.25, idx2, wgt2, order=True).cpu()
    assert torch.equal(idx2, idx) and torch.equal(wgt2, wgt)
    offsets, tiles, perm = meta[:E + 1], meta[E + 1:2 * (E + 1)], meta[2 * (E + 1):]
    flat = idx.cpu().flatten()
    assert sorted(perm.tolist()) == list(range(T * top)) and (flat[perm.long()].diff() >= 0).all()
    assert offsets.tolist() == [int((flat < e).sum()) for e in range(E + 1)]
    assert tiles.tolist() == [sum(-(-int((flat == j).sum()) // 32) for j in range(e)) for e in range(E + 1)]
    x1, x2 = torch.zeros(T, H, device=DEV), torch.zeros(T, H, device=DEV)
    gu, dn = torch.randn(E, 16, H, generator=g).to(DEV), torch.randn(E, H, 8, generator=g).to(DEV)
    K().moe_experts(h.float().to(DEV), gu, dn, idx, wgt, x1, 0)
    K().moe_experts(h.float().to(DEV), gu, dn, idx, wgt, x2, 0, ordered=meta.to(DEV))
    assert torch.equal(x1, x2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H,ff,E,top", [(1, 40, 24, 3, 3), (5, 96, 40, 8, 2), (200, 64, 56, 6, 1), (70, 100, 33, 10, 4),
                                          (1100, 64, 56, 6, 1), (600, 128, 200, 5, 2), (30, 256, 64, 4, 4)])
def test_experts_in_tiles_of_one_expert(T, H, ff, E, top, dtype):
    """Rows spread unevenly over the experts (one expert gets none, one gets most): every tile is one expert's.  The sizes
    reach all three roads of the products: a warp a feature (few pairs), plain tiles, and tensor-core tiles of 256 pairs."""
    g = torch.Generator().manual_seed(T * E)
    h = torch.randn(T, H, generator=g).to(DT[dtype])
    gu, dn = (torch.randn(E, 2 * ff, H, generator=g) * H ** -0.5).to(DT[dtype]), (torch.randn(E, H, ff, generator=g) * ff ** -0.5).to(DT[dtype])
    pick = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)])
    if E > top:
        pick[pick == 1] = 0 if top == 1 else pick[pick == 1]                    # with one choice a row, expert 1 stays empty
    idx = pick.to(torch.int32)
    wgt = torch.rand(T, top, generator=g)
    x = torch.randn(T, H, generator=g)
    xd, xr = x.to(DEV).clone(), x.clone()
    K().moe_experts(h.to(DEV), gu.to(DEV), dn.to(DEV), idx.to(DEV), wgt.to(DEV), xd, 0)
    REF.moe_experts(h, gu, dn, idx, wgt, xr, 0)
    assert close(xd, xr, 1e-5 if dtype == "float32" else 2e-2)


def test_rescaled_rotary_frequencies():
    from cima_b200.config.specs import PositionSpec
    from cima_b200.parts import Runtime, build_position
    rt = Runtime(kernels=None, dtype=torch.float32, device="cpu")
    for dims, base, sc in ((16, 10000.0, (8.0, 1.0, 4.0, 64)), (64, 2e5, (3.0, 1.0, 8.0, 1024)), (48, 500.0, (2.0, 0.5, 8.0, 100)),
                           (32, 1e4, None)):
        params = {"scaling": dict(zip(("factor", "low", "high", "original"), sc))} if sc else {}
        pos = build_position(PositionSpec(kind="rope", head_dim=dims + 16, rotary_dim=dims, theta=base, params=params), rt)
        want = plain_rotary_frequencies(dims, base, params.get("scaling"))
        assert torch.allclose(pos.inv_freq.double(), want, rtol=1e-6, atol=0)
        if sc:                                                       # all three branches of the rule occur
            wave = 2 * np.pi / plain_rotary_frequencies(dims, base).numpy()
            assert (wave < sc[3] / sc[2]).any() and (wave > sc[3] / sc[1]).any()


def _sink_attention(q, k, v, scale, sink, first_pos):
    """q [n, heads, D], k, v [len, kv, D]: row i stands at position first_pos + i."""
    n, heads, D = q.shape
    share = heads // k.shape[1]
    out = torch.zeros(n, heads, D, dtype=torch.float64)
    for i in range(n):
        p = first_pos + i
        for h in range(heads):
            s = (k[:p + 1, h // share].double() @ q[i, h].double()) * scale
            m = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - m)
            out[i, h] = (e / (e.sum() + sink * torch.exp(-m))) @ v[:p + 1, h // share].double()
    return out.view(n, heads * D)


@pytest.mark.parametrize("dtype,D,heads,kv", [("float32", 48, 4, 2), ("bfloat16", 48, 4, 2), ("bfloat16", 64, 4, 1), ("bfloat16", 128, 2, 2),
                                              ("float32", 16, 3, 3)])
def test_attention_with_a_sink_through_every_kernel(dtype, D, heads, kv):
    """Sequences of 1 to 400 positions through prompts (the step's own keys), pieces that go on from the cache and single
    tokens.  In every sequence queries are made so that a single key carries their row (the first, one at a page's
    border, a far one)."""
    g = torch.Generator().manual_seed(D + heads)
    lens = [1, 63, 65, 129, 400]
    scale, sink = 0.3, 1.0
    cache = KVCache([[KVRequest(kv, D, 0)]], max_tokens=64 * 16, max_position=4096, dtype=DT[dtype], device=DEV)
    slots = cache.open(len(lens))
    qs = [torch.randn(n, heads, D, generator=g) for n in lens]
    ks = [torch.randn(n, kv, D, generator=g) for n in lens]
    vs = [torch.randn(n, kv, D, generator=g) for n in lens]
    for q, k, n in zip(qs, ks, lens):
        for row, key in ((n - 1, 0), (n - 1 if n < 66 else 70, min(n - 1, 64)), (n - 1, max(0, n - 300))):
            if key <= row:
                q[row, 0] = k[key, 0] * 3.0                                  # score about 3 * D * 0.3 against a spread of sqrt(D)
    qs = [q.to(DT[dtype]) for q in qs]; ks = [k.to(DT[dtype]) for k in ks]; vs = [v.to(DT[dtype]) for v in vs]
    wants = [_sink_attention(q.float(), k.float(), v.float(), scale, sink, 0) for q, k, v in zip(qs, ks, vs)]
    tol = 2e-5 if dtype == "float32" else 2e-2
    zero = torch.zeros(1, dtype=torch.float32, device=DEV)

    def run(counts, starts, from_cache):
        live = [i for i, c in enumerate(counts) if c > 0]
        b = build_batch([StepEntry(slots[i], [0] * counts[i], []) for i in live], [starts[i] for i in live], 1, DEV)
        for i in live:
            cache.reserve(slots[i], starts[i] + counts[i])
        cache.flush()
        qkv = torch.cat([torch.cat([qs[i][starts[i]:starts[i] + counts[i]].reshape(counts[i], -1),
                                    ks[i][starts[i]:starts[i] + counts[i]].reshape(counts[i], -1),
                                    vs[i][starts[i]:starts[i] + counts[i]].reshape(counts[i], -1)], dim=1) for i in live]).to(DEV).contiguous()
        kvl = cache.layer_kv(0)
        K().rope_append(qkv, zero[:0], 0, b.row_pos, b.row_seq, b.seq_slot, b.seq_len, kvl, heads, kv, D)
        out = torch.empty(qkv.shape[0], heads * D, dtype=DT[dtype], device=DEV)
        K().attention(qkv, kvl, b, out, heads, kv, D, scale, 0, from_cache, sink=sink)
        r = 0
        for i in live:
            w = wants[i][starts[i]:starts[i] + counts[i]]
            assert close(out[r:r + counts[i]], w, tol), (counts, i, float((out[r:r + counts[i]].double().cpu() - w).abs().max()))
            cache.commit(slots[i], starts[i] + counts[i])
            r += counts[i]

    run([1, 40, 40, 100, 300], [0] * 5, False)                                # prompts: the step's own keys
    run([0, 20, 24, 28, 99], [1, 40, 40, 100, 300], True)                     # pieces that go on from the cache (one of 99 rows)
    run([0, 1, 1, 1, 1], [1, 60, 64, 128, 399], True)                         # single tokens: the decode kernel
    run([0, 2, 0, 0, 0], [0, 61, 0, 0, 0], True)
    cache.close(slots)
    # the whole prompts through the cache once more, on the slots and pages just given back: long enough for the tensor-core kernel
    slots = cache.open(len(lens))
    run(lens, [0] * 5, False)
    cache.close(slots)


def test_a_query_far_below_the_sink_gives_nearly_nothing():
    D, heads, n = 32, 2, 70
    g = torch.Generator().manual_seed(3)
    q = torch.randn(n, heads, D, generator=g)
    k = torch.randn(n, 1, D, generator=g)
    v = torch.randn(n, 1, D, generator=g)
    q[-1, 0] = -50.0 * k[:, 0].mean(0) / k[:, 0].mean(0).norm()               # all of its scores negative or small
    k = k + 3.0 * k[:, 0].mean(0) / k[:, 0].mean(0).norm()
    want = _sink_attention(q, k, v, 1.0, 1.0, 0)
    plain = _sink_attention(q, k, v, 1.0, 0.0, 0)
    assert want[-1, :D].abs().max() < 0.05 * plain[-1, :D].abs().max()         # the sink takes the row's weight
    cache = KVCache([[KVRequest(1, D, 0)]], max_tokens=128, max_position=4096, dtype=torch.float32, device=DEV)
    (slot,) = cache.open(1)
    b = build_batch([StepEntry(slot, [0] * n, [])], [0], 1, DEV)
    cache.reserve(slot, n); cache.flush()
    qkv = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], dim=1).to(DEV)
    out = torch.empty(n, heads * D, device=DEV)
    K().attention(qkv, cache.layer_kv(0), b, out, heads, 1, D, 1.0, 0, False, sink=1.0)
    assert close(out, want, 2e-5)


# ------------------------------------------------------------------------------------------- the model
TOL = {"float32": 3e-5, "bfloat16": 6e-2}
_models, _plain = {}, {}


def model_of(name, dtype, max_tokens=2048):
    if (name, dtype) not in _models:
        _models[(name, dtype)] = gpu_model(name, dtype, max_tokens=max_tokens)
    return _models[(name, dtype)]


def plain_logits(name, toks):
    key = (name, tuple(toks))
    if key not in _plain:
        cfg, W = plain_weights(name)
        _plain[key] = plain_forward(cfg, W, toks)
    return _plain[key]


def agrees(got, want, dtype, what=""):
    """32-bit: every row.  bfloat16: the rounding of a router's input can change a close choice of experts, which moves
    that row (and little of what follows): nearly all rows, and the median far inside the tolerance."""
    e = row_errors(got, want)
    if dtype == "float32":
        assert e.max() < TOL[dtype], (what, float(e.max()))
    else:
        assert e.median() < TOL[dtype] / 2 and (e > TOL[dtype]).float().mean() <= 0.25, (what, float(e.median()), float(e.max()))


LENGTHS = {"A": 150, "B": 131, "C": 330}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_and_token_by_token(name, dtype):
    cfg = CONFIGS[name]
    toks = random_tokens(cfg["vocab"], LENGTHS[name], seed=3)
    m = model_of(name, dtype)
    want = plain_logits(name, toks)
    agrees(run_whole(m, toks), want, dtype, "whole")
    agrees(run_tail_one_by_one(m, toks, 70), want, dtype, "tail")            # across a page's border
    agrees(run_tail_one_by_one(m, toks[:5], 5), want[:5], dtype, "first tokens")
    agrees(run_whole(m, toks[:1]), want[:1], dtype, "one token")
    m.cache.check()
    assert m.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_down_to_two_tokens(name, dtype):
    cfg = CONFIGS[name]
    a, b_ = random_tokens(cfg["vocab"], LENGTHS[name], seed=5), random_tokens(cfg["vocab"], 90, seed=6)
    m = model_of(name, dtype)
    got = run_in_pieces(m, [a, b_], [[2, 4, 7, 64, 66, 128, 129], [63, 65, 67]])
    agrees(got[0], plain_logits(name, a), dtype)
    agrees(got[1], plain_logits(name, b_), dtype)
    if dtype == "float32":                                                    # the cutting changes nothing but rounding
        assert row_errors(got[0], run_whole(m, a)).max() < 2e-5
    assert m.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_on_reused_slots_pages_and_state(name, dtype):
    """Three rounds on a cache of three slots and six pages: later sequences get the slots, the pages, the recurrent
    state, the convolution's inputs and the last token of earlier ones; shorter requests end earlier."""
    cfg = CONFIGS[name]
    m = gpu_model(name, dtype, max_tokens=64 * 6, max_seqs=3)
    for rnd in range(3):
        lens = [[5, 1, 130], [66, 3, 64], [1, 1, 63]][rnd]
        seqs = [random_tokens(cfg["vocab"], n + (2 if i == 1 else 9), seed=10 * rnd + i) for i, n in enumerate(lens)]
        got = run_batched(m, seqs, lens)
        for q, g_ in zip(seqs, got):
            agrees(g_, plain_logits(name, q), dtype, (rnd, len(q)))
        m.cache.check()
        assert m.cache.slots.held == 0


def test_sharp_attention_rests_on_far_keys():
    """The test weights do what they are for: in the softmax branch of configuration C's first layer many rows put most
    of their weight on one key, often more than a page back, and among the first positions some give most of it to the sink."""
    from gisirax_plain import plain_dyt, plain_embedding, plain_sink_attention
    cfg, W = plain_weights("C")
    toks = random_tokens(cfg["vocab"], LENGTHS["C"], seed=3)
    big = cfg["embedding"]["bigram"]
    x = plain_embedding(toks, W["embed"], W["bigram"], cfg["embedding"]["scale"], big["buckets"], big["mul_prev"], big["mul_cur"])
    h = plain_dyt(x, W["l0.norm1"], W["l0.norm1.b"], W["l0.norm1.alpha"])
    L = cfg["layers"][0]["mixer"]["left"]
    fr = plain_rotary_frequencies(L["rot"]["dims"], L["rot"]["base"], L["rot"].get("scaling"))
    _, p = plain_sink_attention(h, W["l0.mix.left.q"], W["l0.mix.left.k"], W["l0.mix.left.v"], W["l0.mix.left.o"], L["heads"],
                                L["kv_heads"], L["dim"], L["vdim"], L["scale"], fr, return_weights=True)
    top, where = p.max(dim=2)
    T = len(toks)
    assert ((top > 0.5) & ((torch.arange(T)[None, :] - where) > 64)).sum().item() >= 10
    assert (p.sum(dim=2) < 0.5).sum().item() >= 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    cfg = CONFIGS["A"]
    toks = random_tokens(cfg["vocab"], 300, seed=9)
    agrees(run_tail_one_by_one(model_of("A", dtype), toks, 297), plain_logits("A", toks), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_composition_and_slot_do_not_change_a_row(dtype):
    cfg = CONFIGS["C"]
    m = model_of("C", dtype)
    a, others = random_tokens(cfg["vocab"], 140, seed=1), [random_tokens(cfg["vocab"], n, seed=n) for n in (300, 7)]
    alone = run_batched(m, [a], [130])[0]
    among = run_batched(m, [others[0], a, others[1]], [290, 130, 3])[1]
    e = row_errors(among, alone)
    if dtype == "float32":
        assert e.max() < 1e-5
    else:           # other kernels serve the larger batch; where their rounding turns a close choice of experts, a row moves
        assert e.median() < 1e-2 and (e > 2e-2).float().mean() <= 0.25, (float(e.median()), float(e.max()))


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
            lg = plain_forward(cfg, W, seq)[-1]
            assert lg[t] >= lg.max() - (1e-4 if dtype == "float32" else 0.15)
            seq.append(t)
    assert lm.model.cache.slots.held == 0
    again = lm.generate(prompts[:2], temperature=0, repeat_penalty=1.0, max_tokens=12)     # on used slots, pages and state
    if dtype == "float32":
        assert [r.tokens for r in again] == [r.tokens for r in got[:2]]


def test_ranks_read_off_the_stored_tensors(tmp_path):
    m = cima_b200.engine.load_model(folder("A", drop_ranks=True), dtype="float32", max_tokens=256, verbose=False)
    toks = random_tokens(CONFIGS["A"]["vocab"], 20, seed=1)
    assert row_errors(run_whole(m, toks), plain_logits("A", toks)).max() < TOL["float32"]
    with pytest.raises(cima_b200.ConfigError):
        with open(os.path.join(folder("A", drop_ranks=True), "config.json")) as f:
            cima_b200.GisiraxConfig.from_dict(json.load(f))


def test_model_from_a_configuration_in_memory_and_its_tensors_by_name():
    lm = cima_b200.load(config=CONFIGS["B"], seed=4, dtype="float32", max_tokens=256, verbose=False)
    sd = {k: v.detach().cpu().double() for k, v in lm.model.state_dict().items()}
    toks = random_tokens(CONFIGS["B"]["vocab"], 20, seed=1)
    assert row_errors(run_whole(lm.model, toks), plain_forward(CONFIGS["B"], sd, toks)).max() < TOL["float32"]


def test_trace_replay_of_this_design(tmp_path):
    name = "A"
    V = CONFIGS[name]["vocab"]
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
