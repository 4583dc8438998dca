"""The Lipizen design on the GPU: each new kernel or kernel option alone against a plain statement of it, then the model in
every cutting (whole, token by token, pieces down to two tokens, unequal batches, reused slots, pages and state, long
decoding), in 32-bit and in bfloat16, on configurations that differ in every size, and generation through the entry point."""
import json
import math
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
from lipizen_cases import CONFIGS, folder, gpu_model, plain_weights, row_errors
from lipizen_plain import plain_diff_attention, plain_forward, plain_rms, plain_rotate, plain_visible
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole

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


def entries_batch(counts, starts, slots=None, device=DEV):
    slots = slots or list(range(len(counts)))
    return build_batch([StepEntry(s, [0] * c, []) for s, c in zip(slots, counts)], starts, 1 << 30, device)


def close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,W,groups", [(1, 40, 1), (7, 96, 3), (300, 256, 2), (5, 100, 4), (33, 1536, 6), (2, 4100, 2)])
def test_scaled_sum_and_norm_in_groups(T, W, groups, dtype):
    g = torch.Generator().manual_seed(T + W)
    x, y, w = torch.randn(T, W, generator=g) * 3, torch.randn(T, W, generator=g) * 2, torch.randn(W, generator=g)
    x[0, :W // groups] *= 1e-4                                                  # a part whose mean square is near eps
    for with_y in (True, False):
        xd, h = x.to(DEV).clone(), torch.empty(T, W, dtype=DT[dtype], device=DEV)
        K().scale_add_group_rmsnorm(xd, y.to(DEV) if with_y else None, 1.7, w.to(DEV), groups, 1e-5, h)
        z = (1.7 * x.double() + (y.double() if with_y else 0)).view(T, groups, W // groups)
        want = (z / torch.sqrt((z * z).mean(-1, keepdim=True) + 1e-5)).view(T, W) * w.double()
        assert close(xd, want, 2e-6)                                            # the stream stays float32
        assert close(h, want, 2e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,heads,rep,hd,vdim", [(5, 4, 1, 96, 96), (9, 4, 2, 32, 24), (70, 8, 8, 128, 128), (3, 3, 1, 64, 8), (2, 2, 2, 16, 1)])
def test_difference_of_the_maps_norm_and_gate(T, heads, rep, hd, vdim, dtype):
    g = torch.Generator().manual_seed(T * heads)
    kv = heads // rep
    a = torch.randn(T, kv, 2, rep, hd, generator=g).to(DT[dtype])              # per key head: map 1 of its heads, then map 2
    gate = torch.randn(T, heads + 3, generator=g).to(DT[dtype])
    lam, post, eps = 0.83, 0.4, 1e-5
    for gated in (True, False):
        out = torch.empty(T, heads * vdim, dtype=DT[dtype], device=DEV)
        K().diff_combine(a.view(T, -1).to(DEV), gate.to(DEV)[:, :heads] if gated else None, out, heads, rep, hd, vdim, lam, post, eps)
        o = (a[:, :, 0].double() - lam * a[:, :, 1].double())[..., :vdim].reshape(T, heads, vdim)
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * post
        if gated:
            o = o * torch.sigmoid(gate[:, :heads].double())[:, :, None]
        assert close(out, o.view(T, -1), 2e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_gated_middle_and_soft_cap(dtype):
    g = torch.Generator().manual_seed(1)
    T, ff = 13, 88
    gu = (torch.randn(T, 2 * ff, generator=g) * 3).to(DT[dtype])
    from cima_b200.kernels import ACTIVATIONS
    for limit in (0.5, 1.0, 7.0):
        out = torch.empty(T, ff, dtype=DT[dtype], device=DEV)
        K().swiglu(gu.to(DEV), out, ACTIVATIONS["swish_clamped"], limit)
        a, u = gu[:, :ff].double().clamp(max=limit), gu[:, ff:].double().clamp(-limit, limit)
        assert close(out, a * torch.sigmoid(1.702 * a) * (u + 1), 2e-6 if dtype == "float32" else 1e-2)
    lg = (torch.randn(5, 300, generator=g) * 40).to(DEV)
    want = 30.0 * torch.tanh(lg.double() / 30.0)
    K().softcap(lg, 30.0)
    assert close(lg, want, 2e-6) and float(lg.abs().max()) <= 30.0


def _gate_rule(q, f, v, bias, lower, heads, dim, vdim):
    """One sequence through S <- diag(f) S + (1 - f) v^T, o = S^T silu(q) in float64; returns (o, S)."""
    n = q.shape[0]
    q, f, v = q.double().view(n, heads, dim), f.double().view(n, heads, dim), v.double().view(n, heads, vdim)
    q = q * torch.sigmoid(q)
    low = lower.double().view(heads, dim)
    f = low + (1 - low) * torch.sigmoid(f + bias.double().view(heads, dim))
    S = torch.zeros(heads, dim, vdim, dtype=torch.float64)
    out = []
    for t in range(n):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1))
    return torch.stack(out), S


def _gate_case(heads, dim, vdim, dtype, counts_per_step, seed):
    g = torch.Generator().manual_seed(seed)
    n_seqs = len(counts_per_step[0])
    lens = [sum(step[i] for step in counts_per_step) for i in range(n_seqs)]
    bias, lower = torch.randn(heads * dim, generator=g), torch.rand(heads * dim, generator=g) * 0.95
    lower[0] = 0.0
    data = [tuple(torch.randn(n, c, generator=g).to(DT[dtype]) * s for c, s in ((heads * dim, 1.0), (heads * dim, 3.0), (heads * vdim, 1.0)))
            for n in lens]
    slots = [5, 1, 3, 0][:n_seqs]
    state = torch.randn(7, heads, dim, vdim, generator=g).to(DEV)
    state[slots] = 0
    wants = [_gate_rule(q, f, v, bias, lower, heads, dim, vdim) for q, f, v in data]
    got, pos = [[] for _ in lens], [0] * n_seqs
    qd = heads * dim
    for counts in counts_per_step:
        live = [i for i, c in enumerate(counts) if c > 0]
        b = entries_batch([counts[i] for i in live], [pos[i] for i in live], [slots[i] for i in live])
        wide = torch.cat([torch.cat([data[i][j][pos[i]:pos[i] + counts[i]] for j in range(3)], dim=1) for i in live]).to(DEV)
        o = torch.empty(b.n_rows, heads * vdim, dtype=torch.float32, device=DEV)
        K().recurrence(wide[:, :qd], wide[:, qd:2 * qd], wide[:, 2 * qd:], state, b, o, heads, heads, dim, vdim,
                       gate=(bias.to(DEV), lower.to(DEV)))
        r = 0
        for i in live:
            got[i].append(o[r:r + counts[i]].cpu()); r += counts[i]
            pos[i] += counts[i]
    for gi, (wo, _) in zip(got, wants):
        assert close(torch.cat(gi), wo, 3e-5)
    assert close(state[slots], torch.stack([s for _, s in wants]), 3e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 24), (3, 40, 8), (2, 128, 64), (1, 8, 100), (2, 200, 16), (4, 48, 32), (5, 24, 1)])
def test_gate_rule_whole_in_pieces_and_token_by_token(heads, dim, vdim, dtype):
    _gate_case(heads, dim, vdim, dtype, [[20, 3, 9], [2, 2, 2], [1, 1, 1], [1, 0, 1], [17, 0, 1]], seed=dim + vdim)


def test_gate_rule_long_decoding_holds_its_state():
    _gate_case(2, 32, 32, "float32", [[3, 1]] + [[1, 1]] * 150, seed=5)
    _gate_case(2, 32, 32, "bfloat16", [[3, 1]] + [[1, 1]] * 150, seed=6)


def _maps(q, k, v, scale, window, keep, first_pos, v_group):
    """q [n, nq, D], k [len, nk, D], v [len, nk / v_group, D]: every query head's softmax over the keys it may see."""
    n, nq, D = q.shape
    share = nq // k.shape[1]
    out = torch.zeros(n, nq, D, dtype=torch.float64)
    L = k.shape[0]
    for i in range(n):
        p = first_pos + i
        seen = torch.tensor([plain_visible(p, j, window, keep) for j in range(L)])
        for h in range(nq):
            kh = h // share
            s = (k[:, kh].double() @ q[i, h].double()) * scale
            s = s.masked_fill(~seen, float("-inf"))
            out[i, h] = torch.softmax(s, dim=0) @ v[:, kh // v_group].double()
    return out.view(n, nq * D)


@pytest.mark.parametrize("dtype,D,nq,nk,window,keep", [("float32", 48, 8, 4, 70, 5), ("bfloat16", 48, 8, 4, 70, 5), ("bfloat16", 96, 8, 8, 96, 6),
                                                       ("bfloat16", 64, 8, 2, 64, 70), ("bfloat16", 128, 4, 2, 130, 1), ("float32", 16, 6, 6, 1, 1),
                                                       ("bfloat16", 32, 4, 4, 200, 0), ("bfloat16", 16, 4, 2, 3, 64)])
def test_windows_with_kept_first_positions_through_every_kernel(dtype, D, nq, nk, window, keep):
    """Pairs of key heads on one value head, sequences of 1 to 400 positions through prompts (the step's own keys), pieces
    that go on from the cache and single tokens.  In every sequence queries are made so that a single key would carry their row:
    the last one inside the window and the first outside it, the last kept position and the one behind it, a page's border."""
    g = torch.Generator().manual_seed(D + nq + window)
    lens = [1, 63, 65, 129, 400]
    scale, nv = 0.3, nk // 2
    cache = KVCache([[KVRequest(nk, D, 0)]], max_tokens=64 * 16, max_position=4096, dtype=DT[dtype], device=DEV)
    slots = cache.open(len(lens))
    qs = [torch.randn(n, nq, D, generator=g) for n in lens]
    ks = [torch.randn(n, nk, D, generator=g) for n in lens]
    vs = [torch.randn(n, nv, D, generator=g) for n in lens]
    for q, k, n in zip(qs, ks, lens):
        rows = sorted({n - 1, n // 2, min(n - 1, 64), min(n - 1, window + keep), min(n - 1, window + keep + 1), max(0, n - 2)})
        for x, row in enumerate(rows):
            keys = [row - window + 1, row - window, keep - 1, keep, 63, 64, 0]      # just inside, just outside, kept, not kept, a border
            for h in range(nq):
                key = keys[(x + h) % len(keys)]
                if 0 <= key <= row:
                    q[row, h] = k[key, h // (nq // nk)] * 3.0                    # about 3 * D * 0.3 against a spread of sqrt(D)
    qs = [q.to(DT[dtype]) for q in qs]; ks = [k.to(DT[dtype]) for k in ks]; vs = [v.to(DT[dtype]) for v in vs]
    wants = [_maps(q.float(), k.float(), v.float(), scale, window, keep, 0, 2) for q, k, v in zip(qs, ks, vs)]
    tol = 2e-5 if dtype == "float32" else 2e-2
    zero = torch.zeros(1, dtype=torch.float32, device=DEV)

    def run(counts, starts, from_cache):
        live = [i for i, c in enumerate(counts) if c > 0]
        b = build_batch([StepEntry(slots[i], [0] * counts[i], []) for i in live], [starts[i] for i in live], 1, DEV)
        for i in live:
            cache.reserve(slots[i], starts[i] + counts[i])
        cache.flush()
        qkv = torch.cat([torch.cat([t[i][starts[i]:starts[i] + counts[i]].reshape(counts[i], -1) for t in (qs, ks, vs)], dim=1)
                         for i in live]).to(DEV).contiguous()
        kvl = cache.layer_kv(0)
        K().rope_append(qkv, zero[:0], 0, b.row_pos, b.row_seq, b.seq_slot, b.seq_len, kvl, nq, nk, D, v_heads=nv)
        out = torch.empty(qkv.shape[0], nq * D, dtype=DT[dtype], device=DEV)
        K().attention(qkv, kvl, b, out, nq, nk, D, scale, window, from_cache, keep_first=keep, v_group=2)
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
    slots = cache.open(len(lens))                                             # whole, on the slots and pages just given back
    run(lens, [0] * 5, False)
    cache.close(slots)
    slots = cache.open(len(lens))                                             # every position decoded alone from the first on
    short = [min(n, 140) for n in lens]
    for t in range(max(short)):
        run([1 if t < n else 0 for n in short], [t] * 5, True)
    cache.close(slots)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,hd,rot,factor", [(48, 96, 24, 4.0), (16, 32, 16, 1.0), (64, 64, 0, 1.0), (24, 32, 8, 2.0), (128, 128, 64, 8.0)])
def test_norm_and_rotation_before_the_pages(dim, hd, rot, factor, dtype):
    """q and k normed over their first ``dim`` values and rotated on their first ``rot`` ones, the values untouched; read back
    through an attention whose window is one position (the output is the newest value) and through one over everything."""
    g = torch.Generator().manual_seed(dim + rot)
    nq, nk, nv, n, eps, scale = 4, 2, 1, 75, 1e-5, 0.25
    q, k, v = torch.randn(n, nq, hd, generator=g) * 2, torch.randn(n, nk, hd, generator=g) * 0.5, torch.randn(n, nv, hd, generator=g)
    q[..., dim:] = 0; k[..., dim:] = 0
    wq, wk = torch.rand(dim, generator=g) + 0.5, torch.rand(dim, generator=g) + 0.5
    q, k, v = q.to(DT[dtype]), k.to(DT[dtype]), v.to(DT[dtype])
    base = 500.0
    inv = torch.tensor([base ** (-2.0 * i / rot) / factor for i in range(rot // 2)], dtype=torch.float32)
    nrm = lambda z, w: plain_rms(z.double()[..., :dim], eps) * w.double()
    qn = plain_rotate(nrm(q, wq), rot, base, factor)
    kn = plain_rotate(nrm(k, wk), rot, base, factor)
    pad = lambda z: torch.cat([z, torch.zeros(*z.shape[:-1], hd - dim, dtype=z.dtype)], dim=-1)
    want = _maps(pad(qn), pad(kn), v.float(), scale, 0, 0, 0, 2)
    cache = KVCache([[KVRequest(nk, hd, 0)]], max_tokens=256, max_position=4096, dtype=DT[dtype], device=DEV)
    (slot,) = cache.open(1)
    outs = []
    for start, count in ((0, 40), (40, 30), (70, 1), (71, 1), (72, 3)):
        b = build_batch([StepEntry(slot, [0] * count, [])], [start], 1, DEV)
        cache.reserve(slot, start + count); cache.flush()
        qkv = torch.cat([t[start:start + count].reshape(count, -1) for t in (q, k, v)], dim=1).to(DEV).contiguous()
        K().rope_append(qkv, inv.to(DEV), rot, b.row_pos, b.row_seq, b.seq_slot, b.seq_len, cache.layer_kv(0), nq, nk, hd, v_heads=nv,
                        qk_norm=(wq.to(DEV), wk.to(DEV), dim, eps))
        out = torch.empty(count, nq * hd, dtype=DT[dtype], device=DEV)
        K().attention(qkv, cache.layer_kv(0), b, out, nq, nk, hd, scale, 0, start > 0, v_group=2)
        cache.commit(slot, start + count)
        outs.append(out.cpu())
    assert close(torch.cat(outs), want, 3e-5 if dtype == "float32" else 3e-2)
    cache.close([slot])


# ------------------------------------------------------------------------------------------- the model
# 32-bit sums through sharp softmaxes and 330 steps of a recurrence round to a few 1e-5 (the stand-ins on the CPU do too); a fault
# shows at 1e-2
TOL = {"float32": 1e-4, "bfloat16": 6e-2}
_models, _plain = {}, {}


def model_of(name, dtype, max_tokens=2048):
    """32-bit on the weights that make attention sharp; bfloat16 on the milder ones of the same configuration."""
    if (name, dtype) not in _models:
        _models[(name, dtype)] = gpu_model(name, dtype, max_tokens=max_tokens, sharp=dtype == "float32")
    return _models[(name, dtype)]


def plain_logits(name, toks, dtype="float32"):
    key = (name, tuple(toks), dtype == "float32")
    if key not in _plain:
        cfg, W = plain_weights(name, sharp=dtype == "float32")
        _plain[key] = plain_forward(cfg, W, toks)
    return _plain[key]


def agrees(got, want, dtype, what=""):
    e = row_errors(got, want)
    if dtype == "float32":
        assert e.max() < TOL[dtype], (what, float(e.max()))
    else:
        # In bfloat16 a single row may be ill-conditioned: at a sequence's first position the recurrence's output per head
        # is its value vector times one sum over the key channels, divided by its own root mean square; where that sum
        # nearly cancels, rounding decides its sign. Such rows are rare; the 32-bit runs compare every row sharply.
        over = int((e >= 3 * TOL[dtype]).sum())
        assert e.median() < TOL[dtype] / 2 and over <= max(1, len(e) // 100) and e.max() < 0.5, \
            (what, float(e.median()), float(e.max()), over)


LENGTHS = {"A": 150, "B": 131, "C": 330}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_and_token_by_token(name, dtype):
    cfg = CONFIGS[name]
    toks = random_tokens(cfg["vocab"], LENGTHS[name], seed=3)
    m = model_of(name, dtype)
    want = plain_logits(name, toks, dtype)
    agrees(run_whole(m, toks), want, dtype, "whole")
    agrees(run_tail_one_by_one(m, toks, 70), want, dtype, "tail")            # across a page's border and the windows' edges
    agrees(run_tail_one_by_one(m, toks[:12], 12), want[:12], dtype, "first tokens")
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
    agrees(got[0], plain_logits(name, a, dtype), dtype)
    agrees(got[1], plain_logits(name, b_, dtype), dtype)
    if dtype == "float32":                                                    # the cutting changes nothing but rounding
        assert row_errors(got[0], run_whole(m, a)).max() < 2e-5
    assert m.cache.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_unequal_batches_on_reused_slots_pages_and_state(name, dtype):
    """Three rounds on a cache of three slots and six pages: later sequences get the slots, the pages, the recurrent state and
    the convolutions' inputs of earlier ones; shorter requests end earlier."""
    cfg = CONFIGS[name]
    m = gpu_model(name, dtype, max_tokens=64 * 6, max_seqs=3, sharp=dtype == "float32")
    for rnd in range(3):
        lens = [[5, 1, 130], [66, 3, 64], [1, 1, 63]][rnd]
        seqs = [random_tokens(cfg["vocab"], n + (2 if i == 1 else 9), seed=10 * rnd + i) for i, n in enumerate(lens)]
        got = run_batched(m, seqs, lens)
        for q, g_ in zip(seqs, got):
            agrees(g_, plain_logits(name, q, dtype), dtype, (rnd, len(q)))
        m.cache.check()
        assert m.cache.slots.held == 0


def test_sharp_maps_rest_on_single_keys_at_the_masks_edges():
    """The test weights do what they are for: in configuration C's first layer (a window of a page, 70 kept positions) many rows
    of a map put most of their weight on one key, among them kept positions far below the window and keys at the window's edge."""
    from lipizen_plain import plain_keys_values
    cfg, W = plain_weights("C")
    toks = random_tokens(cfg["vocab"], LENGTHS["C"], seed=3)
    x = W["embed"][torch.tensor(toks)]
    m = cfg["layers"][0]["mixer"]
    sub = {k[len("l0.mix."):]: v for k, v in W.items() if k.startswith("l0.mix.")}
    k, _ = plain_keys_values(x, sub, m, cfg["norm"]["eps"])
    T, H, dim = len(toks), m["heads"], m["dim"]
    from lipizen_plain import plain_causal_conv
    q = plain_rms(plain_causal_conv(x @ sub["q"].T, sub["q.conv"]).reshape(T, H * 2, dim), cfg["norm"]["eps"]) * sub["q.norm"]
    q = plain_rotate(q, m["rot"]["dims"], m["rot"]["base"], m["rot"]["scaling"]["factor"]).reshape(T, H, 2, dim)
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = (j <= i) & ((i - j < size) | (j < keep))
    far = edge = 0
    for hh in range(H):
        for mm in (0, 1):
            p = torch.softmax((q[:, hh, mm] @ k[:, 0, mm].T * m["scale"]).masked_fill(~ok, float("-inf")), dim=1)
            top, where = p.max(dim=1)
            dist = torch.arange(T) - where
            far += int(((top > 0.5) & (dist >= size)).sum())
            edge += int(((top > 0.3) & (dist >= size - 8) & (dist < size)).sum())
    assert far >= 10 and edge >= 3, (far, edge)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    cfg = CONFIGS["A"]
    toks = random_tokens(cfg["vocab"], 300, seed=9)
    agrees(run_tail_one_by_one(model_of("A", dtype), toks, 297), plain_logits("A", toks, dtype), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_composition_and_slot_do_not_change_a_row(dtype):
    cfg = CONFIGS["C"]
    m = model_of("C", dtype)
    a, others = random_tokens(cfg["vocab"], 140, seed=1), [random_tokens(cfg["vocab"], n, seed=n) for n in (300, 7)]
    alone = run_batched(m, [a], [130])[0]
    among = run_batched(m, [others[0], a, others[1]], [290, 130, 3])[1]
    e = row_errors(among, alone)
    assert e.max() < (1e-5 if dtype == "float32" else 3e-2), float(e.max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype):
    name = "B"
    cfg, W = plain_weights(name, sharp=dtype == "float32")
    lm = cima_b200.load(folder(name, sharp=dtype == "float32"), dtype=dtype, max_tokens=1024, verbose=False)
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
