"""The Netezen design on the GPU: each new kernel or kernel option alone against a plain statement of it, then the model in
every cutting (whole, token by token, pieces down to two tokens, unequal batches, reused slots and pages, long decoding),
in 32-bit and in bfloat16, on configurations that differ in every size, and generation through the entry point."""
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
from cima_b200.engine import StepEntry, load_model
from cima_b200.engine.batch import build_batch
from netezen_cases import CONFIGS, carrying_edge, folder, gpu_model, plain_weights, row_errors, variant_folder
from netezen_plain import plain_forward, plain_masked_softmax, read_folder
from reference_kernels import ReferenceKernels
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda:0"
TOL = {"float32": 2e-4, "bfloat16": 6e-2}
_kernels, _models, _plain = [], {}, {}
R = ReferenceKernels()


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


def tol_of(dtype):
    return 2e-5 if dtype == "float32" else 1.2e-2


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,S,W", [(1, 1, 40), (7, 2, 96), (300, 3, 256), (5, 4, 100), (9, 8, 1536), (2, 2, 4100)])
def test_streams_take_an_output_and_are_read(T, S, W, dtype):
    torch.manual_seed(T + S)
    xs, y = torch.randn(T, S, W), torch.randn(T, W)
    C, b, a, w = torch.randn(S, S), torch.randn(S), torch.randn(S), torch.rand(W) + 0.5
    for write, read, spread in ((True, True, False), (True, False, False), (False, True, False), (True, True, True)):
        want_x, want_h = xs.clone(), torch.empty(T, W)
        R.hyper_connect(want_x, y if write else None, C, b, 0.3, a if read else None, w, 1e-5, want_h, spread=spread)
        got_x, got_h = xs.to(DEV), torch.empty(T, W, dtype=DT[dtype], device=DEV)
        K().hyper_connect(got_x, y.to(DEV) if write else None, None if spread else C.to(DEV), None if spread else b.to(DEV), 0.3,
                          a.to(DEV) if read else None, w.to(DEV) if read else None, 1e-5, got_h if read else None, spread=spread)
        assert close(got_x, want_x, 2e-6)
        if read:
            assert close(got_h, want_h, tol_of(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_ungated_activations(dtype):
    torch.manual_seed(1)
    for shape in ((3, 40), (70, 256), (5, 33)):
        z = (torch.randn(*shape) * 3).to(DT[dtype])
        for act in (0, 1, 2, 3, 5):
            want, got = z.clone(), z.to(DEV)
            R.activate(want, act)
            K().activate(got, act)
            assert close(got, want, tol_of(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,heads,K_,N,ha,ho", [(5, 3, 16, 40, 24, 48), (70, 4, 64, 96, 96, 128), (2, 2, 24, 10, 24, 10), (300, 5, 8, 20, 12, 24)])
def test_head_products_on_parts_of_wider_heads(T, heads, K_, N, ha, ho, dtype):
    torch.manual_seed(T)
    a = torch.randn(T, heads * ha + 3).to(DT[dtype])
    w = (torch.randn(heads, N, K_) * K_ ** -0.5).to(DT[dtype])
    want = torch.full((T, heads * ho), 7.0, dtype=DT[dtype])
    got = want.to(DEV)
    R.head_linear(a, w, want, a_head=ha, out_head=ho)
    K().head_linear(a.to(DEV), w.to(DEV), got, a_head=ha, out_head=ho)
    assert close(got, want, tol_of(dtype))                                      # what lies behind a head's N values stays


def _cache(kd, window, planes=1, nkv=1, dtype=torch.float32, tokens=64 * 12):
    return KVCache([[KVRequest(nkv, kd, window, planes)]], tokens, 1 << 20, dtype, DEV, page_size=64, max_seqs=4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("first,rank,rot,interleaved,query_latent", [(32, 40, 8, True, True), (48, 64, 0, False, False), (24, 96, 32, False, True),
                                                                      (20, 10, 6, True, False)])
def test_latents_normed_rotated_and_appended(first, rank, rot, interleaved, query_latent, dtype):
    torch.manual_seed(rank)
    dt = DT[dtype]
    kd = rank + rot
    counts, starts = [5, 70, 1], [0, 60, 130]
    cache_g, cache_r = _cache(kd, 0, dtype=dt), _cache(kd, 0, dtype=dt)
    for c in (cache_g, cache_r):
        slots = c.open(3)
        for s, n, st in zip(slots, counts, starts):
            c.reserve(s, st + n)
        c.flush()
    batch = entries_batch(counts, starts, slots)
    T = sum(counts)
    ql = torch.randn(T, first + kd + 5).to(dt)
    qn, cn = torch.rand(first) + 0.5, torch.rand(rank) + 0.5
    inv = torch.tensor([100.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32)
    H = 2
    for step in (False, True):
        cq_w, cq_g = torch.empty(T, first, dtype=dt), torch.empty(T, first, dtype=dt, device=DEV)
        sr_w, sr_g = torch.zeros(T, (H + 2) * kd, dtype=dt), torch.zeros(T, (H + 2) * kd, dtype=dt, device=DEV)
        cpu_batch = type("B", (), {k: getattr(batch, k).cpu() for k in ("row_pos", "row_seq", "seq_slot", "seq_len")})
        kv_r = cache_r.layer_kv(0)
        kv_cpu = type("KV", (), dict(storage=kv_r.storage.cpu(), block_table=kv_r.block_table.cpu(), page_size=64, ring_pages=0))
        R.latent_prepare(ql, first, qn if query_latent else None, cq_w if query_latent else None, cn, 1e-5, rank, rot, inv, 1.1, interleaved,
                         kv_cpu, cpu_batch, step_rows=(sr_w, H * kd) if step else None)
        K().latent_prepare(ql.to(DEV), first, qn.to(DEV) if query_latent else None, cq_g if query_latent else None, cn.to(DEV), 1e-5, rank, rot,
                           inv.to(DEV) if rot else None, 1.1, interleaved, cache_g.layer_kv(0), batch, step_rows=(sr_g, H * kd) if step else None)
        if query_latent:
            assert close(cq_g, cq_w, tol_of(dtype))
        assert close(sr_g, sr_w, tol_of(dtype))
        for s, n, st in zip(slots, counts, starts):
            for p in range(st, st + n):
                page = int(cache_g.layer_kv(0).block_table[s, p // 64])
                assert close(cache_g.layer_kv(0).storage[page, 0, 0, p % 64], kv_cpu.storage[page, 0, 0, p % 64], tol_of(dtype)), p
    # the queries' rotating parts, into heads of another width
    q = torch.randn(T, H * (first + rot) + 1).to(dt)
    if rot:
        want, got = torch.zeros(T, H * kd, dtype=dt), torch.zeros(T, H * kd, dtype=dt, device=DEV)
        R.rope_rows(q, first, first + rot, want, rank, kd, H, rot, inv, 1.1, interleaved, batch.row_pos.cpu())
        K().rope_rows(q.to(DEV), first, first + rot, got, rank, kd, H, rot, inv.to(DEV), 1.1, interleaved, batch.row_pos)
        assert close(got, want, tol_of(dtype))


def _sink_attention(q, c, scale, window, sinks, first_pos):
    """q [T, H, kd], c [P, kd] (one shared key = value head), query t at position first_pos + t."""
    T, H, kd = q.shape
    out = torch.zeros(T, H, kd, dtype=torch.float64)
    for t in range(T):
        i = first_pos + t
        js = [j for j in range(c.shape[0]) if j <= i and (window <= 0 or i - j < window)]
        for h in range(H):
            s = c[js].double() @ q[t, h].double() * scale
            m = max(float(s.max()), float(sinks[h]))
            e = torch.exp(s - m)
            out[t, h] = (e / (e.sum() + math.exp(float(sinks[h]) - m))) @ c[js].double()
    return out.reshape(T, H * kd)


@pytest.mark.parametrize("dtype,kd,H,window", [("float32", 48, 3, 33), ("bfloat16", 48, 3, 33), ("bfloat16", 64, 4, 70), ("bfloat16", 128, 4, 130),
                                               ("bfloat16", 104, 2, 40), ("bfloat16", 96, 16, 0), ("float32", 128, 2, 64)])
def test_a_number_a_head_in_the_softmax_through_every_attention_kernel(dtype, kd, H, window):
    """One shared plane of keys = values, a window, and exp(sink_h) in head h's denominator: a prompt over its own rows (the
    plain, the tiled and, from 256 rows on, the tcgen05 kernel), rows that go on over the pages, and single rows with
    one and with several splits."""
    torch.manual_seed(kd + H)
    dt = DT[dtype]
    tol = 3e-5 if dtype == "float32" else 2.5e-2
    sinks = torch.randn(H) * 2.0
    total, scale = 420, 0.35
    c = (torch.randn(total, kd) * 0.7).to(dt)
    q = (torch.randn(total, H, kd) * 0.7).to(dt)
    want = _sink_attention(q.float(), c.float(), scale, window, sinks, 0)
    cache = _cache(kd, window, dtype=dt, tokens=64 * 16)
    (slot,) = cache.open(1)
    kv = cache.layer_kv(0)

    def put(lo, hi):
        cache.reserve(slot, hi); cache.flush()
        for p in range(lo, hi):
            e = (p // 64) % kv.ring_pages if kv.ring_pages else p // 64
            kv.storage[int(kv.block_table[slot, e]), 0, 0, p % 64] = c[p].to(DEV)
        cache.commit(slot, hi)

    # a prompt that starts: keys and values from the step's own rows
    for n in (300, 70):
        rows = torch.cat([q[:n].reshape(n, H * kd), c[:n], c[:n]], dim=1).to(DEV)
        out = torch.empty(n, H * kd, dtype=dt, device=DEV)
        K().attention(rows, kv, entries_batch([n], [0], [slot]), out, H, 1, kd, scale, window, False, head_sink=sinks.to(DEV))
        assert close(out, want[:n], tol), ("own rows", n)
    # rows that go on over the pages: 40 rows, then single rows (short context, then with splits)
    put(0, 200)
    put(200, 240)
    out = torch.empty(40, H * kd, dtype=dt, device=DEV)
    K().attention(q[200:240].reshape(40, H * kd).to(DEV), kv, entries_batch([40], [200], [slot]), out, H, 1, kd, scale, window, True,
                  head_sink=sinks.to(DEV))
    assert close(out, want[200:240], tol), "going on"
    for p in range(240, 246):
        put(p, p + 1)
        out = torch.empty(1, H * kd, dtype=dt, device=DEV)
        K().attention(q[p:p + 1].reshape(1, H * kd).to(DEV), kv, entries_batch([1], [p], [slot]), out, H, 1, kd, scale, window, True,
                      head_sink=sinks.to(DEV))
        assert close(out, want[p:p + 1], tol), ("one row", p)
    if dtype == "bfloat16" and kd % 16 == 0:
        put(246, 420)
        b = entries_batch([1], [419], [slot])
        for splits in (1, 2, 5):
            out = torch.empty(1, H * kd, dtype=dt, device=DEV)
            K().attention_decode(q[419:420].reshape(1, H * kd).to(DEV), kv, b.seq_slot, b.seq_len, out, H, 1, kd, scale, window,
                                 n_splits=splits, head_sink=sinks.to(DEV))
            assert close(out, want[419:420], tol), ("splits", splits)
        if kd in (64, 128):                     # 300 rows that go on from the pages: the tcgen05 kernel over one plane
            cache2 = _cache(kd, 0, dtype=dt, tokens=64 * 16)
            (s2,) = cache2.open(1)
            cache2.reserve(s2, 420); cache2.flush()
            kv2 = cache2.layer_kv(0)
            for p in range(420):
                kv2.storage[int(kv2.block_table[s2, p // 64]), 0, 0, p % 64] = c[p].to(DEV)
            cache2.commit(s2, 420)
            out = torch.empty(300, H * kd, dtype=dt, device=DEV)
            K().attention(q[120:420].reshape(300, H * kd).to(DEV), kv2, entries_batch([300], [120], [s2]), out, H, 1, kd, scale, window, True,
                          head_sink=sinks.to(DEV))
            assert close(out, want[120:420], tol), "tcgen05 over the pages"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotation_with_an_amplitude(dtype):
    torch.manual_seed(5)
    dt = DT[dtype]
    nh, nkv, hd, rot = 4, 2, 32, 16
    cache = _cache(hd, 0, planes=2, nkv=nkv, dtype=dt)
    slots = cache.open(2)
    counts, starts = [9, 1], [0, 77]
    for s, n, st in zip(slots, counts, starts):
        cache.reserve(s, st + n)
    cache.flush()
    batch = entries_batch(counts, starts, slots)
    qkv = torch.randn(10, (nh + 2 * nkv) * hd).to(dt)
    inv = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32)
    want, got = qkv.clone(), qkv.to(DEV)
    R.rope_append(want, inv, rot, batch.row_pos.cpu(), batch.row_seq.cpu(), batch.seq_slot.cpu(), batch.seq_len.cpu(), None, nh, nkv, hd, amplitude=1.25)
    K().rope_append(got, inv.to(DEV), rot, batch.row_pos, batch.row_seq, batch.seq_slot, batch.seq_len, cache.layer_kv(0), nh, nkv, hd, amplitude=1.25)
    assert close(got, want, tol_of(dtype))
    kv = cache.layer_kv(0)
    page = int(kv.block_table[slots[1], 1])
    assert close(kv.storage[page, 0, :, 77 % 64].reshape(-1), want[9, nh * hd:(nh + nkv) * hd], tol_of(dtype))


@pytest.mark.parametrize("T,E,top,extra", [(5, 6, 2, 1), (70, 12, 3, 1), (3, 1, 1, 0), (300, 200, 8, 1), (9, 7, 7, 0)])
def test_routing_by_softmax_with_a_correction(T, E, top, extra):
    torch.manual_seed(E)
    scores = torch.randn(T, E + extra) * 2
    corr = torch.randn(E) * 0.2
    wi, ww = torch.empty(T, top, dtype=torch.int32), torch.empty(T, top)
    R.moe_route(scores.clone(), top, 1, 1, 1.0, wi, ww, experts=E, softmax=True, correction=corr)
    for order in (False, True):
        gi, gw = torch.empty(T, top, dtype=torch.int32, device=DEV), torch.empty(T, top, device=DEV)
        sc = scores.to(DEV)
        K().moe_route(sc, top, 1, 1, 1.0, gi, gw, order=order and T <= 64, experts=E, softmax=True, correction=corr.to(DEV))
        assert torch.equal(gi.cpu().sort(dim=1).values, wi.sort(dim=1).values)
        pick = torch.zeros(T, E).scatter_(1, wi.long(), ww)
        assert close(torch.zeros(T, E).scatter_(1, gi.cpu().long(), gw.cpu()), pick, 1e-5)
        if extra:
            assert torch.equal(sc[:, E:].cpu(), scores[:, E:])                      # the column behind the experts is left alone
    # the correction chooses, the softmax weighs
    s = torch.softmax(scores[:, :E], dim=1)
    assert close(ww.sum(1), torch.ones(T), 1e-5)
    t = 0
    assert close(ww[t], s[t, wi[t].long()] / s[t, wi[t].long()].sum(), 1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,ff,H", [(4, 6, 2, 32, 96), (40, 5, 1, 24, 64), (100, 6, 2, 40, 72), (600, 8, 3, 64, 256)])
def test_clamped_experts_on_every_road(T, E, top, ff, H, dtype):
    torch.manual_seed(T)
    dt = DT[dtype]
    h = torch.randn(T, H).to(dt)
    gu, dn = (torch.randn(E, 2 * ff, H) * 0.3).to(dt), (torch.randn(E, H, ff) * 0.2).to(dt)
    idx = torch.stack([torch.randperm(E)[:top] for _ in range(T)]).to(torch.int32)
    wgt = torch.rand(T, top)
    want = torch.zeros(T, H)
    R.moe_experts(h, gu, dn, idx, wgt, want, 4, assign=True, limit=1.5)
    got = torch.full((T, H), 3.0, device=DEV)
    K().moe_experts(h.to(DEV), gu.to(DEV), dn.to(DEV), idx.to(DEV), wgt.to(DEV), got, 4, assign=True, limit=1.5)
    assert close(got, want, 3e-5 if dtype == "float32" else 2.5e-2)
    # a shared expert's rows, gated by a column of a wider matrix or not at all, join the sum in the same launch
    rows, gate = torch.randn(T, H), torch.randn(T, E + 1)
    for g_ in (gate, None):
        want2 = want + (torch.sigmoid(gate[:, E:E + 1]) if g_ is not None else 1.0) * rows
        got = torch.full((T, H), 3.0, device=DEV)
        K().moe_experts(h.to(DEV), gu.to(DEV), dn.to(DEV), idx.to(DEV), wgt.to(DEV), got, 4, assign=True, limit=1.5,
                        shared=(rows.to(DEV), g_.to(DEV) if g_ is not None else None, E))
        assert close(got, want2, 3e-5 if dtype == "float32" else 2.5e-2)


# ------------------------------------------------------------------------------------------- the model
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
        # in bfloat16 a row whose router scores two experts nearly alike may take the other one; such rows are rare and
        # the 32-bit runs compare every row sharply
        over = int((e >= 3 * TOL[dtype]).sum())
        assert e.median() < TOL[dtype] / 2 and over <= max(1, len(e) // 50) and e.max() < 0.6, (what, float(e.median()), float(e.max()), over)


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
def test_unequal_batches_on_reused_slots_and_pages(name, dtype):
    """Three rounds on a cache of three slots and few pages: later sequences get the slots and the pages (rings included) of
    earlier ones; shorter requests end earlier."""
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


@pytest.mark.parametrize("layer,key,candidates", [(0, "size", range(5, 40)), (0, "keep_first", range(1, 8)), (1, "size", range(5, 50)),
                                                  (3, "size", range(60, 70))])
def test_a_key_that_carries_a_row_just_inside_and_just_outside_a_mask(layer, key, candidates):
    """The mask constant is set so that the key which carries the last row is the last one still seen, then the first one
    not seen any more; whole prompts, portions and decoded tokens follow the plain implementation on both sides."""
    cfg, W = plain_weights("A")
    toks = random_tokens(cfg["vocab"], 140, seed=12)
    v, jump = carrying_edge(cfg, W, toks, layer, key, list(candidates))
    assert jump > 0.05, "no key of this layer carries the last row"
    for value in (v, v - 1):
        d = variant_folder("A", lambda c: c["layers"][layer]["mixer"]["mask"].__setitem__(key, value))
        cfg2, W2 = read_folder(d)
        want = plain_forward(cfg2, W2, toks)
        m = load_model(d, dtype="float32", max_tokens=1024, device=DEV, verbose=False)
        assert row_errors(run_whole(m, toks), want).max() < TOL["float32"]
        assert row_errors(run_tail_one_by_one(m, toks, 8), want).max() < TOL["float32"]
        assert row_errors(run_in_pieces(m, [toks], [[66, 130, 138]])[0], want).max() < TOL["float32"]


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
    assert e.max() < (1e-5 if dtype == "float32" else 6e-2), float(e.max())


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
            assert lg[t] >= lg.max() - (1e-4 if dtype == "float32" else 0.3)
            seq.append(t)
    assert lm.model.cache.slots.held == 0
    again = lm.generate(prompts[:2], temperature=0, repeat_penalty=1.0, max_tokens=12)     # on used slots and pages
    if dtype == "float32":
        assert [r.tokens for r in again] == [r.tokens for r in got[:2]]


def test_model_from_a_configuration_in_memory_and_its_tensors_by_name():
    lm = cima_b200.load(config=CONFIGS["A"], seed=4, dtype="float32", max_tokens=256, verbose=False)
    sd = {k: v.detach().cpu().double() for k, v in lm.model.state_dict().items()}
    toks = random_tokens(CONFIGS["A"]["vocab"], 20, seed=1)
    assert row_errors(run_whole(lm.model, toks), plain_forward(CONFIGS["A"], sd, toks)).max() < TOL["float32"]


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
    got = torch.from_numpy(np.fromfile(tmp_path / "4.f32", dtype="<f4").reshape(-1, V).copy())
    assert row_errors(got, torch.stack([wa[69], wb[8]])).max() < TOL["float32"]
