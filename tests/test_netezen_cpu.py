"""The Netezen decoder without a GPU: its configuration, the plain implementation's mechanisms against other statements
of the same mathematics, and the package's host logic (cache, pages, steps, generation) on the CPU stand-in kernels
against the plain implementation."""
import copy
import math

import pytest
import torch

import cima_b200
from cima_b200.config import ConfigError, NetezenConfig, lookup_architecture
from cima_b200.engine import StepEntry, build_plan
from netezen_cases import CONFIGS, N_A, N_B, N_C, cpu_model, plain_weights, row_errors
from netezen_plain import (plain_attention, plain_dense_ff, plain_expert, plain_forward, plain_frequencies, plain_latent_attention,
                           plain_masked_softmax, plain_moe, plain_rms, plain_rotate, plain_route, plain_visible)
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole

TOL = 2e-4
D = torch.float64


# ------------------------------------------------------------------------------------------- configuration
def test_configuration_round_trip_and_plan():
    for cfg in CONFIGS.values():
        entry = lookup_architecture(cfg)
        typed = entry.parse(cfg)
        assert isinstance(typed, NetezenConfig)
        assert NetezenConfig.from_dict(typed.to_dict()) == typed
        plan = build_plan(entry.spec(typed))
        assert "embed" in plan and "final.norm" in plan and "head" not in plan          # the table is the head
    plan = build_plan(NetezenConfig.from_dict(N_A).model_spec())
    assert plan["l0.hc1.mix"].shape == (3, 3) and plan["l0.hc2.in"].shape == (3,) and plan["l2.hc1.out"].shape == (3,)
    assert "l2.hc2.in" not in plan and "l2.norm2" not in plan                          # a layer without feed-forward
    assert plan["l0.mix.k"].shape == (2 * 24, 96) and plan["l0.mix.v"].shape == (2 * 16, 96) and plan["l0.mix.o"].shape == (96, 4 * 16)
    assert plan["l1.mix.dq"].shape == (32, 96) and plan["l1.mix.uq"].shape == (3 * (16 + 8), 32) and plan["l1.mix.dkv"].shape == (40 + 8, 96)
    assert plan["l1.mix.dkv.norm"].shape == (40,) and plan["l1.mix.uk"].shape == (3 * 16, 40) and plan["l1.mix.uv"].shape == (3 * 24, 40)
    assert plan["l1.mix.sink"].shape == (3,) and plan["l1.mlp.up"].shape == (72, 96)
    assert plan["l0.mlp.router"].shape == (6, 96) and plan["l0.mlp.correction"].shape == (6,) and plan["l0.mlp.e5.down"].shape == (96, 32)
    assert plan["l0.mlp.shared.sg"].shape == (1, 96) and plan["l0.mlp.shared.gate"].shape == (40, 96) and "l3.mlp.shared.up" not in plan
    assert not any(".hc" in n for n in build_plan(NetezenConfig.from_dict(N_C).model_spec()))   # no streams: nothing stored
    assert "l0.hc1.mix" in build_plan(NetezenConfig.from_dict(N_B).model_spec())               # one stream with its connection


def test_what_is_stored_is_read_off_the_tensor_names():
    typed = NetezenConfig.from_dict(N_A, shapes={"l0.norm1": (96,)})
    assert not typed.learned_streams and not typed.layers[1].latent.sink and not typed.layers[0].moe.correction
    typed = NetezenConfig.from_dict(N_C, shapes={"l0.hc1.in": (1,), "l1.mix.sink": (4,), "l1.mlp.correction": (8,)})
    assert typed.learned_streams and typed.layers[1].latent.sink and typed.layers[1].moe.correction and not typed.layers[3].latent.sink


@pytest.mark.parametrize("change,word", [
    (lambda c: c.update(architecture="Other"), "architecture"),
    (lambda c: c.update(streams=9), "streams"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.0), "scaling"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
])
def test_configuration_refuses(change, word):
    cfg = copy.deepcopy(N_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        NetezenConfig.from_dict(cfg)
    assert word in str(e.value)


# ------------------------------------------------------------------------------------------- the plain mechanisms
def test_plain_rotation_turns_neighbours_keeps_the_rest_and_depends_on_the_distance_only():
    torch.manual_seed(0)
    rot = {"dims": 8, "base": 100.0}
    q, k = torch.randn(12, 2, 12, dtype=D), torch.randn(12, 2, 12, dtype=D)
    rq, rk = plain_rotate(q, rot), plain_rotate(k, rot)
    assert torch.equal(rq[..., 8:], q[..., 8:])
    assert torch.allclose(rq[0], q[0])                                                   # position 0 turns nothing
    # pair (2, 3) at position 5 by the angle 5 * 100^(-2/8), written out
    a = 5 * 100.0 ** (-2.0 / 8)
    assert torch.allclose(rq[5, 1, 2], q[5, 1, 2] * math.cos(a) - q[5, 1, 3] * math.sin(a))
    assert torch.allclose(rq[5, 1, 3], q[5, 1, 3] * math.cos(a) + q[5, 1, 2] * math.sin(a))
    same = torch.randn(1, 2, 12, dtype=D).expand(12, 2, 12).clone()
    s = torch.einsum("thd,uhd->htu", plain_rotate(same, rot), plain_rotate(same, rot))
    assert torch.allclose(s[:, 3, 1], s[:, 9, 7]) and torch.allclose(s[:, 4, 4], s[:, 0, 0])
    assert torch.allclose(plain_rotate(q[3:], rot, first_position=3), rq[3:])
    assert torch.allclose((rq * rq).sum(-1), (q * q).sum(-1))                            # a rotation of amplitude 1


def test_plain_rescaled_frequencies_blend_by_index_and_stretch_the_amplitude():
    rot = {"dims": 16, "base": 10000.0, "scaling": {"factor": 4.0, "original": 128, "fast": 8.0, "slow": 1.0}}
    f, amp = plain_frequencies(rot)
    plain = torch.tensor([10000.0 ** (-i / 8.0) for i in range(8)], dtype=D)
    d = lambda z: 16 * math.log(128 / (2 * math.pi * z)) / (2 * math.log(10000.0))
    lo, hi = max(math.floor(d(8.0)), 0), min(math.ceil(d(1.0)), 15)
    assert (lo, hi) == (0, 3)
    for i in range(8):
        g = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(float(f[i]) - float(plain[i]) * (g / 4.0 + 1.0 - g)) < 1e-15
    assert float(f[0]) == 1.0 and abs(float(f[7]) - float(plain[7]) / 4.0) < 1e-18    # fast pairs stay, slow ones are stretched
    assert abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    x = torch.randn(3, 1, 16, dtype=D)
    assert torch.allclose((plain_rotate(x, rot) ** 2).sum(-1), amp * amp * (x * x).sum(-1))
    assert plain_frequencies({"dims": 16, "base": 10000.0})[1] == 1.0


def test_plain_mask_window_and_kept_first_positions():
    assert plain_visible(10, 10, 4, 0) and plain_visible(10, 7, 4, 0) and not plain_visible(10, 6, 4, 0)
    assert not plain_visible(10, 11, 4, 0) and plain_visible(10, 0, 0, 0)
    assert plain_visible(10, 1, 4, 2) and not plain_visible(10, 2, 4, 2) and plain_visible(3, 0, 4, 2)
    s = torch.zeros(6, 6, dtype=D)
    p = plain_masked_softmax(s, 2, 1)
    assert torch.allclose(p[5], torch.tensor([1 / 3, 0, 0, 0, 1 / 3, 1 / 3], dtype=D)) and torch.allclose(p[1], torch.tensor([.5, .5, 0, 0, 0, 0], dtype=D))
    # a sink is one more column of the softmax that carries nothing
    torch.manual_seed(1)
    s = torch.randn(5, 5, dtype=D)
    sink = torch.tensor(0.7, dtype=D)
    p = plain_masked_softmax(s, 0, 0, sink)
    for i in range(5):
        full = torch.softmax(torch.cat([s[i, :i + 1], sink[None]]), 0)
        assert torch.allclose(p[i, :i + 1], full[:-1]) and float(p[i].sum()) < 1.0


def test_plain_grouped_attention_written_out_for_one_row():
    torch.manual_seed(2)
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 3, "scale": 0.4, "rot": {"dims": 4, "base": 50.0}, "mask": {"size": 3, "keep_first": 1}}
    W = {"q": torch.randn(24, 10, dtype=D), "k": torch.randn(12, 10, dtype=D), "v": torch.randn(6, 10, dtype=D), "o": torch.randn(10, 12, dtype=D)}
    h = torch.randn(7, 10, dtype=D)
    got = plain_attention(h, W, m)
    i, rows = 6, []
    q = plain_rotate((h @ W["q"].T).reshape(7, 4, 6), m["rot"])
    k = plain_rotate((h @ W["k"].T).reshape(7, 2, 6), m["rot"])
    v = (h @ W["v"].T).reshape(7, 2, 3)
    for a in range(4):
        js = [0, 4, 5, 6]                                                                 # the kept first position, then the window
        w = torch.softmax(torch.stack([q[i, a] @ k[j, a // 2] * 0.4 for j in js]), 0)
        rows.append(sum(w[n] * v[j, a // 2] for n, j in enumerate(js)))
    assert torch.allclose(got[i], torch.cat(rows) @ W["o"].T)


def test_plain_latent_attention_equals_attention_over_the_moved_queries():
    """q . (W_uk c) = (W_uk^T q) . c and sum p (W_uv c) = W_uv sum p c: the form the package computes."""
    torch.manual_seed(3)
    m = {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 8, "q_rank": 7, "scale": 0.3, "rot": {"dims": 4, "base": 30.0}, "mask": {"size": 4}}
    W = {"dq": torch.randn(7, 10, dtype=D), "dq.norm": torch.rand(7, dtype=D) + 0.5, "uq": torch.randn(20, 7, dtype=D),
         "dkv": torch.randn(12, 10, dtype=D), "dkv.norm": torch.rand(8, dtype=D) + 0.5, "uk": torch.randn(12, 8, dtype=D),
         "uv": torch.randn(10, 8, dtype=D), "sink": torch.tensor([0.3, -1.0], dtype=D), "o": torch.randn(10, 10, dtype=D)}
    h = torch.randn(9, 10, dtype=D)
    got = plain_latent_attention(h, W, m, 1e-6)
    cq = plain_rms(h @ W["dq"].T, 1e-6) * W["dq.norm"]
    q = (cq @ W["uq"].T).reshape(9, 2, 10)
    both = h @ W["dkv"].T
    c = plain_rms(both[:, :8], 1e-6) * W["dkv.norm"]
    kr = plain_rotate(both[:, 8:].reshape(9, 1, 4), m["rot"])[:, 0]
    qr = plain_rotate(q[:, :, 6:], m["rot"])
    out = torch.zeros(9, 2, 5, dtype=D)
    for a in range(2):
        moved = q[:, a, :6] @ W["uk"][a * 6:(a + 1) * 6]                                  # [T, kv_rank]
        s = (moved @ c.T + qr[:, a] @ kr.T) * 0.3
        out[:, a] = (plain_masked_softmax(s, 4, 0, W["sink"][a]) @ c) @ W["uv"][a * 5:(a + 1) * 5].T
    assert torch.allclose(got, out.reshape(9, 10) @ W["o"].T)
    # the sink takes weight: without it the rows are larger
    W2 = dict(W, sink=torch.tensor([-50.0, -50.0], dtype=D))
    assert not torch.allclose(plain_latent_attention(h, W2, m, 1e-6), got)


def test_plain_routing_chooses_with_the_correction_and_weighs_without_it():
    h = torch.eye(4, dtype=D)[:1]
    router = torch.tensor([[2.0, 0, 0, 0], [1.0, 0, 0, 0], [0.0, 0, 0, 0], [-1.0, 0, 0, 0]], dtype=D)
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0], dtype=D), 0)
    chosen, w = plain_route(h, router, torch.zeros(4, dtype=D), 2)
    assert chosen.tolist() == [[0, 1]] and torch.allclose(w[0], s[:2] / s[:2].sum())
    chosen, w = plain_route(h, router, torch.tensor([0.0, 0.0, 0.0, 1.0], dtype=D), 2)
    assert sorted(chosen[0].tolist()) == [0, 3]
    pick = {int(e): float(x) for e, x in zip(chosen[0], w[0])}
    assert abs(pick[0] - float(s[0] / (s[0] + s[3]))) < 1e-12 and abs(pick[3] - float(s[3] / (s[0] + s[3]))) < 1e-12


def test_plain_experts_clamp_and_the_shared_one_is_gated():
    one = torch.ones(1, 1, dtype=D)
    big, neg = torch.tensor([[10.0]], dtype=D), torch.tensor([[-10.0]], dtype=D)
    y = plain_expert(one, big, big, one, 2.0)                                             # g = 2, u = 2
    assert abs(float(y) - 2.0 / (1 + math.exp(-3.404)) * 3.0) < 1e-12
    y = plain_expert(one, neg, neg, one, 2.0)                                             # g = -10 stays, u = -2
    assert abs(float(y) - (-10.0 / (1 + math.exp(17.02))) * (-1.0)) < 1e-12
    assert abs(float(plain_dense_ff(one, {"up": torch.tensor([[3.0], [-3.0]], dtype=D), "down": torch.ones(1, 2, dtype=D)})) - 9.0) < 1e-12
    torch.manual_seed(4)
    mlp = {"router": {"experts": 3, "top": 1}, "expert": {"limit": 1.0}, "shared": {"ff": 2, "limit": 5.0}}
    W = {"router": torch.randn(3, 4, dtype=D), "correction": torch.zeros(3, dtype=D), "shared.gate": torch.randn(2, 4, dtype=D),
         "shared.up": torch.randn(2, 4, dtype=D), "shared.down": torch.randn(4, 2, dtype=D), "shared.sg": torch.randn(1, 4, dtype=D)}
    for e in range(3):
        W.update({f"e{e}.gate": torch.randn(2, 4, dtype=D), f"e{e}.up": torch.randn(2, 4, dtype=D), f"e{e}.down": torch.randn(4, 2, dtype=D)})
    h = torch.randn(5, 4, dtype=D)
    got = plain_moe(h, W, mlp)
    for t in range(5):
        e = int(torch.argmax(W["router"] @ h[t]))
        want = plain_expert(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], 1.0)[0]          # one chosen expert weighs 1
        want = want + torch.sigmoid(W["shared.sg"][0] @ h[t]) * plain_expert(h[t:t + 1], W["shared.gate"], W["shared.up"], W["shared.down"], 5.0)[0]
        assert torch.allclose(got[t], want)


def test_plain_streams_with_unit_connections_are_the_plain_sum():
    cfg, W = plain_weights("C")
    toks = random_tokens(cfg["vocab"], 12, seed=5)
    want = plain_forward(cfg, W, toks)
    for S in (1, 3):
        W2 = dict(W)
        for i, layer in enumerate(cfg["layers"]):
            for q in (1, 2) if layer["mlp"] else (1,):
                W2[f"l{i}.hc{q}.in"] = torch.full((S,), 1.0 / S, dtype=D)
                W2[f"l{i}.hc{q}.out"] = torch.ones(S, dtype=D)
                W2[f"l{i}.hc{q}.mix"] = torch.eye(S, dtype=D)
        # S equal copies, each read with 1 / S and written alike, stay equal; their sum is S times the one stream,
        # which the final norm does not see (but for its eps)
        got = plain_forward(dict(cfg, streams=S), W2, toks)
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-6)


# ------------------------------------------------------------------------------------------- host logic on the stand-ins
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_on_the_cpu(name):
    cfg, W = plain_weights(name)
    toks, other = random_tokens(cfg["vocab"], 150, seed=3), random_tokens(cfg["vocab"], 70, seed=4)
    want, want2 = plain_forward(cfg, W, toks), plain_forward(cfg, W, other)
    m = cpu_model(name)
    assert row_errors(run_whole(m, toks), want).max() < TOL
    assert row_errors(run_tail_one_by_one(m, toks[:90], 25), want[:90]).max() < TOL
    got = run_in_pieces(m, [toks, other], [[2, 4, 7, 64, 66, 140], [63, 65]])
    assert row_errors(got[0], want).max() < TOL and row_errors(got[1], want2).max() < TOL
    got = run_batched(m, [toks[:80], other[:9], other], [70, 3, 64])
    assert row_errors(got[0], want[:80]).max() < TOL and row_errors(got[1], want2[:9]).max() < TOL and row_errors(got[2], want2).max() < TOL
    m.cache.check()
    assert m.cache.slots.held == 0


def test_the_sum_of_the_streams_after_every_layer():
    cfg, W = plain_weights("A")
    toks = random_tokens(cfg["vocab"], 30, seed=8)
    _, streams = plain_forward(cfg, W, toks, return_layers=True)
    m = cpu_model("A")
    (slot,) = m.cache.open(1)
    seen = []
    for blk in m.blocks:
        orig = blk.forward
        def wrapped(xs, *a, _o=orig, **k):
            r = _o(xs, *a, **k)
            seen.append(xs.detach().double().sum(dim=1))
            return r
        blk.forward = wrapped
    m.step([StepEntry(slot, toks, [len(toks) - 1])])
    m.cache.close([slot])
    assert len(seen) == len(cfg["layers"])
    for got, want in zip(seen, streams):
        assert float((got - want).abs().max()) < 2e-4 * float(want.abs().max())


def test_window_layers_keep_a_ring_of_pages_and_kept_positions_every_page():
    m = cpu_model("A", max_tokens=2048)
    rings = {g.request.head_dim: (g.request.window, g.ring_pages, g.request.planes) for g in m.cache.groups}
    assert rings[48] == (33, 2, 1) and rings[64] == (64, 2, 1)            # the latent layers: one plane of kv_rank + rot_dim values
    # the layer without a window and the one whose window keeps first positions (heads of 24 | 16 values in places of 32)
    # share one group that keeps every page
    assert rings[32] == (0, 0, 2) and len(rings) == 3
    cfg, W = plain_weights("A")
    toks = random_tokens(cfg["vocab"], 300, seed=9)                       # longer than every ring
    want = plain_forward(cfg, W, toks)
    assert row_errors(run_tail_one_by_one(m, toks, 40), want).max() < TOL
    got = run_in_pieces(m, [toks], [[130, 131, 200, 290]])
    assert row_errors(got[0], want).max() < TOL


def test_reused_slots_and_pages_start_from_nothing():
    cfg, W = plain_weights("B")
    m = cpu_model("B", max_tokens=128, max_seqs=1)
    for seed in (1, 2, 3):
        toks = random_tokens(cfg["vocab"], 70, seed=seed)
        assert row_errors(run_tail_one_by_one(m, toks, 10), plain_forward(cfg, W, toks)).max() < TOL


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
    for name in ("A", "B", "C"):
        m = cpu_model(name)
        sd = m.state_dict()
        cfg, W = plain_weights(name)
        assert set(sd) == set(W)
        for n, t in W.items():
            assert torch.allclose(sd[n].double().reshape(t.shape), t, atol=1e-6 if "norm" in n else 0, rtol=0), n


@pytest.mark.parametrize("layer,key,candidates", [(0, "size", range(5, 40)), (0, "keep_first", range(1, 8)), (1, "size", range(5, 50)),
                                                  (3, "size", range(5, 60))])
def test_a_key_that_carries_a_row_just_inside_and_just_outside_a_mask(layer, key, candidates):
    """The weights are sharp: single keys carry rows.  The mask constant is set so that the key which carries the last row
    is the last one still seen, and then the first one not seen any more; the logits differ widely, and the package
    follows on both sides, whole and with the last tokens decoded."""
    from netezen_cases import carrying_edge, variant_folder
    from netezen_plain import read_folder
    from reference_kernels import ReferenceKernels
    from cima_b200.engine import load_model
    cfg, W = plain_weights("A")
    toks = random_tokens(cfg["vocab"], 75, seed=12)
    v, jump = carrying_edge(cfg, W, toks, layer, key, list(candidates))
    assert jump > 0.5, "no key of this layer carries the last row"
    for value in (v, v - 1):
        d = variant_folder("A", lambda c: c["layers"][layer]["mixer"]["mask"].__setitem__(key, value))
        cfg2, W2 = read_folder(d)
        want = plain_forward(cfg2, W2, toks)
        m = load_model(d, dtype="float32", max_tokens=1024, device="cpu", kernels=ReferenceKernels(), verbose=False)
        assert row_errors(run_whole(m, toks), want).max() < TOL
        assert row_errors(run_tail_one_by_one(m, toks, 8), want).max() < TOL


def test_the_sink_takes_its_share():
    cfg, W = plain_weights("A")
    toks = random_tokens(cfg["vocab"], 40, seed=13)
    base = plain_forward(cfg, W, toks)
    W2 = dict(W)
    W2["l1.mix.sink"] = W["l1.mix.sink"] - 30.0
    assert float((plain_forward(cfg, W2, toks) - base).abs().max()) > 0.05
