"""The Lipizen design without a GPU: its configuration, the plain implementation against independent statements of the
same mechanisms, and the package's host logic (cache, state, step function, generation loop) driven on the CPU through
the plain PyTorch stand-ins of the kernels."""
import copy
import math

import pytest
import torch

import cima_b200
from cima_b200.config import ConfigError, LipizenConfig, lookup_architecture
from cima_b200.engine import build_plan
from lipizen_cases import CONFIGS, L_A, L_B, cpu_model, plain_weights, row_errors
from lipizen_plain import (plain_causal_conv, plain_dense_ff, plain_diff_attention, plain_forward, plain_group_norm, plain_hgrn2,
                           plain_keys_values, plain_rms, plain_rotate, plain_softmax_attention, plain_visible)
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole

TOL = 3e-5


# ------------------------------------------------------------------------------------------- configuration
def test_configuration_round_trip_and_plan():
    entry = lookup_architecture(L_A)
    cfg = entry.parse(L_A)
    assert isinstance(cfg, LipizenConfig) and LipizenConfig.from_dict(cfg.to_dict()) == cfg
    spec = entry.spec(cfg)
    assert not spec.tie_head and spec.logit_softcap == 20.0 and spec.final_norm.params["groups"] == 3
    assert [b.kind for b in spec.layers] == ["postnorm"] * 5 and spec.layers[2].feed_forward is None and spec.layers[0].stream_mult == 1.5
    assert [b.mixer.kind for b in spec.layers] == ["gated_recurrence", "diff_attention", "diff_attention", "gated_recurrence", "diff_attention"]
    assert [b.mixer.cache_from for b in spec.layers] == [None, None, 1, None, 1]
    # layer 1's pages serve a reader without kept positions and a wider mask, and itself with kept positions: every page stays
    assert spec.layers[1].mixer.params["cache_window"] == 0
    plan = build_plan(spec)
    assert plan["embed"].shape == (300, 96) and plan["head"].shape == (300, 96) and plan["final.norm"].shape == (96,)
    assert plan["l0.mix.q"].shape == (48, 96) and plan["l0.mix.f"].shape == (48, 96) and plan["l0.mix.f.b"].shape == (48,)
    assert plan["l0.mix.lower"].shape == (48,) and plan["l0.mix.v"].shape == (80, 96) and plan["l0.mix.norm"].shape == (40,)
    assert plan["l0.mix.o"].shape == (96, 80) and plan["l0.mlp.gate"].shape == (72, 96) and plan["l0.mlp.down"].shape == (96, 72)
    assert plan["l1.mix.q"].shape == (128, 96) and plan["l1.mix.k"].shape == (64, 96) and plan["l1.mix.v"].shape == (48, 96)
    assert plan["l1.mix.q.conv"].shape == (128, 2) and plan["l1.mix.v.conv"].shape == (48, 2) and plan["l1.mix.k.norm"].shape == (16,)
    assert plan["l1.mix.g"].shape == (4, 96) and plan["l1.mix.o"].shape == (96, 96) and plan["l1.mix.lq2"].shape == (16,)
    assert plan["l2.mix.q.conv"].shape == (128, 4) and "l2.mix.k" not in plan and "l2.mix.v.conv" not in plan and "l2.mix.k.norm" not in plan
    assert "l2.norm2" not in plan and "l2.mlp.gate" not in plan and "l3.norm2" not in plan and plan["l4.norm2"].shape == (96,)


def test_the_widest_reader_sizes_a_layers_pages():
    from lipizen_cases import attention, config, dense
    rot = (8, 100.0, None)
    c = config(50, 32, 1e-5, 1, 1.0, 0.0, [attention(2, 1, 16, 16, 0.5, 0.5, 2, rot, (40, 0), dense(16, 1.0)),
                                           attention(2, 1, 16, 16, 0.5, 0.5, 2, rot, (100, 0), None, kv_from=0),
                                           attention(2, 1, 16, 16, 0.5, 0.5, 2, rot, (30, 0), None)])
    spec = LipizenConfig.from_dict(c).model_spec()
    assert [b.mixer.params["cache_window"] for b in spec.layers][::2] == [100, 30]
    c["layers"][1]["mixer"]["mask"] = None                                     # a reader without a window
    assert LipizenConfig.from_dict(c).model_spec().layers[0].mixer.params["cache_window"] == 0


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c.update(architecture="Other"), "architecture"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0.0), "factor"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),          # a recurrence has no keys
    (lambda c: c["layers"][2]["mixer"].update(kv_from=4), "kv_from"),          # a later layer
    (lambda c: c["layers"][4]["mixer"].update(kv_from=2), "kv_from"),          # a layer that reads another's itself
    (lambda c: c["layers"][4]["mixer"].update(vdim=32), "differs"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "dense"),
    (lambda c: c["layers"][0]["mlp"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_configuration_refuses(change, word):
    cfg = copy.deepcopy(L_A)
    change(cfg)
    with pytest.raises(ConfigError, match=word):
        LipizenConfig.from_dict(cfg)


# ------------------------------------------------------------------------------------------- the plain side
def test_plain_group_norm_is_a_norm_per_part():
    torch.manual_seed(0)
    x, w = torch.randn(5, 12, dtype=torch.float64) * 3, torch.randn(12, dtype=torch.float64)
    got = plain_group_norm(x, w, 3, 1e-3)
    for g in range(3):
        part = x[:, 4 * g:4 * g + 4]
        assert torch.allclose(got[:, 4 * g:4 * g + 4], part / torch.sqrt((part ** 2).mean(1, keepdim=True) + 1e-3) * w[4 * g:4 * g + 4], atol=1e-12)
    assert torch.allclose(plain_group_norm(x, w, 1, 1e-3), plain_rms(x, 1e-3) * w, atol=1e-12)
    # eps stands inside the root: a row of zeros stays zero, a tiny row is divided by about sqrt(eps)
    tiny = torch.full((1, 4), 1e-9, dtype=torch.float64)
    assert torch.allclose(plain_rms(tiny, 1e-4), tiny / 1e-2, rtol=1e-6)


def test_plain_convolution_against_conv1d():
    torch.manual_seed(4)
    for taps in (1, 2, 3, 5):
        z, w = torch.randn(9, 5, dtype=torch.float64), torch.randn(5, taps, dtype=torch.float64)
        want = torch.nn.functional.conv1d(torch.nn.functional.pad(z.T[None], (taps - 1, 0)), w[:, None, :], groups=5)[0].T
        assert torch.allclose(plain_causal_conv(z, w), want, atol=1e-12)
    # the newest tap is the last column
    w = torch.zeros(5, 3, dtype=torch.float64); w[:, -1] = 1.0
    assert torch.equal(plain_causal_conv(z, w), z)


def test_plain_rotation_depends_on_the_distance_only_and_leaves_the_rest():
    torch.manual_seed(1)
    x, y = torch.randn(1, 1, 12, dtype=torch.float64), torch.randn(1, 1, 12, dtype=torch.float64)
    dots = [float((plain_rotate(x, 8, 50.0, 4.0, a)[0, 0, :8] * plain_rotate(y, 8, 50.0, 4.0, a + 3)[0, 0, :8]).sum()) for a in (0, 5, 40)]
    assert max(dots) - min(dots) < 1e-9
    assert torch.equal(plain_rotate(x, 8, 50.0, 4.0, 9)[..., 8:], x[..., 8:])
    # value i turns with value i + dims / 2, by position * base^(-2 i / dims) / factor
    r = plain_rotate(x, 8, 50.0, 4.0, 6)[0, 0]
    for i in range(4):
        a = 6 * 50.0 ** (-2 * i / 8) / 4.0
        assert math.isclose(float(r[i]), float(x[0, 0, i] * math.cos(a) - x[0, 0, i + 4] * math.sin(a)), abs_tol=1e-12)
        assert math.isclose(float(r[i + 4]), float(x[0, 0, i + 4] * math.cos(a) + x[0, 0, i] * math.sin(a)), abs_tol=1e-12)
    # a factor of 4 is the same as positions a quarter as large
    assert torch.allclose(plain_rotate(x, 8, 50.0, 4.0, 8), plain_rotate(x, 8, 50.0, 1.0, 2), atol=1e-12)


def test_plain_mask_window_and_kept_first_positions():
    seen = lambda i, size, keep: [j for j in range(i + 3) if plain_visible(i, j, size, keep)]
    assert seen(10, 4, 0) == [7, 8, 9, 10] and seen(10, 4, 2) == [0, 1, 7, 8, 9, 10] and seen(2, 4, 2) == [0, 1, 2]
    assert seen(5, 1, 1) == [0, 5] and seen(5, 0, 0) == list(range(6)) and seen(4, 4, 3) == [0, 1, 2, 3, 4]
    # as a softmax over a masked score matrix
    torch.manual_seed(2)
    T, D = 12, 6
    q, k, v = (torch.randn(T, D, dtype=torch.float64) for _ in range(3))
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = (j <= i) & ((i - j < 5) | (j < 2))
    s = (q @ k.T * 0.3).masked_fill(~ok, float("-inf"))
    assert torch.allclose(plain_softmax_attention(q, k, v, 0.3, 5, 2), torch.softmax(s, dim=1) @ v, atol=1e-12)


def test_plain_differential_attention_from_two_score_matrices():
    """Both maps in matrix form, four query heads on two key heads, the shared values and the one lambda of the layer."""
    torch.manual_seed(3)
    T, W, H, G, D, Dv, eps, d = 9, 10, 4, 2, 6, 5, 1e-5, 0.3
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.4, "diff": d, "conv": 0, "mask": {"size": 4, "keep_first": 1}}
    Wt = {"q": torch.randn(H * 2 * D, W), "k": torch.randn(G * 2 * D, W), "v": torch.randn(G * Dv, W), "q.norm": torch.rand(D) + 0.5,
          "k.norm": torch.rand(D) + 0.5, "g": torch.randn(H, W), "o": torch.randn(W, H * Dv), "lq1": torch.randn(D) * 0.3,
          "lk1": torch.randn(D) * 0.3, "lq2": torch.randn(D) * 0.3, "lk2": torch.randn(D) * 0.3}
    Wt = {k: v.double() for k, v in Wt.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    got = plain_diff_attention(h, Wt, m, eps)
    q = (h @ Wt["q"].T).view(T, H, 2, D); k = (h @ Wt["k"].T).view(T, G, 2, D); v = (h @ Wt["v"].T).view(T, G, Dv)
    q = q / torch.sqrt((q ** 2).mean(-1, keepdim=True) + eps) * Wt["q.norm"]
    k = k / torch.sqrt((k ** 2).mean(-1, keepdim=True) + eps) * Wt["k.norm"]
    lam = math.exp(float(Wt["lq1"] @ Wt["lk1"])) - math.exp(float(Wt["lq2"] @ Wt["lk2"])) + d
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = (j <= i) & ((i - j < 4) | (j < 1))
    out = []
    for hh in range(H):
        maps = [torch.softmax((q[:, hh, mm] @ k[:, hh // 2, mm].T * 0.4).masked_fill(~ok, float("-inf")), dim=1) for mm in (0, 1)]
        o = (maps[0] - lam * maps[1]) @ v[:, hh // 2]                         # the difference of the maps, then the values
        o = o / torch.sqrt((o ** 2).mean(-1, keepdim=True) + eps) * (1 - d)
        out.append(o * torch.sigmoid(h @ Wt["g"][hh])[:, None])
    assert torch.allclose(got, torch.cat(out, dim=1) @ Wt["o"].T, atol=1e-10)


def test_plain_recurrence_as_a_weighted_sum_over_the_past():
    """o_t[j] = sum_(s <= t) sum_c q_t[c] (prod_(s < r <= t) f_r[c]) (1 - f_s[c]) v_s[j]: the recurrence unrolled."""
    torch.manual_seed(5)
    T, W, H, D, Dv, eps = 6, 8, 2, 3, 4, 1e-5
    Wt = {"q": torch.randn(H * D, W), "f": torch.randn(H * D, W), "f.b": torch.randn(H * D), "lower": torch.rand(H * D) * 0.9,
          "v": torch.randn(H * Dv, W), "norm": torch.rand(Dv) + 0.5, "o": torch.randn(W, H * Dv)}
    Wt = {k: v.double() for k, v in Wt.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    got = plain_hgrn2(h, Wt, {"heads": H, "dim": D, "vdim": Dv}, eps)
    z = h @ Wt["q"].T
    q = (z / (1 + torch.exp(-z))).view(T, H, D)
    f = (Wt["lower"] + (1 - Wt["lower"]) / (1 + torch.exp(-(h @ Wt["f"].T + Wt["f.b"])))).view(T, H, D)
    v = (h @ Wt["v"].T).view(T, H, Dv)
    assert bool((f >= Wt["lower"].view(H, D)).all()) and bool((f < 1).all())
    o = torch.zeros(T, H, Dv, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            keep = torch.ones(H, D, dtype=torch.float64)
            for r in range(s + 1, t + 1):
                keep = keep * f[r]
            o[t] += ((q[t] * keep * (1 - f[s])).sum(-1, keepdim=True)) * v[s]
    o = o / torch.sqrt((o ** 2).mean(-1, keepdim=True) + eps) * Wt["norm"]
    assert torch.allclose(got, o.view(T, -1) @ Wt["o"].T, atol=1e-10)


def test_plain_feed_forward_clamps():
    W = {"gate": torch.eye(3, dtype=torch.float64), "up": torch.eye(3, dtype=torch.float64), "down": torch.eye(3, dtype=torch.float64)}
    h = torch.tensor([[5.0, -5.0, 0.5]], dtype=torch.float64)
    g = torch.tensor([2.0, -5.0, 0.5], dtype=torch.float64)                   # the gate is cut from above only
    u = torch.tensor([2.0, -2.0, 0.5], dtype=torch.float64)                   # the other branch from both sides
    assert torch.allclose(plain_dense_ff(h, W, 2.0), (g / (1 + torch.exp(-1.702 * g)) * (u + 1))[None], atol=1e-12)


def test_a_layer_that_reads_anothers_keys_sees_them_as_they_were_stored():
    cfg, W = plain_weights("A")
    torch.manual_seed(6)
    h1, h2 = torch.randn(7, 96, dtype=torch.float64), torch.randn(7, 96, dtype=torch.float64)
    sub = lambda i: {k[len(f"l{i}.mix."):]: v for k, v in W.items() if k.startswith(f"l{i}.mix.")}
    m1, m2 = cfg["layers"][1]["mixer"], cfg["layers"][2]["mixer"]
    kv = plain_keys_values(h1, sub(1), m1, 1e-6)
    assert kv[0].shape == (7, 2, 2, 16) and kv[1].shape == (7, 2, 24)
    a = plain_diff_attention(h2, sub(2), m2, 1e-6, kv)
    b = plain_diff_attention(h2, sub(2), m2, 1e-6, plain_keys_values(h1 * 2.0, sub(1), m1, 1e-6))
    assert not torch.allclose(a, b)                                            # the values (not normed) carry the other layer's input


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


def test_the_stream_after_every_layer():
    cfg, W = plain_weights("A")
    toks = random_tokens(cfg["vocab"], 30, seed=8)
    _, streams = plain_forward(cfg, W, toks, return_layers=True)
    m = cpu_model("A")
    from cima_b200.engine import StepEntry
    (slot,) = m.cache.open(1)
    seen = []
    for i, blk in enumerate(m.blocks):
        orig = blk.forward
        def wrapped(x, *a, _o=orig, **k):
            r = _o(x, *a, **k)
            seen.append(x.detach().double().clone())
            return r
        blk.forward = wrapped
    m.step([StepEntry(slot, toks, [len(toks) - 1])])
    m.cache.close([slot])
    assert len(seen) == len(cfg["layers"])
    for got, want in zip(seen, streams):
        assert float((got - want).abs().max()) < 2e-4 * float(want.abs().max())


def test_reused_slots_start_from_nothing():
    """A slot that held a sequence is handed to the next one with its recurrent state and the convolution's inputs zeroed."""
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
    for name in ("A", "B"):
        m = cpu_model(name)
        sd = m.state_dict()
        cfg, W = plain_weights(name)
        assert set(sd) == set(W)
        for n, t in W.items():
            assert torch.allclose(sd[n].double().reshape(t.shape), t, atol=0, rtol=0), n
