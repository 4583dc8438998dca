"""Lipizen configurations drawn at random (every size and constant that config.json gives, layer by layer, in any order
of the two layer kinds, with layers that read an earlier layer's keys) in cuttings drawn at random too (whole, a tail one
by one, pieces, unequal batches): in 32-bit against the plain implementation on weights that make attention sharp, and in
bfloat16 against the 32-bit engine on milder weights of the same configuration."""
import os
import random

import pytest
import torch
from safetensors.torch import load_file, save_file

import cima_b200
from cima_b200.engine import load_model
from lipizen_cases import _boost, attention, config, dense, hgrn2, row_errors
from lipizen_plain import plain_forward, read_folder
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole

pytestmark = pytest.mark.gpu

SEEDS = list(range(int(os.environ.get("CIMA_RANDOM_CONFIGS", "6"))))


def draw_mlp(rng: random.Random):
    return None if rng.random() < 0.3 else dense(rng.choice([8, 20, 33, 64, 96, 130]), rng.choice([0.5, 1.0, 2.0, 7.0]))


def draw_config(rng: random.Random) -> dict:
    groups = rng.choice([1, 1, 2, 3, 4])
    width = groups * rng.choice([16, 24, 25, 32, 48, 64, 80])                 # some are no multiple of 8
    layers, sources = [], []
    for i in range(rng.randint(1, 6)):
        if rng.random() < 0.6:
            if sources and rng.random() < 0.4:                                  # reads an earlier layer's keys and values
                src = rng.choice(sources)
                s = layers[src]["mixer"]
                kv, dim, vdim = s["kv_heads"], s["dim"], s["vdim"]
                rotary = (s["rot"]["dims"], s["rot"]["base"], (s["rot"].get("scaling") or {}).get("factor")) if s.get("rot") else None
            else:
                src = None
                kv = rng.choice([1, 2, 3])
                dim = rng.choice([8, 16, 24, 32, 48, 64, 80, 128])
                vdim = rng.choice([8, 16, 24, 32, 48, 64, 96, 128])
                rotary = None
                if rng.random() < 0.85:
                    dims = rng.choice([d for d in (4, 8, 16, 32, 64, dim, dim) if d <= dim])
                    rotary = (dims, rng.choice([100.0, 10000.0, 500000.0]), rng.choice([None, 1.0, 2.0, 4.0, 8.0]))
            heads = kv * rng.choice([1, 2, 4])
            mask = None
            if rng.random() < 0.85:
                mask = (rng.choice([1, 2, 17, 63, 64, 65, 100, 128, 500]), rng.choice([0, 0, 1, 4, 64, 70]))
            if src is None:
                sources.append(i)
            layers.append(attention(heads, kv, dim, vdim, rng.choice([0.1, 0.25, 0.5]), rng.choice([0.1, 0.3, 0.6, 0.8]),
                                    rng.choice([0, 1, 2, 3, 4, 5]) if src is None else rng.choice([1, 2, 4]), rotary, mask, draw_mlp(rng),
                                    kv_from=src))
        else:
            layers.append(hgrn2(rng.randint(1, 5), rng.choice([8, 16, 40, 64, 128, 160]), rng.choice([8, 16, 24, 64, 100]), draw_mlp(rng)))
    return config(rng.choice([129, 333, 512, 1001]), width, rng.choice([1e-6, 1e-5, 3e-4]), groups, rng.choice([0.5, 1.0, 2.0, 3.5]),
                  rng.choice([0.0, 15.0, 30.0, 50.0]), layers)


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(seed, tmp_path):
    rng = random.Random(7000 + seed)
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
