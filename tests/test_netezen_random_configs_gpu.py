"""Netezen configurations drawn at random (every size and constant that config.json gives, layer by layer, in any order of
the two layer kinds and the three feed-forwards, with one to six streams or none) in cuttings drawn at random too (whole,
a tail one by one, pieces, unequal batches): in 32-bit against the plain implementation on weights that make attention
sharp, and in bfloat16 against the 32-bit engine on milder weights of the same configuration."""
import os
import random

import pytest
import torch
from safetensors.torch import load_file, save_file

import cima_b200
from cima_b200.engine import load_model
from netezen_cases import _boost, attention, config, dense, latent, moe, row_errors
from netezen_plain import plain_forward, read_folder
from helpers import random_tokens, run_batched, run_in_pieces, run_tail_one_by_one, run_whole

pytestmark = pytest.mark.gpu

SEEDS = list(range(int(os.environ.get("CIMA_RANDOM_CONFIGS", "8"))))
WINDOWS = [1, 2, 17, 63, 64, 65, 100, 128, 500]


def draw_mlp(rng: random.Random):
    r = rng.random()
    if r < 0.2:
        return None
    if r < 0.45:
        return dense(rng.choice([8, 20, 33, 64, 96, 130]))
    experts = rng.choice([1, 2, 3, 5, 8, 12, 20])
    shared = (rng.choice([8, 24, 40, 64]), rng.choice([0.5, 1.0, 3.0])) if rng.random() < 0.6 else None
    return moe(experts, rng.randint(1, min(experts, 4)), rng.choice([8, 16, 24, 40, 64]), rng.choice([0.5, 1.0, 2.0, 7.0]), shared)


def draw_config(rng: random.Random) -> dict:
    width = rng.choice([16, 24, 25, 32, 48, 64, 80, 100, 128, 192, 256])            # some are no multiple of 8
    layers = []
    for _ in range(rng.randint(1, 6)):
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 32, 48, 64, 80, 128])
            rotary = None
            if rng.random() < 0.85:
                dims = rng.choice([d for d in (2, 4, 8, 16, 32, 64, dim, dim) if d <= dim])
                scaling = None
                if rng.random() < 0.6:
                    scaling = (rng.choice([2.0, 4.0, 8.0, 40.0]), rng.choice([16, 64, 4096]), rng.choice([8.0, 32.0]), rng.choice([1.0, 2.0]))
                rotary = (dims, rng.choice([100.0, 10000.0, 500000.0]), scaling)
            mask = (rng.choice(WINDOWS), rng.choice([0, 0, 1, 4, 64, 70])) if rng.random() < 0.85 else None
            layers.append(attention(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([8, 16, 24, 32, 48, 64, 96, 128]), rng.choice([0.08, 0.15, 0.3]),
                                    rotary, mask, draw_mlp(rng)))
        else:
            rank, rot = rng.choice([8, 16, 24, 40, 48, 64, 96, 112]), rng.choice([2, 4, 8, 16, 32])
            layers.append(latent(rng.randint(1, 6), rng.choice([8, 16, 24, 32, 64, 96]), rot, rng.choice([8, 16, 24, 32, 64, 100]), rank,
                                 rng.choice([8, 16, 24, 48, 96]), rng.choice([0.08, 0.15, 0.3]), rng.choice([50.0, 10000.0, 200000.0]),
                                 rng.choice([0] + WINDOWS), draw_mlp(rng),
                                 scaling=(rng.choice([2.0, 8.0]), rng.choice([16, 256]), rng.choice([8.0, 32.0]), 1.0) if rng.random() < 0.3 else None))
    return config(rng.choice([129, 333, 512, 1001]), width, rng.choice([1e-6, 1e-5, 3e-4]), rng.choice([0.3, 0.5, 1.0, 1.4]),
                  rng.choice([None, 1, 2, 2, 3, 4, 6]), layers)


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(seed, tmp_path):
    rng = random.Random(9000 + seed)
    cfg = draw_config(rng)
    folders = {}
    for kind in ("sharp", "mild"):
        folders[kind] = str(tmp_path / kind)
        cima_b200.write_random_model(folders[kind], cfg, seed=seed)
        path = os.path.join(folders[kind], "model.safetensors")
        save_file({n: _boost(n, t, sharp=kind == "sharp").contiguous() for n, t in load_file(path).items()}, path)
    c, W = read_folder(folders["sharp"])
    n = rng.choice([40, 130, 300])
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
                assert e.max() < 3e-4, (cfg, what, float(e.max()))      # sums of float32 through sharp softmaxes; a fault shows at 1e-2
            elif dtype == "float32":
                exact[what] = got
            else:
                e = row_errors(got, exact[what])
                assert torch.isfinite(got).all() and e.median() < 6e-2, (cfg, what, float(e.median()), float(e.max()))
        m.cache.check()
        assert m.cache.slots.held == 0
        del m
        torch.cuda.empty_cache()
