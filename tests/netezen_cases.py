"""Small Netezen configurations, their weights and helpers shared by the tests of that design.

The weights are drawn by ``cima_b200.write_random_model`` and then scaled by tensor name, so that the stream stays of
order one behind every norm, the attention maps are sharp (single keys carry rows, near or far, inside and outside a
window), the routers prefer different experts for different tokens, the corrections change choices, the clamps of the
experts are reached and the sinks take a visible share of a row's weight."""
from __future__ import annotations

import os
import tempfile

import torch

import cima_b200
from cima_b200.engine import load_model


def attention(heads, kv_heads, dim, vdim, scale, rot, mask, mlp):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        dims, base, scaling = rot
        m["rot"] = {"dims": dims, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, window, mlp, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def config(vocab, width, eps, mult, streams, layers):
    c = {"architecture": "Netezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if streams is not None:
        c["streams"] = streams
    return c


# three streams; grouped key heads with a value size below the key size, a partial rotation with rescaled frequencies, a
# window with kept first positions; a latent layer whose position keeps 48 values, with a window that is no multiple of
# a page; a layer without feed-forward, window or rotation; experts with and without a shared one
N_A = config(300, 96, 1e-5, 0.5, 3, [
    attention(4, 2, 24, 16, 0.2, (8, 10000.0, (8.0, 64, 16.0, 2.0)), (20, 3), moe(6, 2, 32, 1.5, (40, 0.8))),
    latent(3, 16, 8, 24, 40, 32, 0.25, 5000.0, 33, dense(72)),
    attention(2, 2, 32, 32, 0.18, None, None, None),
    latent(2, 24, 16, 16, 48, 24, 0.2, 300.0, 64, moe(5, 1, 24, 0.75))])
# one stream that still has its stored connection; a width that is no multiple of 8; a multiplier of 1; one key head for
# all; whole heads rotate, frequencies as they are; a window of one position with one kept position; a window no test
# sequence reaches; one expert of one; a latent layer without a window whose key part rotates with rescaled frequencies; a
# layer whose heads rotate whole and have keys and values of one size (a decode step's projection rotates and appends itself)
N_B = config(513, 100, 1e-6, 1.0, 1, [
    latent(5, 8, 4, 12, 20, 16, 0.3, 100.0, 0, moe(1, 1, 16, 2.0, (8, 3.0)), scaling=(4.0, 32, 8.0, 1.0)),
    attention(3, 1, 16, 40, 0.25, (16, 500.0, None), (1, 1), dense(33)),
    attention(6, 3, 8, 8, 0.35, (4, 50000.0, (2.0, 16, 4.0, 1.0)), (4096, 0), moe(7, 7, 8, 1.0)),
    attention(4, 2, 16, 16, 0.3, (16, 1000.0, None), (50, 0), None)])
# no streams at all (the plain pre-norm sum); heads of 64 and 128 values; kept positions that fill a page and more behind a
# window of exactly a page; a position that keeps 128 values and one that keeps 104 (no multiple of 16)
N_C = config(640, 256, 1e-5, 0.7, None, [
    attention(4, 1, 64, 64, 0.12, (32, 200000.0, (4.0, 128, 32.0, 1.0)), (64, 70), dense(192)),
    latent(4, 64, 32, 64, 96, 80, 0.1, 20000.0, 130, moe(8, 3, 64, 2.0, (96, 1.0))),
    attention(2, 2, 128, 128, 0.09, (64, 10000.0, None), (100, 0), None),
    latent(2, 48, 24, 32, 80, 0, 0.12, 1000.0, 40, dense(96))])
CONFIGS = {"A": N_A, "B": N_B, "C": N_C}

# factor by the last part of a tensor's name (a drawn matrix has entries of about 0.02)
_BOOST = {"embed": 40.0, "q": 14.0, "k": 14.0, "uq": 3.0, "dq": 10.0, "dkv": 10.0, "uk": 1.5, "uv": 1.0, "router": 25.0, "gate": 15.0,
          "up": 15.0, "sg": 3.0}
_DEFAULT_BOOST = 6.0


def _boost(name: str, t: torch.Tensor, sharp: bool = True) -> torch.Tensor:
    """``sharp`` False leaves the attention's scores of order one: bfloat16 runs are compared on such weights, since with
    scores of tens the rounding of a query decides which key carries a row."""
    last = name.rsplit(".", 1)[-1]
    if last == "correction":
        return (t.float() * 8.0).to(t.dtype)                # of the size of the softmax scores' differences
    if t.dim() < 2 or ".hc" in name:
        return t
    f = _BOOST.get(last, _DEFAULT_BOOST)
    if not sharp and last in ("q", "k", "uq"):
        f = f / 3.0
    return (t.float() * f).to(t.dtype)


_FOLDERS = {}


def write_folder(d: str, cfg: dict, seed: int = 0, sharp: bool = True) -> str:
    from safetensors.torch import load_file, save_file
    cima_b200.write_random_model(d, cfg, seed=seed)
    path = os.path.join(d, "model.safetensors")
    save_file({n: _boost(n, t, sharp).contiguous() for n, t in load_file(path).items()}, path)
    return d


def folder(name: str, seed: int = 0, sharp: bool = True) -> str:
    key = (name, seed, sharp)
    if key not in _FOLDERS:
        _FOLDERS[key] = write_folder(tempfile.mkdtemp(prefix=f"cima_netezen_{name}_"), CONFIGS[name], seed, sharp)
    return _FOLDERS[key]


def variant_folder(name: str, edit, seed: int = 0, sharp: bool = True) -> str:
    """A folder of configuration ``name`` after ``edit(cfg)`` changed constants in it (masks, multipliers): tensors are drawn
    by name, so the weights are those of the unchanged configuration."""
    import copy
    cfg = copy.deepcopy(CONFIGS[name])
    edit(cfg)
    return write_folder(tempfile.mkdtemp(prefix=f"cima_netezen_{name}_variant_"), cfg, seed, sharp)


def carrying_edge(cfg, W, toks, layer: int, key: str, candidates):
    """Among ``candidates`` for the mask constant ``key`` of ``layer``, the value v whose step to v - 1 changes the last
    row of the plain implementation's logits most: at v a key that carries that row is just visible, at v - 1 just not."""
    import copy
    from netezen_plain import plain_forward
    rows = {}
    for v in sorted(set(candidates) | {c - 1 for c in candidates}):
        c2 = copy.deepcopy(cfg)
        c2["layers"][layer]["mixer"]["mask"][key] = v
        rows[v] = plain_forward(c2, W, toks)[-1]
    best = max(candidates, key=lambda v: float((rows[v] - rows[v - 1]).abs().max()))
    return best, float((rows[best] - rows[best - 1]).abs().max())


def plain_weights(name: str, seed: int = 0, sharp: bool = True):
    """(config dict, tensors in float64) of a folder, read without the package."""
    from netezen_plain import read_folder
    return read_folder(folder(name, seed, sharp))


def cpu_model(name, dtype="float32", max_tokens=1024, seed=0, sharp=True, **kw):
    from reference_kernels import ReferenceKernels
    return load_model(folder(name, seed, sharp), dtype=dtype, max_tokens=max_tokens, device="cpu", kernels=ReferenceKernels(),
                      verbose=False, **kw)


def gpu_model(name, dtype="float32", max_tokens=1024, seed=0, sharp=True, **kw):
    return load_model(folder(name, seed, sharp), dtype=dtype, max_tokens=max_tokens, device="cuda:0", verbose=False, **kw)


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference (its mean taken off) over that of the wanted row."""
    d = got.double() - want.double()
    d = d - d.mean(dim=1, keepdim=True)
    w = want.double() - want.double().mean(dim=1, keepdim=True)
    return d.pow(2).mean(dim=1).sqrt() / w.pow(2).mean(dim=1).sqrt().clamp_min(1e-30)
