"""Small Lipizen configurations, their weights and helpers shared by the tests of that design.

The weights are drawn by ``cima_b200.write_random_model`` and then scaled by tensor name, so that the stream stays of
order one behind every norm, the two attention maps are sharp (single keys carry rows, near or far, inside and outside
the window), the recurrence's gates range from fast to slow and the clamps of the feed-forward are reached."""
from __future__ import annotations

import os
import tempfile

import torch

import cima_b200
from cima_b200.engine import load_model


def attention(heads, kv_heads, dim, vdim, scale, diff, conv, rot, mask, mlp, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff, "conv": conv}
    if rot is not None:
        dims, base, factor = rot
        m["rot"] = {"dims": dims, "base": base}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def hgrn2(heads, dim, vdim, mlp):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(vocab, width, eps, groups, alpha, softcap, layers):
    c = {"architecture": "Lipizen", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "postln_alpha": alpha,
         "layers": layers}
    if softcap:
        c["logit_softcap"] = softcap
    return c


# the recurrence first; grouped key heads (2 query heads a key head); value size above and below the key size; partial
# rotation with compressed positions; two readers of one layer's keys, one with a wider mask and no kept positions,
# one with a narrower mask; layers without feed-forward of either kind; three norm groups
L_A = config(300, 96, 1e-6, 3, 1.5, 20.0, [
    hgrn2(2, 24, 40, dense(72, 1.5)),
    attention(4, 2, 16, 24, 0.7, 0.3, 2, (8, 10000.0, 2.0), (40, 3), dense(56, 0.75)),
    attention(4, 2, 16, 24, 0.7, 0.5, 4, (8, 10000.0, 2.0), (70, 0), None, kv_from=1),
    hgrn2(3, 16, 8, None),
    attention(4, 2, 16, 24, 0.6, 0.3, 1, (8, 10000.0, 2.0), (9, 5), dense(40, 2.0), kv_from=1)])
# a width that is no multiple of 8; one norm group; alpha 1; no soft cap; whole heads rotate, positions as they are; a window
# no test sequence reaches, and one of a single position with a kept first position; one key head for all; one head
L_B = config(513, 100, 1e-5, 1, 1.0, 0.0, [
    attention(3, 3, 24, 8, 0.5, 0.8, 3, (24, 500.0, None), (4096, 0), dense(33, 1.0)),
    hgrn2(1, 40, 24, None),
    attention(2, 1, 32, 64, 0.45, 0.1, 5, (16, 50000.0, 8.0), (1, 1), None),
    hgrn2(5, 8, 20, dense(24, 0.5))])
# heads of 64 and 128 values, a window of exactly a page and kept positions that fill a page and more, a recurrence over 128
# key channels, four query heads on one key head
L_C = config(640, 256, 1e-5, 4, 2.5, 50.0, [
    attention(4, 1, 64, 128, 0.3, 0.4, 3, (32, 200000.0, 1.0), (64, 70), dense(192, 1.0)),
    hgrn2(2, 128, 64, None),
    attention(2, 2, 128, 64, 0.2, 0.7, 2, None, (130, 2), dense(96, 3.0)),
    attention(8, 1, 64, 128, 0.3, 0.2, 3, (32, 200000.0, 1.0), (100, 0), None, kv_from=0)])
CONFIGS = {"A": L_A, "B": L_B, "C": L_C}

# factor by the last part of a tensor's name (a drawn matrix of fan-in K has entries of about 0.02)
_BOOST = {"embed": 40.0, "head": 10.0, "g": 20.0, "f": 12.0, "gate": 15.0, "up": 15.0}
_DEFAULT_BOOST = 6.0


def _boost(name: str, t: torch.Tensor, sharp: bool = True) -> torch.Tensor:
    """``sharp`` False leaves the attention's scores of order one: bfloat16 runs are compared on such weights, since with
    scores of tens the rounding of a query decides which key carries a row."""
    last = name.rsplit(".", 1)[-1]
    if name.endswith("q.norm") or name.endswith("k.norm"):
        return (t.float() * (2.2 if sharp else 1.0)).to(t.dtype)          # q and k are unit vectors times this weight
    if t.dim() < 2 or last == "conv":
        return t
    return (t.float() * _BOOST.get(last, _DEFAULT_BOOST)).to(t.dtype)


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
        _FOLDERS[key] = write_folder(tempfile.mkdtemp(prefix=f"cima_lipizen_{name}_"), CONFIGS[name], seed, sharp)
    return _FOLDERS[key]


def plain_weights(name: str, seed: int = 0, sharp: bool = True):
    """(config dict, tensors in float64) of a folder, read without the package."""
    from lipizen_plain import read_folder
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
