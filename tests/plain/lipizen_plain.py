"""Plain, slow implementation of the Lipizen decoder: the oracle of its tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 by default.  It shares no code
with the ``cima_b200`` package: the configuration is a plain dict with config.json's own keys, the weights a
plain dict name -> tensor (``read_folder`` reads both from a model folder with nothing but the standard library
and torch).

The design in this file's notation (T tokens of one sequence, width W, t a position counted from 0):

  x_t   = E[tok_t]
  N(z)  = z split into n equal parts, each part / sqrt(mean(part^2) + eps), the whole times w
  x    <- N1(a x + mixer(x));   x <- N2(a x + ff(x))   (second line only where the layer has a feed-forward)
  logits = c tanh(H N_f(x) / c)

  mixer "attention" (differential):  per query head two maps (q1, k1), (q2, k2) over one v.  q, k, v projected, then a
        causal convolution over time per channel (y_t = sum_j w[:, j] u_(t - taps + 1 + j)), then q and k normed per
        head and map (rms over dim, times a shared weight), then rotated on their first r dims (pairs (i, i + r/2),
        angle t * base^(-2i/r) / factor).  Key j is seen from i when j <= i and (i - j < size or j < keep_first).
        A_m = softmax(q_m . k_m * scale) v;  lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + d;
        o = rms(A_1 - lambda A_2) * (1 - d) per head, times sigmoid(W_g h) (one number a head), then W_o.
        A layer with ``kv_from`` j takes layer j's finished keys and values instead of making its own.
  mixer "hgrn2":  q = silu(W_q h), f = l + (1 - l) sigmoid(W_f h + b), v = W_v h;  per head S <- diag(f) S + (1 - f) v^T,
        o = S^T q;  rms(o) * w per head, then W_o
  ff "dense":  g = min(W_g h, L), u = clamp(W_u h, -L, L);  W_d (g sigmoid(1.702 g) (u + 1))
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch


# ---------------------------------------------------------------------------------------------- files
def read_folder(folder: str, dtype=torch.float64):
    """(config dict, {name: tensor}) of a model folder; floating tensors in ``dtype``, integer ones as they are."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64, "I32": torch.int32,
             "I64": torch.int64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, out


# ---------------------------------------------------------------------------------------------- small pieces
def plain_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def plain_group_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """Every row in ``groups`` equal consecutive parts, each divided by its own root mean square; the whole times w."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    return plain_rms(parts, eps).reshape(T, W) * w


def plain_causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the first row."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def plain_rotate(x: torch.Tensor, dims: int, base: float, factor: float, first_position: int = 0) -> torch.Tensor:
    """x [T, heads, dim]: the first ``dims`` values of every head rotate, value i with value i + dims / 2, by the angle
    position * base^(-2 i / dims) / factor; the rest pass."""
    if dims == 0:
        return x
    T = x.shape[0]
    half = dims // 2
    out = x.clone()
    for t in range(T):
        p = first_position + t
        for i in range(half):
            a = p * (base ** (-2.0 * i / dims)) / factor
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, i], x[t, :, i + half]
            out[t, :, i] = u * c - v * s
            out[t, :, i + half] = v * c + u * s
    return out


def plain_visible(i: int, j: int, size: int, keep_first: int) -> bool:
    """``size`` 0: no window, every earlier position is seen."""
    return j <= i and (size <= 0 or i - j < size or j < keep_first)


def plain_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, size: int, keep_first: int):
    """q, k [T, dim], v [T, vdim] of one head and map -> [T, vdim]."""
    T = q.shape[0]
    out = torch.zeros((T, v.shape[1]), dtype=q.dtype)
    for i in range(T):
        seen = [j for j in range(T) if plain_visible(i, j, size, keep_first)]
        s = torch.stack([(q[i] * k[j]).sum() * scale for j in seen])
        p = torch.softmax(s, dim=0)
        out[i] = (p[:, None] * v[seen]).sum(dim=0)
    return out


def plain_keys_values(h, W, m: dict, eps: float):
    """A layer's finished keys [T, kv_heads, 2, dim] (convolved, normed, rotated) and values [T, kv_heads, vdim]
    (convolved only)."""
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k, v = h @ W["k"].T, h @ W["v"].T
    if m.get("conv"):
        k, v = plain_causal_conv(k, W["k.conv"]), plain_causal_conv(v, W["v.conv"])
    k, v = k.reshape(T, G * 2, dim), v.reshape(T, G, vdim)
    k = plain_rms(k, eps) * W["k.norm"]
    rot = m.get("rot") or {}
    k = plain_rotate(k, rot.get("dims", 0), rot.get("base", 1.0), (rot.get("scaling") or {}).get("factor", 1.0))
    return k.reshape(T, G, 2, dim), v


def plain_diff_attention(h, W, m: dict, eps: float, keys_values=None):
    """The differential attention mixer; ``keys_values`` (another layer's, from ``plain_keys_values``) where the layer
    has none of its own."""
    H, G, dim, vdim, d = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    T = h.shape[0]
    q = h @ W["q"].T
    if m.get("conv"):
        q = plain_causal_conv(q, W["q.conv"])
    q = plain_rms(q.reshape(T, H * 2, dim), eps) * W["q.norm"]
    rot = m.get("rot") or {}
    q = plain_rotate(q, rot.get("dims", 0), rot.get("base", 1.0), (rot.get("scaling") or {}).get("factor", 1.0)).reshape(T, H, 2, dim)
    k, v = keys_values if keys_values is not None else plain_keys_values(h, W, m, eps)
    lam = math.exp(float((W["lq1"] * W["lk1"]).sum())) - math.exp(float((W["lq2"] * W["lk2"]).sum())) + d
    gate = torch.sigmoid(h @ W["g"].T)                         # [T, H]
    mask = m.get("mask") or {}
    size, keep = mask.get("size") or 0, mask.get("keep_first") or 0
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        a1 = plain_softmax_attention(q[:, hh, 0], k[:, g, 0], v[:, g], m["scale"], size, keep)
        a2 = plain_softmax_attention(q[:, hh, 1], k[:, g, 1], v[:, g], m["scale"], size, keep)
        o = plain_rms(a1 - lam * a2, eps) * (1.0 - d)
        heads.append(o * gate[:, hh:hh + 1])
    return torch.cat(heads, dim=1) @ W["o"].T


def plain_hgrn2(h, W, m: dict, eps: float):
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    z = h @ W["q"].T
    q = (z * torch.sigmoid(z)).reshape(T, H, dim)
    low = W["lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ W["f"].T + W["f.b"])).reshape(T, H, dim)
    v = (h @ W["v"].T).reshape(T, H, vdim)
    S = torch.zeros((H, dim, vdim), dtype=h.dtype)
    outs = []
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        outs.append(torch.einsum("hdv,hd->hv", S, q[t]))
    o = plain_rms(torch.stack(outs), eps) * W["norm"]          # [T, H, vdim]
    return o.reshape(T, H * vdim) @ W["o"].T


def plain_dense_ff(h, W, limit: float):
    g = torch.clamp(h @ W["gate"].T, max=limit)
    u = torch.clamp(h @ W["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W["down"].T


# ---------------------------------------------------------------------------------------------- the model
def _sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def plain_forward(cfg: dict, weights: dict, ids, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    eps, groups, alpha = cfg["norm"]["eps"], cfg["norm"].get("groups", 1), cfg["postln_alpha"]
    x = weights["embed"][torch.as_tensor(ids, dtype=torch.long)]
    streams, kept = [], {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m, W = layer["mixer"], _sub(weights, p + "mix.")
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = plain_keys_values(x, W, m, eps)
            y = plain_diff_attention(x, W, m, eps, kept[i if src is None else src])
        elif layer["type"] == "hgrn2":
            y = plain_hgrn2(x, W, m, eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = plain_group_norm(alpha * x + y, weights[p + "norm1"], groups, eps)
        if layer.get("mlp") is not None:
            y = plain_dense_ff(x, _sub(weights, p + "mlp."), layer["mlp"]["limit"])
            x = plain_group_norm(alpha * x + y, weights[p + "norm2"], groups, eps)
        streams.append(x)
    logits = plain_group_norm(x, weights["final.norm"], groups, eps) @ weights["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if return_layers else logits
