"""Plain, slow implementation of the Netezen decoder: the oracle of its tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 by default.  It shares no code
with the ``cima_b200`` package: the configuration is a plain dict with config.json's own keys, the weights a
plain dict name -> tensor (``read_folder`` reads both from a model folder with nothing but the standard library
and torch).

The design in this file's notation (T tokens of one sequence, width W, t a position counted from 0, m the config's
``residual_mult``):

  e_t      = E[tok_t]
  N(z; w)  = z / sqrt(mean(z^2) + eps) * (1 + w)                 (a latent's norm multiplies by w itself)
  one stream:      x <- x + m mixer(N1(x));   x <- x + m ff(N2(x))
  S streams:       X_1 = ... = X_S = e.  For sublayer q with vectors a_q, b_q [S] and a matrix C_q [S, S]:
                   u = sum_s a_q[s] X_s;  y = sublayer(N_q(u));  X_t <- sum_s C_q[s, t] X_s + m b_q[t] y   (all t from the old X)
                   and behind the last layer x = sum_s X_s
  logits   = E N_f(x)

  rotation: of a head's first r values, neighbours (2i, 2i + 1) form a pair that turns by the angle t f_i,
        f_i = base^(-2i / r).  With "scaling" {factor c, original L, fast, slow}: d(z) = r ln(L / (2 pi z)) / (2 ln base),
        lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), r - 1), g_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1);
        f_i <- g_i f_i / c + (1 - g_i) f_i, and sine and cosine are multiplied by 0.1 ln(c) + 1.
  mixer "attention":  q, k, v projected without bias; query head h reads key head h // (H / G); q and k rotated;
        key j is seen from i when j <= i and (i - j < size or j < keep_first); softmax(q . k * scale) v; W_o.
  mixer "latent_attention":  c_q = rms(W_dq h) * w_q,  q = W_uq c_q (with q_rank 0: q = W_q h), a head = [dim plain | rot_dim rotated];
        W_dkv h = [kv_rank | rot_dim]: c = rms(first part) * w_c, the second part rotated is one key part for all heads;
        head h: k = [W_uk[h] c | shared rotated part], v = W_uv[h] c;  key j is seen from i when 0 <= i - j < size;
        p_j = exp(s_j) / (exp(sink_h) + sum_j' exp(s_j')),  s = q . k * scale;  W_o.
  ff "dense":  W_down relu(W_up h)^2
  ff "moe":    z = W_r h, s = softmax(z); the ``top`` experts of largest s + correction; weights s_e / (sum of the chosen s + 1e-20);
        expert: g = min(W_g h, L), u = clamp(W_u h, -L, L);  W_d (g sigmoid(1.702 g) (u + 1));
        a shared expert of the same form (its own L) for every token, times sigmoid(w_sg . h)
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


def plain_frequencies(rot: dict, dtype=torch.float64):
    """(frequencies [dims / 2], the factor of sine and cosine) of a rotation's description."""
    r, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / r) for i in range(r // 2)], dtype=dtype)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    c, L = float(sc["factor"]), float(sc["original"])

    def d(z):
        return r * math.log(L / (2.0 * math.pi * z)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(sc["fast"]))), 0)
    hi = min(math.ceil(d(float(sc["slow"]))), r - 1)
    g = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(r // 2)], dtype=dtype)
    return g * f / c + (1.0 - g) * f, 0.1 * math.log(c) + 1.0


def plain_rotate(x: torch.Tensor, rot: dict, first_position: int = 0) -> torch.Tensor:
    """x [T, heads, n]: the first rot["dims"] values of every head turned pair by pair, (2i, 2i + 1) by t f_i."""
    r = int(rot["dims"])
    f, amp = plain_frequencies(rot, x.dtype)
    t = torch.arange(first_position, first_position + x.shape[0], dtype=x.dtype)
    ang = t[:, None] * f[None, :]                               # [T, r / 2]
    cos, sin = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:r:2], x[..., 1:r:2]
    out[..., 0:r:2] = a * cos - b * sin
    out[..., 1:r:2] = b * cos + a * sin
    return out


def plain_visible(i: int, j: int, size: int, keep_first: int) -> bool:
    """Whether the query at position i sees the key at position j (size 0: no window)."""
    return j <= i and (size <= 0 or i - j < size or j < keep_first)


def plain_masked_softmax(s: torch.Tensor, size: int, keep_first: int, sink=None) -> torch.Tensor:
    """s [T, T] scores of one head -> weights over the visible keys; ``sink``: a number whose exponential joins every
    row's denominator and carries nothing."""
    T = s.shape[0]
    p = torch.zeros_like(s)
    for i in range(T):
        js = [j for j in range(T) if plain_visible(i, j, size, keep_first)]
        row = s[i, js]
        top = row.max() if sink is None else torch.maximum(row.max(), sink)
        e = torch.exp(row - top)
        den = e.sum() + (torch.exp(sink - top) if sink is not None else 0.0)
        p[i, js] = e / den
    return p


# ---------------------------------------------------------------------------------------------- mixers
def plain_attention(h: torch.Tensor, W: dict, m: dict) -> torch.Tensor:
    """Grouped-query softmax attention; W holds "q", "k", "v", "o"."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"]))
    q = (h @ W["q"].T).reshape(T, H, D)
    k = (h @ W["k"].T).reshape(T, G, D)
    v = (h @ W["v"].T).reshape(T, G, V)
    if m.get("rot"):
        q, k = plain_rotate(q, m["rot"]), plain_rotate(k, m["rot"])
    mask = m.get("mask") or {}
    size, keep = int(mask.get("size", 0)), int(mask.get("keep_first", 0))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        p = plain_masked_softmax(q[:, a] @ k[:, g].T * float(m["scale"]), size, keep)
        out[:, a] = p @ v[:, g]
    return out.reshape(T, H * V) @ W["o"].T


def plain_latent_attention(h: torch.Tensor, W: dict, m: dict, eps: float) -> torch.Tensor:
    """Attention whose keys and values are projected from one small vector a position; W holds "dq", "dq.norm", "uq",
    "dkv", "dkv.norm", "uk", "uv", "sink", "o"."""
    T = h.shape[0]
    H, D, R, V, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    if int(m.get("q_rank", 0)):
        cq = plain_rms(h @ W["dq"].T, eps) * W["dq.norm"]
        q = (cq @ W["uq"].T).reshape(T, H, D + R)
    else:                                                        # no query latent: the queries straight from the input
        q = (h @ W["q"].T).reshape(T, H, D + R)
    both = h @ W["dkv"].T
    c = plain_rms(both[:, :C], eps) * W["dkv.norm"]
    rot = dict(m["rot"], dims=R)
    shared = plain_rotate(both[:, C:].reshape(T, 1, R), rot)[:, 0]          # [T, R]
    q_rot = plain_rotate(q[:, :, D:], rot)
    k = (c @ W["uk"].T).reshape(T, H, D)
    v = (c @ W["uv"].T).reshape(T, H, V)
    size = int((m.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for a in range(H):
        s = (q[:, a, :D] @ k[:, a].T + q_rot[:, a] @ shared.T) * float(m["scale"])
        sink = W["sink"][a] if "sink" in W else None
        out[:, a] = plain_masked_softmax(s, size, 0, sink) @ v[:, a]
    return out.reshape(T, H * V) @ W["o"].T


# ---------------------------------------------------------------------------------------------- feed-forwards
def plain_dense_ff(h: torch.Tensor, W: dict) -> torch.Tensor:
    return torch.relu(h @ W["up"].T).pow(2) @ W["down"].T


def plain_expert(h: torch.Tensor, gate, up, down, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def plain_route(h: torch.Tensor, router, correction, top: int):
    """(chosen experts [T, top], their weights [T, top]): chosen by softmax score plus correction, weighted by the scores alone."""
    s = torch.softmax(h @ router.T, dim=-1)
    chosen = torch.topk(s + correction, top, dim=-1).indices
    w = torch.gather(s, 1, chosen)
    return chosen, w / (w.sum(dim=-1, keepdim=True) + 1e-20)


def plain_moe(h: torch.Tensor, W: dict, mlp: dict) -> torch.Tensor:
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    limit = float(mlp["expert"]["limit"])
    correction = W["correction"] if "correction" in W else torch.zeros(E, dtype=h.dtype)
    chosen, w = plain_route(h, W["router"], correction, top)
    y = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(chosen[t, j])
            y[t] += w[t, j] * plain_expert(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], limit)[0]
    if mlp.get("shared"):
        sh = plain_expert(h, W["shared.gate"], W["shared.up"], W["shared.down"], float(mlp["shared"]["limit"]))
        y = y + sh * torch.sigmoid(h @ W["shared.sg"].T)
    return y


# ---------------------------------------------------------------------------------------------- the model
def _sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def plain_mixer(h, layer: dict, W: dict, eps: float):
    if layer["type"] == "attention":
        return plain_attention(h, W, layer["mixer"])
    if layer["type"] == "latent_attention":
        return plain_latent_attention(h, W, layer["mixer"], eps)
    raise ValueError(f"unknown mixer '{layer['type']}'")


def plain_ff(h, mlp: dict, W: dict):
    return plain_dense_ff(h, W) if mlp["kind"] == "dense" else plain_moe(h, W, mlp)


def plain_forward(cfg: dict, weights: dict, ids, return_layers: bool = False):
    """Logits [T, vocab] of one sequence; with ``return_layers`` also the stream (the sum of the streams) behind every layer."""
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    E = weights["embed"]
    e = E[torch.as_tensor(ids, dtype=torch.long)]
    S = int(cfg["streams"]) if "streams" in cfg else 0
    X = [e.clone() for _ in range(max(S, 1))]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        L = _sub(weights, f"l{i}.")
        subs = [(1, lambda z: plain_mixer(z, layer, _sub(L, "mix."), eps))]
        if layer.get("mlp"):
            subs.append((2, lambda z: plain_ff(z, layer["mlp"], _sub(L, "mlp."))))
        for q, run in subs:
            if S:
                a, b, C = L[f"hc{q}.in"], L[f"hc{q}.out"], L[f"hc{q}.mix"]
                u = sum(a[s] * X[s] for s in range(S))
                y = run(plain_rms(u, eps) * (1.0 + L[f"norm{q}"]))
                X = [sum(C[s, t] * X[s] for s in range(S)) + m * b[t] * y for t in range(S)]
            else:
                X[0] = X[0] + m * run(plain_rms(X[0], eps) * (1.0 + L[f"norm{q}"]))
        layers.append(sum(X))
    x = plain_rms(sum(X), eps) * (1.0 + weights["final.norm"])
    logits = x @ E.T
    return (logits, torch.stack(layers)) if return_layers else logits
