"""Differential attention over the paged cache (mixer kind ``diff_attention``): every query head computes two softmax
maps over the same values and subtracts them.

    q = conv(W_q h)  [heads, 2, dim];   k = conv(W_k h)  [kv_heads, 2, dim];   v = conv(W_v h)  [kv_heads, v_dim]
          conv: a causal convolution over time on each channel (``taps`` taps, zeros before the start, no bias)
    q, k <- rms(q), rms(k) over dim per head and map, times a weight [dim] (one for q, one for k); then rotated
    A_m  = softmax(q_m . k_m * scale) v      m = 1, 2;  key j is seen from i when j <= i and (i - j < window or j < keep_first)
    o    = rms(A_1 - lambda A_2) * (1 - diff) * sigmoid(W_g h)[head];    y = W_o o
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff      one number for the layer

W_g's rows stand behind q | k | v in the same matrix product and pass through the convolution unchanged (taps 0, ..., 0, 1).
Head h reads key head h // (heads / kv_heads).  The two maps run as one grouped-query attention over 2 * heads query
heads and 2 * kv_heads key heads: key head 2 g + m is map m of key head g, the query heads are laid out so that the
heads that read it stand together (block g holds map 1 of its heads, then map 2), and ``v_group = 2`` tells the
kernels that two neighbouring key heads share a value head.  A head's size in a step's rows and in the cache is the
larger of dim and v_dim rounded up to 16; the rows of W_q, W_k, W_v that pad a head are zero.  Per sequence the mixer keeps
the projections' newest ``taps - 1`` rows (the convolution's state).  A layer with ``cache_from`` has no k and v of
its own and reads that site's pages.  The kept first positions make a window's ring of pages impossible, so a layer
with ``keep_first`` keeps every page.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

from ..cache.kv import KVRequest
from ..config.specs import ShortConvSpec
from ..weights.loader import TensorSpec
from .linear import Linear
from .registry import build_position, register_mixer
from .short_conv import ShortConv


class DiffAttention:
    def __init__(self, spec, layer: int, rt):
        p = spec.params
        self.heads, self.kv_heads, self.dim, self.vdim = spec.n_heads, spec.n_kv_heads, spec.head_dim, int(p["v_dim"])
        self.diff, self.eps, self.taps = float(p["diff"]), float(p["eps"]), int(p.get("taps", 1))
        self.keep_first = int(p.get("keep_first", 0))
        if min(self.heads, self.kv_heads, self.dim, self.vdim) <= 0:
            raise ValueError("diff_attention: heads, key heads, key size and value size must be positive")
        if self.heads % self.kv_heads:
            raise ValueError(f"diff_attention: {self.heads} heads are not a multiple of {self.kv_heads} key heads")
        self.hd = -(-max(self.dim, self.vdim) // 16) * 16
        if self.hd > 256:
            raise ValueError(f"diff_attention: key size {self.dim} and value size {self.vdim} must be at most 256")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.writes = spec.cache_from is None
        self.rep = self.heads // self.kv_heads
        self.position = build_position(spec.position, rt)
        self.nq, self.nk, self.nv = 2 * self.heads, 2 * self.kv_heads, self.kv_heads       # heads of a step's rows
        if not self.writes:
            self.nk = self.nv = 0
        self.channels = (self.nq + self.nk + self.nv) * self.hd
        # the gate's rows stand behind q | k | v in the same product (up to a multiple of 8 with zero rows, so that a row of
        # the result keeps its 16-byte alignment); through the convolution they pass with the taps 0, ..., 0, 1
        self.gate_rows = -(-self.heads // 8) * 8
        self.row = self.channels + self.gate_rows
        self.conv = ShortConv(ShortConvSpec(channels=self.row, taps=self.taps), rt) if self.taps > 0 else None      # 0 taps: none
        self.proj = self.out = self.q_norm = self.k_norm = None
        self.lam = 0.0
        self._lam_vectors = None

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _n(prefix, names, key, tail=""):
        return f"{prefix}{names[key]}{tail}{names.get('suffix', '.weight')}"

    def _kinds(self):
        """(key, heads of the model, size of a head) of the projections this layer owns."""
        out = [("q", 2 * self.heads, self.dim)]
        if self.writes:
            out += [("k", 2 * self.kv_heads, self.dim), ("v", self.kv_heads, self.vdim)]
        return out

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        W = self.spec.hidden
        p: Dict[str, TensorSpec] = {}
        for key, heads, size in self._kinds():
            p[self._n(prefix, names, key)] = TensorSpec((heads * size, W))
            if self.conv is not None:
                p[self._n(prefix, names, key, ".conv")] = TensorSpec((heads * size, self.taps), std=0.3)
            if key != "v":
                p[self._n(prefix, names, key, ".norm")] = TensorSpec((self.dim,), init="ones_normal")
        for key in ("lq1", "lk1", "lq2", "lk2"):
            p[self._n(prefix, names, key)] = TensorSpec((self.dim,), std=0.1)
        p[self._n(prefix, names, "g")] = TensorSpec((self.heads, W))
        p[self._n(prefix, names, "o")] = TensorSpec((W, self.heads * self.vdim))
        return p

    def _q_order(self) -> torch.Tensor:
        """Row-block order of W_q: position g * 2 rep + m * rep + i holds map m of head g * rep + i."""
        order = [2 * (g * self.rep + i) + m for g in range(self.kv_heads) for m in range(2) for i in range(self.rep)]
        return torch.tensor(order, dtype=torch.long)

    def _padded(self, t: torch.Tensor, heads: int, size: int, order=None) -> torch.Tensor:
        """[heads * size, K] -> [heads * hd, K]: heads in ``order``, each followed by zero rows up to the cache's head size."""
        t = t.view(heads, size, -1)
        if order is not None:
            t = t[order.to(t.device)]
        if size == self.hd:
            return t.reshape(heads * self.hd, -1)
        out = torch.zeros((heads, self.hd, t.shape[2]), dtype=t.dtype, device=t.device)
        out[:, :size] = t
        return out.view(heads * self.hd, -1)

    def _unpadded(self, t: torch.Tensor, heads: int, size: int, order=None) -> torch.Tensor:
        t = t.view(heads, self.hd, -1)[:, :size]
        if order is not None:
            back = torch.empty_like(order)
            back[order] = torch.arange(order.numel())
            t = t[back.to(t.device)]
        return t.reshape(heads * size, -1)

    def load(self, tensors, prefix: str, names: Dict[str, str]) -> None:
        rt = self.rt
        order = self._q_order()
        mats, taps = [], []
        for key, heads, size in self._kinds():
            o = order if key == "q" else None
            mats.append(self._padded(tensors[self._n(prefix, names, key)], heads, size, o))
            if self.conv is not None:
                taps.append(self._padded(tensors[self._n(prefix, names, key, ".conv")].float(), heads, size, o))
        g = tensors[self._n(prefix, names, "g")]
        gate = torch.zeros((self.gate_rows, g.shape[1]), dtype=g.dtype, device=g.device)
        gate[:self.heads] = g
        self.proj = Linear(mats + [gate], None, rt)
        if self.conv is not None:
            through = torch.zeros((self.gate_rows, self.taps), dtype=torch.float32, device=taps[0].device)
            through[:, -1] = 1.0
            self.conv.load({"w": torch.cat(taps + [through])}, "w")
        self.q_norm = rt.vector(tensors[self._n(prefix, names, "q", ".norm")])
        self.k_norm = rt.vector(tensors[self._n(prefix, names, "k", ".norm")]) if self.writes else self.q_norm
        self._lam_vectors = [rt.vector(tensors[self._n(prefix, names, k)]) for k in ("lq1", "lk1", "lq2", "lk2")]
        a, b, c, d = (v.double().cpu() for v in self._lam_vectors)
        self.lam = math.exp(float((a * b).sum())) - math.exp(float((c * d).sum())) + self.diff
        self.out = Linear(tensors[self._n(prefix, names, "o")], None, rt)

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        out, r = {}, 0
        order = self._q_order()
        taps = self.conv.weight.t() if self.conv is not None else None
        for key, heads, size in self._kinds():
            rows = heads * self.hd
            o = order if key == "q" else None
            out[self._n(prefix, names, key)] = self._unpadded(self.proj.weight[r:r + rows], heads, size, o)
            if taps is not None:
                out[self._n(prefix, names, key, ".conv")] = self._unpadded(taps[r:r + rows], heads, size, o)
            r += rows
        out[self._n(prefix, names, "q", ".norm")] = self.q_norm
        if self.writes:
            out[self._n(prefix, names, "k", ".norm")] = self.k_norm
        for k, v in zip(("lq1", "lk1", "lq2", "lk2"), self._lam_vectors):
            out[self._n(prefix, names, k)] = v
        out[self._n(prefix, names, "g")] = self.proj.weight[r:r + self.heads]
        out[self._n(prefix, names, "o")] = self.out.weight
        return out

    def nbytes(self) -> int:
        return (self.proj.nbytes() + self.out.nbytes() + (self.conv.nbytes() if self.conv is not None else 0)
                + (self.q_norm.numel() + self.k_norm.numel() + 4 * self.dim) * 4)

    def scratch_row(self) -> int:
        return 2 * self.row + self.nq * self.hd + self.heads * self.vdim

    graph_safe = True

    @property
    def short_context(self) -> int:
        from ..kernels import short_context
        return short_context(self.hd)

    # ------------------------------------------------------------------ cache
    def cache_requests(self, site: int) -> List[object]:
        reqs: List[object] = list(self.conv.cache_requests(site)) if self.conv is not None else []
        if self.writes:
            # kept first positions live below the window: every page stays (a ring would hand their pages on);
            # ``cache_window`` is the widest mask of the layers that read these pages, where the spec gives it
            own = 0 if self.keep_first > 0 else self.spec.window
            reqs.append(KVRequest(2 * self.kv_heads, self.hd, int(self.spec.params.get("cache_window", own))))
        return reqs

    # ------------------------------------------------------------------ step
    def forward(self, h, x: torch.Tensor, batch, cache, site: int, next_norm=None):
        return self.out.accumulate(self._attend(h, batch, cache, site), x, next_norm)

    def produce(self, h, batch, cache, site: int) -> torch.Tensor:
        """The mixer's output as float32 rows of its own (what ``forward`` adds into x)."""
        return self.out.logits(self._attend(h, batch, cache, site))

    def _attend(self, h, batch, cache, site: int) -> torch.Tensor:
        s, K_, rt = self.spec, self.rt.kernels, self.rt
        if hasattr(h, "tensor"):
            h = h.tensor()
        rows = h.shape[0]
        kv = cache.layer_kv(site)
        raw = self.proj.store(h)                                      # [rows, q | k | v | gate] (no k, v where the layer reads another's)
        if self.conv is None:
            qkv = raw
        else:
            qkv = rt.empty(rows, self.row)
            conv_state = cache.state[self.conv.state_name(site)] if self.taps > 1 else None
            K_.short_conv(raw, self.conv.weight, conv_state, batch, qkv, add_input=False)
        K_.rope_append(qkv, self.position.inv_freq, self.position.rotary_dim, batch.row_pos, batch.row_seq, batch.seq_slot,
                       batch.seq_len, kv if self.writes else None, self.nq, self.nk, self.hd, v_heads=self.nv,
                       qk_norm=(self.q_norm, self.k_norm, self.dim, self.eps))
        att = rt.empty(rows, self.nq * self.hd)
        from_cache = (not batch.prefill) or not self.writes
        K_.attention(qkv, kv, batch, att, self.nq, 2 * self.kv_heads, self.hd, s.scale, s.window, from_cache,
                     after_append=self.writes, keep_first=self.keep_first, v_group=2)
        o = rt.empty(rows, self.heads * self.vdim)
        K_.diff_combine(att, qkv[:, self.channels:self.channels + self.heads], o, self.heads, self.rep, self.hd, self.vdim, self.lam, 1.0 - self.diff, self.eps)
        return o


register_mixer("diff_attention", DiffAttention)
