"""Causal attention over latents, without position encoding or with a rotated key part beside the latent.

Every position keeps ONE vector c of ``kv_rank`` values, c = RMSNorm(W_d u) (its own norm weight); head h's key
and value are k = W_uk[h] c and v = W_uv[h] c, of ``head_dim`` and ``v_dim`` values.  Nothing but c is cached,
and it is cached once (a cache request of one plane): it serves as key and as value.

The step never builds k or v.  Since q.k = q.(W_uk[h] c) = (W_uk[h]^T q).c and sum_s p_s v_s = W_uv[h] (sum_s p_s c_s),

    qa[t, h] = W_uk[h]^T q[t, h]                  the query moved into the latents' space   (kv_rank values)
    ol[t, h] = softmax_s(scale * qa[t, h] . c_s) c_s      attention of all heads over ONE shared "kv head" c
    a[t, h]  = W_uv[h] ol[t, h]                   and out again                               (v_dim values)
    x       += W_o a

so the attention kernels of the grouped-query mixer serve: ``heads`` query heads on one kv head of ``kv_rank``
values whose pages hold one plane.  The step appends its latents first and every row reads the pages, whether
the sequences start or go on.  A layer with ``cache_from`` makes no latents and reads that site's pages with its
own W_uk and W_uv.  Scores and softmax are float32 in every attention kernel; the latent's norm is float32.

Sizes and constants (heads, head_dim, v_dim, kv_rank, scale, the latent norm's eps) are the spec's.

Four options, each off by default (``params``):
  ``rot_dim`` r > 0 (with the spec's ``position`` of r rotary dims): the latent projection has r more rows; their output,
      rotated at the row's position, is one key part for all heads and is cached behind the latent (a position keeps
      kv_rank + r values).  A query head is [head_dim plain | r rotated] and its score q_plain . k_plain + q_rot . k_rot.
      The moved query is [W_uk[h]^T q_plain | q_rot], the attention runs over heads of kv_rank + r values on the one
      shared plane, and the value product reads the first kv_rank values of its result.
  ``q_rank`` > 0: the queries come through a latent of their own, q = W_uq (RMSNorm(W_dq u) * w); W_dq stands in one
      matrix with the latent projection, and one kernel norms both latents, rotates the key part and appends.
  the spec's ``window`` w > 0: a row sees itself and the w - 1 positions before it; the pages form a ring.
  ``head_sink``: a stored number a head (tensor "sink") whose exponential joins the softmax's denominator without a value.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.kv import KVRequest
from ..weights.loader import TensorSpec
from .linear import Linear
from .registry import build_position, register_mixer


class LatentAttention:
    def __init__(self, spec, layer: int, rt):
        p = spec.params
        self.heads, self.dim = spec.n_heads, spec.head_dim
        self.vdim, self.rank, self.latent_eps = int(p["v_dim"]), int(p["kv_rank"]), float(p["latent_eps"])
        if min(self.heads, self.dim, self.vdim, self.rank) <= 0:
            raise ValueError(f"latent_attention: heads {self.heads}, head_dim {self.dim}, v_dim {self.vdim} and kv_rank "
                             f"{self.rank} must be positive")
        self.rot, self.q_rank, self.has_sink = int(p.get("rot_dim", 0)), int(p.get("q_rank", 0)), bool(p.get("head_sink", False))
        self.spec, self.layer, self.rt = spec, layer, rt
        self.own = spec.cache_from is None
        self.extended = bool(self.rot or self.q_rank or self.has_sink or spec.window)
        if self.extended and not self.own:
            raise ValueError("latent_attention: a layer that reads another's latents takes no rotated part, query latent, window or sink")
        self.position = build_position(spec.position, rt) if self.rot else None
        if self.rot and self.position.rotary_dim != self.rot:
            raise ValueError(f"latent_attention: the rotated part has {self.rot} values, its position encoding turns {self.position.rotary_dim}")
        self.qh = self.dim + self.rot              # a query head: plain part, rotated part
        self.kd = self.rank + self.rot             # what a position keeps: latent, rotated key part
        self.qd, self.od = self.heads * self.qh, self.heads * self.vdim
        self.q_up = self.q_norm = self.sink = None
        self.q_latent = None       # W_q (and W_d under it) as one matrix
        self.latent_norm = None    # float32 [kv_rank]
        self.k_up_t = None         # [heads, kv_rank, head_dim]: W_uk's heads, transposed
        self.v_up = None           # [heads, v_dim, kv_rank]
        self.out = None

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _n(prefix, names, key):
        return f"{prefix}{names[key]}{names.get('suffix', '.weight')}"

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        s = self.spec
        if self.q_rank:
            p = {self._n(prefix, names, "q_down"): TensorSpec((self.q_rank, s.hidden)),
                 self._n(prefix, names, "q_norm"): TensorSpec((self.q_rank,), init="ones_normal"),
                 self._n(prefix, names, "q"): TensorSpec((self.qd, self.q_rank), std=self.q_rank ** -0.5)}
        else:
            p = {self._n(prefix, names, "q"): TensorSpec((self.qd, s.hidden))}
        if self.own:
            p[self._n(prefix, names, "latent")] = TensorSpec((self.kd, s.hidden))
            p[self._n(prefix, names, "latent_norm")] = TensorSpec((self.rank,), init="ones_normal")
        p[self._n(prefix, names, "k_up")] = TensorSpec((self.heads * self.dim, self.rank), std=self.rank ** -0.5)
        p[self._n(prefix, names, "v_up")] = TensorSpec((self.od, self.rank), std=self.rank ** -0.5)
        if self.has_sink:
            p[self._n(prefix, names, "sink")] = TensorSpec((self.heads,), std=1.0)
        p[self._n(prefix, names, "o")] = TensorSpec((s.hidden, self.od))
        return p

    def load(self, tensors, prefix: str, names: Dict[str, str]) -> None:
        rt = self.rt
        if self.q_rank:
            mats = [tensors[self._n(prefix, names, "q_down")]]
            self.q_norm = rt.vector(tensors[self._n(prefix, names, "q_norm")])
            self.q_up = Linear(tensors[self._n(prefix, names, "q")], None, rt)
        else:
            mats = [tensors[self._n(prefix, names, "q")]]
        if self.own:
            mats.append(tensors[self._n(prefix, names, "latent")])
            self.latent_norm = rt.vector(tensors[self._n(prefix, names, "latent_norm")])
        if self.has_sink:
            self.sink = rt.vector(tensors[self._n(prefix, names, "sink")])
        self.q_latent = Linear(mats, None, rt)
        del mats
        k_up = rt.matrix(tensors[self._n(prefix, names, "k_up")])
        self.k_up_t = k_up.view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        del k_up
        self.v_up = rt.matrix(tensors[self._n(prefix, names, "v_up")]).view(self.heads, self.vdim, self.rank)
        self.out = Linear(tensors[self._n(prefix, names, "o")], None, rt)
        if len({self.k_up_t.dtype, self.v_up.dtype, rt.dtype}) != 1:
            # a head's projection runs in the activations' dtype (a matrix stored in 32-bit is rounded on the bfloat16 path)
            self.k_up_t, self.v_up = self.k_up_t.to(rt.dtype), self.v_up.to(rt.dtype)

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        first = self.q_rank or self.qd                    # rows of the first matrix of the stacked product
        if self.q_rank:
            out = {self._n(prefix, names, "q_down"): self.q_latent.weight[:first], self._n(prefix, names, "q_norm"): self.q_norm,
                   self._n(prefix, names, "q"): self.q_up.weight}
        else:
            out = {self._n(prefix, names, "q"): self.q_latent.weight[:first]}
        if self.own:
            out[self._n(prefix, names, "latent")] = self.q_latent.weight[first:]
            out[self._n(prefix, names, "latent_norm")] = self.latent_norm
        out[self._n(prefix, names, "k_up")] = self.k_up_t.transpose(1, 2).reshape(self.heads * self.dim, self.rank)
        out[self._n(prefix, names, "v_up")] = self.v_up.reshape(self.od, self.rank)
        if self.has_sink:
            out[self._n(prefix, names, "sink")] = self.sink
        out[self._n(prefix, names, "o")] = self.out.weight
        return out

    def nbytes(self) -> int:
        e = self.k_up_t.element_size()
        return (self.q_latent.nbytes() + self.out.nbytes() + (self.k_up_t.numel() + self.v_up.numel()) * e
                + (self.latent_norm.numel() * 4 if self.own else 0) + (self.q_up.nbytes() + self.q_rank * 4 if self.q_rank else 0))

    def scratch_row(self) -> int:
        return self.qd + self.q_rank + self.kd + 2 * self.heads * self.kd + self.od

    graph_safe = True

    @property
    def short_context(self) -> int:
        from ..kernels import short_context
        return short_context(self.kd)

    # ------------------------------------------------------------------ cache
    def cache_requests(self, site: int) -> List[object]:
        if not self.own:
            return []
        return [KVRequest(n_kv_heads=1, head_dim=self.kd, window=int(self.spec.window), planes=1)]

    # ------------------------------------------------------------------ step
    def forward(self, u, x: torch.Tensor, batch, cache, site: int, next_norm=None):
        if self.extended:
            return self.out.accumulate(self._attend(u, batch, cache, site), x, next_norm)
        K_, rt = self.rt.kernels, self.rt
        if hasattr(u, "tensor"):
            u = u.tensor()
        rows = u.shape[0]
        kv = cache.layer_kv(site)
        ql = self.q_latent.store(u)                                  # [rows, heads * head_dim (+ kv_rank)]
        qa = rt.empty(rows, self.heads * self.rank)
        # (the step's latents go into the pages before the attention reads them: in the same launch for the few rows
        # of a decode step, in one of their own before it otherwise)
        K_.head_linear(ql[:, :self.qd], self.k_up_t, qa,
                       append=(ql[:, self.qd:], self.latent_norm, self.latent_eps, kv, batch) if self.own else None)
        ol = rt.empty(rows, self.heads * self.rank)
        K_.attention(qa, kv, batch, ol, self.heads, 1, self.rank, self.spec.scale, 0, True)
        att = rt.empty(rows, self.od)
        K_.head_linear(ol, self.v_up, att)
        return self.out.accumulate(att, x, next_norm)

    def produce(self, u, batch, cache, site: int) -> torch.Tensor:
        """The mixer's output as float32 rows of its own (what ``forward`` adds into x)."""
        if self.extended:
            return self.out.logits(self._attend(u, batch, cache, site))
        y = torch.zeros((u.shape[0], self.spec.hidden), dtype=torch.float32, device=self.rt.device)
        self.forward(u, y, batch, cache, site)
        return y

    def _attend(self, u, batch, cache, site: int) -> torch.Tensor:
        """The road of the options: [rows, heads * v_dim] in front of W_o."""
        K_, rt, s = self.rt.kernels, self.rt, self.spec
        if hasattr(u, "tensor"):
            u = u.tensor()
        rows = u.shape[0]
        kv = cache.layer_kv(site)
        first = self.q_rank or self.qd
        ql = self.q_latent.store(u)                                  # [rows, (q latent or q) | latent | key part to rotate]
        cq = rt.empty(rows, self.q_rank) if self.q_rank else None
        pos = self.position
        # A prompt that starts reads its own rows (a window's ring of pages does not hold a long prompt): the moved
        # queries are followed by the row's [latent | key part] twice, as the one key head and the one value head of a
        # grouped-query attention.  Rows that go on read the pages.
        own_rows = bool(batch.prefill)
        qa = rt.empty(rows, (self.heads + (2 if own_rows else 0)) * self.kd)
        # both latents normed, the key part rotated, latent and key part into the row's place in the pages
        K_.latent_prepare(ql, first, self.q_norm, cq, self.latent_norm, self.latent_eps, self.rank, self.rot,
                          pos.inv_freq if pos is not None else None, pos.amplitude if pos is not None else 1.0,
                          bool(pos.interleaved) if pos is not None else False, kv, batch,
                          step_rows=(qa, self.heads * self.kd) if own_rows else None)
        q = self.q_up.store(cq) if self.q_rank else ql                # [rows, heads * (head_dim + rot)] (in ql: its first columns)
        K_.head_linear(q, self.k_up_t, qa, a_head=self.qh, out_head=self.kd)
        if self.rot:
            K_.rope_rows(q, self.dim, self.qh, qa, self.rank, self.kd, self.heads, self.rot, pos.inv_freq, pos.amplitude,
                         pos.interleaved, batch.row_pos)
        ol = rt.empty(rows, self.heads * self.kd)
        more = {"head_sink": self.sink} if self.sink is not None else {}
        K_.attention(qa, kv, batch, ol, self.heads, 1, self.kd, s.scale, int(s.window), not own_rows, **more)
        att = rt.empty(rows, self.od)
        K_.head_linear(ol, self.v_up, att, a_head=self.kd, out_head=self.vdim)
        return att


register_mixer("latent_attention", LatentAttention)
