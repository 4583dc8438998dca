"""Grouped-query causal attention over the paged cache, with optional window.

forward: qkv = h Wqkv^T + b  ->  rotate q, k and append k, v to the layer's pages  ->
attention (prefill: over the step's own keys; decode: over the cache)  ->  x += att Wo^T.
Formulas and order as the reference's layer loop, steps 2-7 (src/models/transformer.rs:1039-1264):
bias before rotation, rotation before caching, scale = spec.scale, head h reads kv head
h / (heads / kv_heads), no output bias unless the spec says so.

Every size (heads, kv heads, head_dim, window, scale, bias flags) is a field of the spec.  Two more are ``params``:
``v_dim``, a value size that differs from the key size, and ``sink``, a number of entries of score 0 that carry no
value and join every row's softmax denominator (1: p_j = exp(s_j) / (1 + sum exp(s))); ``keep_first``: with a window, a
sequence's first so many positions stay visible below it, at their own positions (such a layer keeps every page: a ring
would hand the first pages on).  A position encoding whose pairs are neighbours (``interleaved``) is served by
permuting the rows of W_q and W_k at load, alike in every head, which leaves every score as it is; a position
encoding's ``amplitude`` multiplies sine and cosine in the rotating kernel.  Keys and values live in the
cache at one size, the larger of the two rounded up to 16: the rows of W_q, W_k, W_v (and the columns of W_o) that
pad a head are zero, so scores and outputs are what the unpadded sizes give.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.kv import KVRequest
from ..weights.loader import TensorSpec
from .linear import Linear
from .registry import build_position, register_mixer


class Attention:
    def __init__(self, spec, layer: int, rt):
        self.dim, self.vdim = spec.head_dim, int(spec.params.get("v_dim", spec.head_dim))
        self.sink = float(spec.params.get("sink", 0.0))
        self.keep_first = int(spec.params.get("keep_first", 0)) if spec.window else 0
        self.padded = self.dim != self.vdim or self.dim % 16 != 0
        self.hd = -(-max(self.dim, self.vdim) // 16) * 16 if self.padded else self.dim      # a head's size in a step's rows and in the cache
        if min(self.dim, self.vdim) <= 0 or self.hd > 256:
            raise ValueError(f"attention: key size {self.dim} and value size {self.vdim} must be positive, at most 256")
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"attention: {spec.n_heads} heads are not a multiple of {spec.n_kv_heads} kv heads")
        if self.padded and (spec.qkv_bias or spec.out_bias):
            raise ValueError(f"attention: head_dim {self.dim} must be a multiple of 16 and equal to the value size {self.vdim} "
                             f"where the projections have biases (heads are padded in the cache only without biases)")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.position = build_position(spec.position, rt)
        # (a position part registered elsewhere may offer neither: half-split pairs, amplitude 1)
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        self.amplitude = float(getattr(self.position, "amplitude", 1.0))
        self.qd = spec.n_heads * self.hd
        self.kvd = spec.n_kv_heads * self.hd
        self.qkv = None
        self.out = None

    # ------------------------------------------------------------------ weights
    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        s = self.spec
        sfx = names.get("suffix", ".weight")
        p: Dict[str, TensorSpec] = {}
        for key, rows in (("q", s.n_heads * self.dim), ("k", s.n_kv_heads * self.dim), ("v", s.n_kv_heads * self.vdim)):
            p[f"{prefix}{names[key]}{sfx}"] = TensorSpec((rows, s.hidden))
            if s.qkv_bias:
                p[f"{prefix}{names[key]}.bias"] = TensorSpec((rows,))
        p[f"{prefix}{names['o']}{sfx}"] = TensorSpec((s.hidden, s.n_heads * self.vdim))
        if s.out_bias:
            p[f"{prefix}{names['o']}.bias"] = TensorSpec((s.hidden,))
        return p

    def _pad_rows(self, t: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        """[heads * size, K] -> [heads * hd, K]: every head's rows followed by zero rows up to the cache's head size."""
        if size == self.hd:
            return t
        out = torch.zeros((heads, self.hd, t.shape[1]), dtype=t.dtype, device=t.device)
        out[:, :size] = t.view(heads, size, t.shape[1])
        return out.view(heads * self.hd, t.shape[1])

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str, names: Dict[str, str]) -> None:
        s = self.spec
        sfx = names.get("suffix", ".weight")
        bias = None
        if s.qkv_bias:
            bias = torch.cat([tensors[f"{prefix}{names[k]}.bias"].float() for k in ("q", "k", "v")])
        sizes = {"q": (s.n_heads, self.dim), "k": (s.n_kv_heads, self.dim), "v": (s.n_kv_heads, self.vdim)}

        def rows(k):
            t = tensors[f"{prefix}{names[k]}{sfx}"]
            if k != "v" and self.interleaved:
                t = t[self.position.to_half_split(sizes[k][0], self.dim).to(t.device)]
            return self._pad_rows(t, *sizes[k])

        if self.interleaved and s.qkv_bias:
            raise ValueError("attention: neighbouring rotary pairs with biases on q and k are not implemented")
        self.qkv = Linear([rows(k) for k in ("q", "k", "v")], bias, self.rt)
        ob = tensors[f"{prefix}{names['o']}.bias"] if s.out_bias else None
        wo = tensors[f"{prefix}{names['o']}{sfx}"]
        if self.vdim != self.hd:
            wo = self._pad_rows(wo.t().contiguous(), s.n_heads, self.vdim).t().contiguous()
        self.out = Linear(wo, ob, self.rt)

    def nbytes(self) -> int:
        return self.qkv.nbytes() + self.out.nbytes()

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        """The tensors of ``plan`` back out of the stacked matrices, as they are kept on the device."""
        out: Dict[str, torch.Tensor] = {}
        s, sfx = self.spec, names.get("suffix", ".weight")
        r = 0
        for key, rows, heads, size in (("q", self.qd, s.n_heads, self.dim), ("k", self.kvd, s.n_kv_heads, self.dim),
                                       ("v", self.kvd, s.n_kv_heads, self.vdim)):
            w = self.qkv.weight[r:r + rows]
            w = w if size == self.hd else w.view(heads, self.hd, -1)[:, :size].reshape(heads * size, -1)
            if key != "v" and self.interleaved:
                order = self.position.to_half_split(heads, size).to(w.device)
                back = torch.empty_like(w)
                back[order] = w
                w = back
            out[f"{prefix}{names[key]}{sfx}"] = w
            if self.qkv.bias is not None:
                out[f"{prefix}{names[key]}.bias"] = self.qkv.bias[r:r + rows]
            r += rows
        wo = self.out.weight
        out[f"{prefix}{names['o']}{sfx}"] = wo if self.vdim == self.hd else wo.view(-1, s.n_heads, self.hd)[:, :, :self.vdim].reshape(wo.shape[0], -1)
        if self.out.bias is not None:
            out[f"{prefix}{names['o']}.bias"] = self.out.bias
        return out

    def scratch_row(self) -> int:
        """Values of the widest activation row a step of this part holds (its q | k | v row)."""
        return self.qd + 2 * self.kvd

    graph_safe = True              # a decode step reads nothing of the batch on the host

    @property
    def short_context(self) -> int:
        """Positions up to which this mixer's decode kernel takes another road than for long contexts (none if 0):
        the stepper records decode steps for such contexts apart (``StepBatch.max_len`` is their bound)."""
        from ..kernels import short_context
        return short_context(self.hd)

    # ------------------------------------------------------------------ cache
    def cache_requests(self, site: int) -> List[object]:
        if self.spec.cache_from is not None:
            return []
        return [KVRequest(self.spec.n_kv_heads, self.hd, 0 if self.keep_first > 0 else self.spec.window)]

    # ------------------------------------------------------------------ step
    takes_pending_norm = True      # h may be a NormedInput: the q/k/v product folds the norm in when it can
    takes_next_norm = True         # forward(..., next_norm=): the norm that will read x next, for its last product

    def forward(self, h, x: torch.Tensor, batch, cache, site: int, next_norm=None):
        return self.out.accumulate(self._attend(h, batch, cache, site), x, next_norm)

    def produce(self, h, batch, cache, site: int) -> torch.Tensor:
        """The mixer's output as float32 rows of its own (what ``forward`` adds into x)."""
        return self.out.logits(self._attend(h, batch, cache, site))

    def _attend(self, h, batch, cache, site: int) -> torch.Tensor:
        s, K_ = self.spec, self.rt.kernels
        kv = cache.layer_kv(site)
        writes = s.cache_from is None
        rows = h.shape[0]
        if (not batch.prefill and writes and self.qkv._skinny(rows) and kv.storage.dtype is torch.bfloat16
                and self.position.rotary_dim == self.hd and self.amplitude == 1.0 and hasattr(K_, "qkv_rope")):
            # decoding: projection, rotation and the append to the cache as one kernel
            qkv = self.rt.empty(rows, self.qd + 2 * self.kvd)
            if self.qkv._folds(h, rows):
                K_.qkv_rope(h.xw, self.qkv.weight, self.qkv.bias, qkv, self.position.inv_freq, batch.row_pos,
                            batch.row_seq, batch.seq_slot, kv, s.n_heads, s.n_kv_heads, self.hd,
                            norm=(h.ssq, h.norm.spec.eps))
            else:
                K_.qkv_rope(h.tensor() if hasattr(h, "tensor") else h, self.qkv.weight, self.qkv.bias, qkv,
                            self.position.inv_freq, batch.row_pos, batch.row_seq, batch.seq_slot, kv, s.n_heads,
                            s.n_kv_heads, self.hd)
        else:
            qkv = self.qkv.store(h)
            if self.amplitude != 1.0:
                K_.rope_append(qkv, self.position.inv_freq, self.position.rotary_dim, batch.row_pos, batch.row_seq,
                               batch.seq_slot, batch.seq_len, kv if writes else None, s.n_heads, s.n_kv_heads, self.hd,
                               amplitude=self.amplitude)
            else:
                K_.rope_append(qkv, self.position.inv_freq, self.position.rotary_dim, batch.row_pos, batch.row_seq,
                               batch.seq_slot, batch.seq_len, kv if writes else None, s.n_heads, s.n_kv_heads, self.hd)
        att = self.rt.empty(h.shape[0], self.qd)
        from_cache = (not batch.prefill) or not writes
        more = {}
        if self.sink:
            more["sink"] = self.sink
        if self.keep_first:
            more["keep_first"] = self.keep_first
        K_.attention(qkv, kv, batch, att, s.n_heads, s.n_kv_heads, self.hd, s.scale, s.window, from_cache,
                     after_append=True, **more)
        return att


register_mixer("attention", Attention)
