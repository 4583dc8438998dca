"""Linear attention whose forget gate also decides what is written (HGRN2; mixer kind ``gated_recurrence``).

    q = silu(W_q h)   [heads, dim];     v = W_v h   [heads, v_dim]
    f = l + (1 - l) * sigmoid(W_f h + b)                 one gate a head and key channel, l its lower bound
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T;           o_t = S_t^T q_t          per head: no key, no other scale
    y   = W_o ( rms(o over a head's values) * w )         w [v_dim], one for all heads

The state S [heads, dim, v_dim] is float32, starts at zero and travels with the sequence (a ``StateRequest``); a step
walks its rows in order from the state the steps before left, so prompts, pieces of prompts and single tokens are one
path.  q | f | v are one product; SiLU, the gate with its bias and bound, and everything after them are float32 inside the
recurrence kernel.  Sizes (heads, head_dim, ``v_dim``) and the norm's ``eps`` are the spec's.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.kv import StateRequest
from ..weights.loader import TensorSpec
from .linear import Linear
from .registry import register_mixer


class GatedRecurrence:
    def __init__(self, spec, layer: int, rt):
        p = spec.params
        self.heads, self.dim, self.vdim = spec.n_heads, spec.head_dim, int(p["v_dim"])
        self.eps = float(p["eps"])
        if min(self.heads, self.dim, self.vdim) <= 0 or self.dim > 256:
            raise ValueError(f"gated_recurrence: heads {self.heads}, key size {self.dim} (at most 256) and value size {self.vdim} must be positive")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.qd, self.vd = self.heads * self.dim, self.heads * self.vdim
        self.proj = self.out = self.norm = self.bias = self.lower = None

    @staticmethod
    def _n(prefix, names, key):
        return f"{prefix}{names[key]}{names.get('suffix', '.weight')}"

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        H = self.spec.hidden
        return {self._n(prefix, names, "q"): TensorSpec((self.qd, H)), self._n(prefix, names, "f"): TensorSpec((self.qd, H)),
                self._n(prefix, names, "v"): TensorSpec((self.vd, H)), self._n(prefix, names, "o"): TensorSpec((H, self.vd)),
                self._n(prefix, names, "f_bias"): TensorSpec((self.qd,), std=0.5),
                self._n(prefix, names, "lower"): TensorSpec((self.qd,), init="unit"),
                self._n(prefix, names, "norm"): TensorSpec((self.vdim,), init="ones_normal")}

    def load(self, tensors, prefix: str, names: Dict[str, str]) -> None:
        self.proj = Linear([tensors[self._n(prefix, names, k)] for k in ("q", "f", "v")], None, self.rt)
        self.out = Linear(tensors[self._n(prefix, names, "o")], None, self.rt)
        self.bias = self.rt.vector(tensors[self._n(prefix, names, "f_bias")])
        self.lower = self.rt.vector(tensors[self._n(prefix, names, "lower")])
        self.norm = self.rt.vector(tensors[self._n(prefix, names, "norm")])

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        w, out = self.proj.weight, {}
        out[self._n(prefix, names, "q")] = w[:self.qd]
        out[self._n(prefix, names, "f")] = w[self.qd:2 * self.qd]
        out[self._n(prefix, names, "v")] = w[2 * self.qd:]
        out[self._n(prefix, names, "o")] = self.out.weight
        out[self._n(prefix, names, "f_bias")] = self.bias
        out[self._n(prefix, names, "lower")] = self.lower
        out[self._n(prefix, names, "norm")] = self.norm
        return out

    def nbytes(self) -> int:
        return self.proj.nbytes() + self.out.nbytes() + (self.bias.numel() + self.lower.numel() + self.norm.numel()) * 4

    def scratch_row(self) -> int:
        return 2 * self.qd + 4 * self.vd

    graph_safe = True

    @staticmethod
    def state_name(site: int) -> str:
        return f"gated_recurrence.{site}"

    def cache_requests(self, site: int) -> List[object]:
        return [StateRequest(self.state_name(site), (self.heads, self.dim, self.vdim), torch.float32)]

    def forward(self, h, x: torch.Tensor, batch, cache, site: int, next_norm=None):
        return self.out.accumulate(self._normed(h, batch, cache, site), x, next_norm)

    def produce(self, h, batch, cache, site: int) -> torch.Tensor:
        """The mixer's output as float32 rows of its own (what ``forward`` adds into x)."""
        return self.out.logits(self._normed(h, batch, cache, site))

    def _normed(self, h, batch, cache, site: int) -> torch.Tensor:
        K_, rt = self.rt.kernels, self.rt
        if hasattr(h, "tensor"):
            h = h.tensor()
        rows, qd = h.shape[0], self.qd
        p = self.proj.store(h)                                        # [rows, q | f | v]
        o = rt.empty(rows, self.vd, dtype=torch.float32)
        K_.recurrence(p[:, :qd], p[:, qd:2 * qd], p[:, 2 * qd:], cache.state[self.state_name(site)], batch, o,
                      self.heads, self.heads, self.dim, self.vdim, gate=(self.bias, self.lower))
        normed = rt.empty(rows, self.vd)
        K_.group_rmsnorm_gate(o, self.norm, None, normed, self.heads, self.eps)
        return normed


register_mixer("gated_recurrence", GatedRecurrence)
