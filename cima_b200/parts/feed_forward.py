"""Gated feed-forward: x += (act(h Wg^T) * (h Wu^T)) Wd^T in float32, act by the spec's ``activation``: SiLU
g / (1 + exp(-g)) as the reference has it (src/kernels.cu:81-84; src/models/transformer.rs:1219-1229 and
:1273-1291), or one of the other entries of ``kernels.ACTIVATIONS`` (tanh or erf GELU, ReLU), which every kernel
that applies the activation takes as a parameter.  ``swish_clamped`` is a form of the whole middle,
min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u, -L, L) + 1), with the limit L = ``params["limit"]``.  Rows are independent, so a long step is cut into row chunks
that bound the [rows, 2I] scratch."""
from __future__ import annotations

from typing import Dict

import torch

from ..weights.loader import TensorSpec
from .linear import GatedLinearPair, Linear
from .registry import register_feed_forward

_SCRATCH_ELEMS = 1 << 29          # elements of the [rows, 2I] gate|up scratch per chunk


class GatedMLP:
    def __init__(self, spec, layer: int, rt):
        from ..kernels import ACTIVATIONS
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"gated_mlp: activation '{spec.activation}' is not one of {sorted(ACTIVATIONS)}")
        if spec.bias:
            raise ValueError("gated_mlp: biases are not implemented")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.gate_up = None
        self.down = None

    @staticmethod
    def _names(prefix: str, names: Dict[str, str]):
        sfx = names.get("suffix", ".weight")
        return tuple(f"{prefix}{names[k]}{sfx}" for k in ("gate", "up", "down"))

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        s = self.spec
        gate, up, down = self._names(prefix, names)
        return {gate: TensorSpec((s.intermediate, s.hidden)), up: TensorSpec((s.intermediate, s.hidden)),
                down: TensorSpec((s.hidden, s.intermediate))}

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str, names: Dict[str, str]) -> None:
        gate, up, down = self._names(prefix, names)
        self.gate_up = GatedLinearPair(tensors[gate], tensors[up], self.rt, self.spec.activation,
                                       limit=float(self.spec.params.get("limit", 0.0)))
        self.down = Linear(tensors[down], None, self.rt)

    def nbytes(self) -> int:
        return self.gate_up.nbytes() + self.down.nbytes()

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        w, I = self.gate_up.lin.weight, self.spec.intermediate
        gate, up, down = self._names(prefix, names)
        return {gate: w[:I], up: w[I:], down: self.down.weight}

    def scratch_row(self) -> int:
        return 2 * self.spec.intermediate

    graph_safe = True

    takes_pending_norm = True
    takes_next_norm = True

    def forward(self, h, x: torch.Tensor, batch, next_norm=None):
        rows = h.shape[0]
        chunk = max(64, _SCRATCH_ELEMS // (2 * self.spec.intermediate))
        chunk -= chunk % 256 if chunk >= 256 else 0          # whole row tiles for the tensor-core product
        if rows <= chunk:
            return self.down.accumulate(self.gate_up.activated(h), x, next_norm)
        if hasattr(h, "tensor"):
            h = h.tensor()
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            self.down.accumulate(self.gate_up.activated(h[r0:r1]), x[r0:r1])
        return None

    def produce(self, h, batch) -> torch.Tensor:
        """The feed-forward's output as float32 rows of its own (what ``forward`` adds into x)."""
        return self.down.logits(self.gate_up.activated(h))


class PlainMLP:
    """An ungated feed-forward (kind ``mlp``): y = W_down act(W_up h), act by the spec's ``activation``: one of the gate
    activations of ``kernels.ACTIVATIONS`` or ``relu2`` (the square of ReLU).  The activation runs on the stored
    projection (the activations' dtype), in float32 inside the kernel."""

    def __init__(self, spec, layer: int, rt):
        from ..kernels import UNGATED_ACTIVATIONS
        if spec.activation not in UNGATED_ACTIVATIONS:
            raise ValueError(f"mlp: activation '{spec.activation}' is not one of {sorted(UNGATED_ACTIVATIONS)}")
        if spec.bias:
            raise ValueError("mlp: biases are not implemented")
        self.act = UNGATED_ACTIVATIONS[spec.activation]
        self.spec, self.layer, self.rt = spec, layer, rt
        self.up = self.down = None

    @staticmethod
    def _names(prefix: str, names: Dict[str, str]):
        sfx = names.get("suffix", ".weight")
        return tuple(f"{prefix}{names[k]}{sfx}" for k in ("up", "down"))

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        s = self.spec
        up, down = self._names(prefix, names)
        return {up: TensorSpec((s.intermediate, s.hidden)), down: TensorSpec((s.hidden, s.intermediate))}

    def load(self, tensors, prefix: str, names: Dict[str, str]) -> None:
        up, down = self._names(prefix, names)
        self.up = Linear(tensors[up], None, self.rt)
        self.down = Linear(tensors[down], None, self.rt)

    def nbytes(self) -> int:
        return self.up.nbytes() + self.down.nbytes()

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        up, down = self._names(prefix, names)
        return {up: self.up.weight, down: self.down.weight}

    def scratch_row(self) -> int:
        return self.spec.intermediate

    graph_safe = True

    def _middle(self, h) -> torch.Tensor:
        if hasattr(h, "tensor"):
            h = h.tensor()
        z = self.up.store(h)
        self.rt.kernels.activate(z, self.act)
        return z

    def forward(self, h, x: torch.Tensor, batch, next_norm=None):
        self.down.accumulate(self._middle(h), x)
        return None

    def produce(self, h, batch) -> torch.Tensor:
        """The feed-forward's output as float32 rows of its own (what ``forward`` adds into x)."""
        return self.down.logits(self._middle(h))


register_feed_forward("gated_mlp", GatedMLP)
register_feed_forward("mlp", PlainMLP)
