"""A routed feed-forward (kind ``moe``): ``experts`` small gated feed-forward layers of which every token uses ``top``.

    s = sigmoid(W_router h)                                   router logits and scores in float32
    the experts form ``groups`` equal groups of neighbours; a group's score is the sum of its two largest s; only
    experts of the best ``keep`` groups can be chosen; of those, the ``top`` with the largest s are
    weights  w_e = s_e / (sum of the chosen s + 1e-20) * scale
    y = sum_e  w_e * W_down[e] (act(W_gate[e] h) * (W_up[e] h))

Options (``params``), each off by default:
  ``scoring`` "softmax": s = softmax(W_router h) over all experts instead of the sigmoid;
  ``correction``: a stored vector (tensor "correction", [experts]) that is added to s where experts are chosen and left
      out of the weights;
  activation "swish_clamped" with ``limit`` L: an expert's middle is min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1);
  ``shared`` {"ff", "activation", "limit"}: one more expert of that form for every token (tensors "shared.gate",
      "shared.up", "shared.down"), added unweighted, or with ``shared_gate`` times sigmoid(w_sg . h) (tensor "shared.sg",
      [1, hidden]; its row stands under the router's in one matrix, so the routing product gives its logit too).

The experts' matrices are kept stacked, [E, 2 ff, H] (an expert's gate rows, then its up rows) and [E, H, ff]; a step
sorts its (row, choice) pairs by expert on the device and runs two grouped products over tiles of one expert's pairs,
so nothing of the routing is read on the host.  Tensors: ``router`` and, per expert j, ``e<j>.gate``, ``e<j>.up``,
``e<j>.down`` under the feed-forward's stem (names["experts"]).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..weights.loader import TensorSpec
from ..kernels import GATED_ONLY
from .linear import Linear
from .registry import register_feed_forward


class RoutedExperts:
    def __init__(self, spec, layer: int, rt):
        from ..kernels import ACTIVATIONS
        p = spec.params
        self.E, self.top = int(p["experts"]), int(p["top"])
        self.groups, self.keep, self.scale = int(p.get("groups", 1)), int(p.get("keep", p.get("groups", 1))), float(p.get("scale", 1.0))
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"moe: activation '{spec.activation}' is not one of {sorted(ACTIVATIONS)}")
        self.limit = float(p.get("limit", 0.0))
        self.softmax = p.get("scoring", "sigmoid") == "softmax"
        if p.get("scoring", "sigmoid") not in ("sigmoid", "softmax"):
            raise ValueError(f"moe: scoring '{p.get('scoring')}' is neither 'sigmoid' nor 'softmax'")
        self.has_correction = bool(p.get("correction", False))
        self.shared_spec = p.get("shared")
        self.shared_gate = bool(p.get("shared_gate", False)) and self.shared_spec is not None
        if self.E <= 0 or self.groups <= 0 or self.E % self.groups or not (0 < self.keep <= self.groups):
            raise ValueError(f"moe: {self.E} experts in {self.groups} groups of which {self.keep} stay are not a valid routing")
        if not (0 < self.top <= self.keep * (self.E // self.groups)):
            raise ValueError(f"moe: {self.top} choices among the {self.keep * (self.E // self.groups)} experts that stay")
        if self.E > 1024 or self.groups > 64:
            raise ValueError("moe: at most 1024 experts in at most 64 groups")
        self.act = ACTIVATIONS[spec.activation]
        self.spec, self.layer, self.rt = spec, layer, rt
        self.router = self.gate_up = self.down = self.correction = self.shared_up = self.shared_down = None

    def _n(self, prefix, names, tail):
        return f"{prefix}{names['experts']}{tail}{names.get('suffix', '.weight')}"

    def plan(self, prefix: str, names: Dict[str, str]) -> Dict[str, TensorSpec]:
        s = self.spec
        p = {self._n(prefix, names, "router"): TensorSpec((self.E, s.hidden), std=0.1)}
        for j in range(self.E):
            p[self._n(prefix, names, f"e{j}.gate")] = TensorSpec((s.intermediate, s.hidden))
            p[self._n(prefix, names, f"e{j}.up")] = TensorSpec((s.intermediate, s.hidden))
            p[self._n(prefix, names, f"e{j}.down")] = TensorSpec((s.hidden, s.intermediate))
        if self.has_correction:
            p[self._n(prefix, names, "correction")] = TensorSpec((self.E,), std=0.02)
        if self.shared_spec is not None:
            ffs = int(self.shared_spec["ff"])
            p[self._n(prefix, names, "shared.gate")] = TensorSpec((ffs, s.hidden))
            p[self._n(prefix, names, "shared.up")] = TensorSpec((ffs, s.hidden))
            p[self._n(prefix, names, "shared.down")] = TensorSpec((s.hidden, ffs))
            if self.shared_gate:
                p[self._n(prefix, names, "shared.sg")] = TensorSpec((1, s.hidden), std=0.1)
        return p

    def load(self, tensors, prefix: str, names: Dict[str, str]) -> None:
        s, rt = self.spec, self.rt
        rows = [tensors[self._n(prefix, names, "router")]]
        if self.shared_gate:
            # the gate's row under the router's, then zero rows up to a multiple of 8 outputs (a row of the scores keeps its
            # 16-byte alignment, and the library's product of many rows its fast kernels)
            rows.append(tensors[self._n(prefix, names, "shared.sg")])
            pad = -(self.E + 1) % 8
            if pad:
                rows.append(torch.zeros((pad, s.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.router = Linear(rows, None, rt)
        del rows
        if self.has_correction:
            self.correction = rt.vector(tensors[self._n(prefix, names, "correction")])
        if self.shared_spec is not None:
            from .linear import GatedLinearPair
            sh = self.shared_spec
            self.shared_up = GatedLinearPair(tensors[self._n(prefix, names, "shared.gate")], tensors[self._n(prefix, names, "shared.up")],
                                             rt, sh.get("activation", s.activation), limit=float(sh.get("limit", 0.0)))
            self.shared_down = Linear(tensors[self._n(prefix, names, "shared.down")], None, rt)
        ff, H = s.intermediate, s.hidden
        first = rt.matrix(tensors[self._n(prefix, names, "e0.gate")])
        self.gate_up = torch.empty((self.E, 2 * ff, H), dtype=first.dtype, device=rt.device)
        self.down = torch.empty((self.E, H, ff), dtype=first.dtype, device=rt.device)
        for j in range(self.E):
            self.gate_up[j, :ff].copy_(first if j == 0 else tensors[self._n(prefix, names, f"e{j}.gate")])
            self.gate_up[j, ff:].copy_(tensors[self._n(prefix, names, f"e{j}.up")])
            self.down[j].copy_(tensors[self._n(prefix, names, f"e{j}.down")])

    def state(self, prefix: str, names: Dict[str, str]) -> Dict[str, torch.Tensor]:
        ff = self.spec.intermediate
        out = {self._n(prefix, names, "router"): self.router.weight[:self.E]}
        if self.has_correction:
            out[self._n(prefix, names, "correction")] = self.correction
        if self.shared_spec is not None:
            w, I = self.shared_up.lin.weight, self.shared_up.I
            out[self._n(prefix, names, "shared.gate")], out[self._n(prefix, names, "shared.up")] = w[:I], w[I:]
            out[self._n(prefix, names, "shared.down")] = self.shared_down.weight
            if self.shared_gate:
                out[self._n(prefix, names, "shared.sg")] = self.router.weight[self.E:self.E + 1]
        for j in range(self.E):
            out[self._n(prefix, names, f"e{j}.gate")] = self.gate_up[j, :ff]
            out[self._n(prefix, names, f"e{j}.up")] = self.gate_up[j, ff:]
            out[self._n(prefix, names, f"e{j}.down")] = self.down[j]
        return out

    def nbytes(self) -> int:
        """Bytes a decode step reads: the router and, of the experts, the ``top`` that one token uses."""
        per = (self.gate_up[0].numel() + self.down[0].numel()) * self.gate_up.element_size()
        shared = self.shared_up.nbytes() + self.shared_down.nbytes() if self.shared_spec is not None else 0
        return self.router.nbytes() + self.top * per + shared

    def extra_bytes(self, rows: int) -> int:
        """What a step of ``rows`` tokens reads beyond ``nbytes()`` when every token chooses other experts."""
        per = (self.gate_up[0].numel() + self.down[0].numel()) * self.gate_up.element_size()
        return (min(self.E, rows * self.top) - self.top) * per

    def scratch_row(self) -> int:
        shared = 2 * int(self.shared_spec["ff"]) if self.shared_spec is not None else 0
        return self.top * (2 * self.spec.intermediate + 2 * self.spec.hidden) + self.E + 1 + shared

    graph_safe = True

    def forward(self, h, x: torch.Tensor, batch, next_norm=None):
        self._run(h, x, False)
        return None

    def produce(self, h, batch) -> torch.Tensor:
        """The feed-forward's output as float32 rows of its own (what ``forward`` adds into x)."""
        y = self.rt.empty(h.shape[0], self.spec.hidden, dtype=torch.float32)
        self._run(h, y, True)
        return y

    def _run(self, h, x: torch.Tensor, assign: bool) -> None:
        K_, rt = self.rt.kernels, self.rt
        if hasattr(h, "tensor"):
            h = h.tensor()
        rows = h.shape[0]
        scores = self.router.logits(h)                                # float32 [rows, E (+ 1: the shared expert's gate)]
        route = {}
        if self.softmax or self.correction is not None:
            route = {"softmax": self.softmax, "correction": self.correction}
        if self.limit or self.act >= GATED_ONLY:
            expert = {"limit": self.limit}
        else:
            expert = {}
        idx = rt.empty(rows, self.top, dtype=torch.int32)
        wgt = rt.empty(rows, self.top, dtype=torch.float32)
        # (a decode step's few rows: the routing launch also orders the pairs by expert)
        small = rows <= getattr(K_, "ROUTE_SORT_ROWS", 0) and rows * self.top < getattr(K_, "MOE_TC_PAIRS", 0)
        if self.shared_spec is not None:
            # the shared expert's rows (float32) join the chosen experts' weighted sum in its launch, each row times the
            # sigmoid of its gate logit (the last column of the routing product)
            expert["shared"] = (self.shared_down.logits(self.shared_up.activated(h)), scores if self.shared_gate else None, self.E)
        if small:
            ordered = K_.moe_route(scores, self.top, self.groups, self.keep, self.scale, idx, wgt, order=True, experts=self.E, **route)
            K_.moe_experts(h, self.gate_up, self.down, idx, wgt, x, self.act, assign=assign, ordered=ordered, **expert)
        else:
            K_.moe_route(scores, self.top, self.groups, self.keep, self.scale, idx, wgt, experts=self.E, **route)
            K_.moe_experts(h, self.gate_up, self.down, idx, wgt, x, self.act, assign=assign, **expert)


register_feed_forward("moe", RoutedExperts)
