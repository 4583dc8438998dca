"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, computed in float32 from the float32 residual stream
(src/kernels.cu:37-50).  ``size`` and ``eps`` come from the spec; with ``params["offset"]`` c the stored tensor w
multiplies as c + w (a weight kept around zero: c = 1), formed once at load in float32."""
from __future__ import annotations

from typing import Dict

import torch

from ..weights.loader import TensorSpec
from .registry import register_norm


class RowsInfo:
    """What the kernel that last wrote the residual rows left behind, handed from part to part:
    ``ssq`` - partial sums of squares of the rows [rows, parts] (a skinny product can fold the next norm in),
    with ``xw`` = bf16(rows * weight of ``xw_norm``) when the writer knew which norm follows;
    ``norm`` / ``h`` - the rows already normalised with that norm (the residual add and the norm ran as one)."""

    def __init__(self, ssq=None, norm=None, h=None, xw=None, xw_norm=None):
        self.ssq, self.norm, self.h = ssq, norm, h
        self.xw, self.xw_norm = xw, xw_norm       # rows times the weight of ``xw_norm``, bf16 (goes with ssq)
        self.conv, self.u = None, None            # a short convolution that has already read ``h``, and its output


class NormedInput:
    """RMSNorm(x) not yet computed.  A product that can fold the norm in (few rows, bf16) takes ``xw``
    (bf16(x * weight)) and ``ssq`` (partial sums of squares of x's rows), both left by the kernel that
    wrote the rows; everything else calls ``tensor()`` and gets the normalised activations."""

    def __init__(self, norm: "RMSNorm", x: torch.Tensor, ssq, xw=None):
        self.norm, self.x, self.ssq, self.xw = norm, x, ssq, xw
        self._h = None

    @property
    def shape(self):
        return self.x.shape

    def tensor(self) -> torch.Tensor:
        if self._h is None:
            self._h = self.norm(self.x)
        return self._h


class RMSNorm:
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.offset = float(spec.params.get("offset", 0.0)) if spec.params else 0.0
        self.weight = None                       # offset + the stored tensor: what the kernels multiply by

    def plan(self, name: str) -> Dict[str, TensorSpec]:
        if self.offset:
            return {name: TensorSpec((self.spec.size,), std=0.1)}
        return {name: TensorSpec((self.spec.size,), init="ones_normal")}

    def load(self, tensors: Dict[str, torch.Tensor], name: str) -> None:
        self.weight = self.rt.vector(tensors[name])
        if self.offset:
            self.weight = self.weight + self.offset

    def nbytes(self) -> int:
        return self.weight.numel() * 4

    def state(self, name: str) -> Dict[str, torch.Tensor]:
        return {name: self.weight - self.offset if self.offset else self.weight}

    graph_safe = True

    def lazy(self, x: torch.Tensor, ssq=None, xw=None) -> NormedInput:
        return NormedInput(self, x, ssq, xw)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty(*x.shape)
        self.rt.kernels.rmsnorm(x, self.weight, self.spec.eps, out)
        return out


class DynamicTanh:
    """y = tanh(alpha * x) * w + b: a norm that computes no mean and no variance.  ``alpha`` is one stored scalar (it
    stays on the device: a recorded step reads it there), w and b vectors; tensors ``name``, ``name.b``, ``name.alpha``.
    The spec's eps is not used.  Everything float32, one rounding at the store."""

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.weight = self.bias = self.alpha = None

    def plan(self, name: str) -> Dict[str, TensorSpec]:
        return {name: TensorSpec((self.spec.size,), init="ones_normal"), name + ".b": TensorSpec((self.spec.size,), std=0.05),
                name + ".alpha": TensorSpec((), init="ones_normal")}

    def load(self, tensors, name: str) -> None:
        self.weight = self.rt.vector(tensors[name])
        self.bias = self.rt.vector(tensors[name + ".b"])
        self.alpha = self.rt.vector(tensors[name + ".alpha"]).reshape(1)

    def nbytes(self) -> int:
        return (self.weight.numel() + self.bias.numel() + 1) * 4

    def state(self, name: str) -> Dict[str, torch.Tensor]:
        return {name: self.weight, name + ".b": self.bias, name + ".alpha": self.alpha.reshape(())}

    graph_safe = True

    @property
    def tensors(self):
        return (self.alpha, self.weight, self.bias)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty(*x.shape)
        self.rt.kernels.dyt(x, self.alpha, self.weight, self.bias, out)
        return out


class GroupRMSNorm:
    """RMS norm in groups: a row is split into ``params["groups"]`` equal consecutive parts, each divided by its own
    sqrt(mean(part^2) + eps), and the whole multiplied by a weight of the row's size.  Float32, one rounding at the store."""

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.groups = int(spec.params.get("groups", 1))
        if self.groups <= 0 or spec.size % self.groups:
            raise ValueError(f"group_rmsnorm: {self.groups} groups do not divide the size {spec.size}")
        self.weight = None

    def plan(self, name: str) -> Dict[str, TensorSpec]:
        return {name: TensorSpec((self.spec.size,), init="ones_normal")}

    def load(self, tensors, name: str) -> None:
        self.weight = self.rt.vector(tensors[name])

    def nbytes(self) -> int:
        return self.weight.numel() * 4

    def state(self, name: str) -> Dict[str, torch.Tensor]:
        return {name: self.weight}

    graph_safe = True

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty(*x.shape)
        self.rt.kernels.group_rmsnorm_gate(x, self.weight, None, out, self.groups, self.spec.eps)
        return out

    def close(self, x: torch.Tensor, y: torch.Tensor, mult: float) -> torch.Tensor:
        """x <- norm(mult * x + y) in place (the stream, float32); returns the new rows in the activations' dtype (x
        itself where that is float32)."""
        h = None if self.rt.full_precision else self.rt.empty(*x.shape)
        self.rt.kernels.scale_add_group_rmsnorm(x, y, mult, self.weight, self.groups, self.spec.eps, h)
        return x if h is None else h


register_norm("rmsnorm", RMSNorm)
register_norm("group_rmsnorm", GroupRMSNorm)
register_norm("dyt", DynamicTanh)
