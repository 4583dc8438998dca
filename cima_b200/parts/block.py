"""Arrangement of a layer's parts.  ``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x))
(src/models/transformer.rs:1024-1319).  ``parallel``: h = norm(x); x += mixer(conv(h)) + feed_forward(h): one norm
feeds both sublayers, the mixer optionally through a short causal convolution, the feed-forward optionally absent.
``sandwich``: a norm in front of and behind each sublayer, x += m * post(mixer(norm(x))); x += m * post(ffn(norm(x))) with
the spec's ``residual_mult`` m; the feed-forward with its two norms may be absent.  ``postnorm``: the norm stands behind
the sum, x = norm(a x + mixer(x)); x = norm(a x + feed_forward(x)) with the spec's ``stream_mult`` a; the sublayers read the
stream itself and the feed-forward may be absent.  ``hyper``: the model carries several copies of the stream, and a
sublayer reads a weighted sum of them and writes into all of them (``HyperBlock``).  The block builds its parts from the spec through the
registries; it does not know which kinds they are, nor which model it is in.

Interface of the parts it holds:
  norm(x) -> h, norm.lazy(x, ssq)   mixer.forward(h, x, batch, cache, site[, next_norm=])   (adds into x)
  feed_forward.forward(h, x, batch) (adds into x)
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..weights.loader import TensorSpec
from .registry import build_feed_forward, build_mixer, build_norm, register_block


class PreNormBlock:
    def __init__(self, spec, layer: int, rt):
        self.spec, self.layer, self.rt = spec, layer, rt
        self.mixer_norm = build_norm(spec.mixer_norm, rt)
        self.mixer = build_mixer(spec.mixer, layer, rt)
        self.ffn_norm = build_norm(spec.ffn_norm, rt)
        self.feed_forward = build_feed_forward(spec.feed_forward, layer, rt)

    def plan(self) -> Dict[str, TensorSpec]:
        s = self.spec
        p: Dict[str, TensorSpec] = {}
        p.update(self.mixer_norm.plan(f"{s.prefix}{s.names['mixer_norm']}.weight"))
        p.update(self.mixer.plan(s.prefix, s.names))
        p.update(self.ffn_norm.plan(f"{s.prefix}{s.names['ffn_norm']}.weight"))
        p.update(self.feed_forward.plan(s.prefix, s.names))
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.mixer_norm.load(tensors, f"{s.prefix}{s.names['mixer_norm']}.weight")
        self.mixer.load(tensors, s.prefix, s.names)
        self.ffn_norm.load(tensors, f"{s.prefix}{s.names['ffn_norm']}.weight")
        self.feed_forward.load(tensors, s.prefix, s.names)

    def cache_requests(self, site: int) -> List[object]:
        return list(self.mixer.cache_requests(site))

    def state(self) -> Dict[str, torch.Tensor]:
        """The layer's tensors by name as they are kept on the device (the inverse of ``load``).  A part offers
        ``state`` with the arguments of its ``plan``; one that does not cannot be written out."""
        s = self.spec
        out: Dict[str, torch.Tensor] = {}
        for part, args in ((self.mixer_norm, (f"{s.prefix}{s.names['mixer_norm']}.weight",)), (self.mixer, (s.prefix, s.names)),
                           (self.ffn_norm, (f"{s.prefix}{s.names['ffn_norm']}.weight",)), (self.feed_forward, (s.prefix, s.names))):
            if not hasattr(part, "state"):
                raise NotImplementedError(f"{type(part).__name__} of layer {self.layer} offers no state(): its tensors "
                                          f"cannot be given back by name")
            out.update(part.state(*args))
        return out

    def scratch_row(self) -> int:
        """Values of the widest activation row that a step holds inside this layer (sizes the memory forecast)."""
        return max(int(getattr(p, "scratch_row", lambda: 0)()) for p in (self.mixer, self.feed_forward))

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this layer may be recorded as a CUDA graph: every part says so itself
        (``graph_safe = True``: it reads nothing of the batch on the host and keeps its buffers' addresses); a part
        that says nothing is taken as unfit, and the stepper then decodes step by step."""
        return all(getattr(p, "graph_safe", False) for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward))

    def nbytes(self) -> int:
        return self.mixer_norm.nbytes() + self.mixer.nbytes() + self.ffn_norm.nbytes() + self.feed_forward.nbytes()

    def forward(self, x: torch.Tensor, batch, cache, site: int, info=None, next_norm=None):
        """``info`` (a ``RowsInfo`` or None): what the kernel that last wrote x left behind; the same for the
        rows as this block leaves them is returned.  ``next_norm``: the norm that reads x after this block.
        A part that declares ``takes_pending_norm`` gets its norm as a ``NormedInput`` and may fold it into
        its first product; one that declares ``takes_next_norm`` is told which norm follows it and may produce
        it with its last product.  Any other part gets the normalised tensor, and what it returns is
        ignored."""
        info = self._run(self.mixer, self.mixer_norm, info, self.ffn_norm, x, (batch, cache, site))
        return self._run(self.feed_forward, self.ffn_norm, info, next_norm, x, (batch,))

    @staticmethod
    def _run(part, norm, info, next_norm, x, args):
        if info is not None and getattr(info, "norm", None) is norm and info.h is not None:
            h = info.h                                             # the rows came normalised already
        elif getattr(part, "takes_pending_norm", False) and hasattr(norm, "lazy"):
            ssq = getattr(info, "ssq", None) if info is not None else None
            xw = info.xw if (info is not None and getattr(info, "xw_norm", None) is norm) else None
            h = norm.lazy(x, ssq, xw)
        else:
            h = norm(x)
        if getattr(part, "takes_next_norm", False):
            return part.forward(h, x, *args, next_norm=next_norm)
        part.forward(h, x, *args)
        return None


class ParallelBlock:
    """h = norm(x); x += mixer(u) + feed_forward(h), with u = h, or h + conv(h) where the spec has a ``mixer_conv``
    (a ``ShortConv``, which keeps a sequence's newest inputs as state).  Both sublayers add into the float32
    stream, so their sum is formed there."""

    def __init__(self, spec, layer: int, rt):
        from .short_conv import ShortConv
        self.spec, self.layer, self.rt = spec, layer, rt
        self.mixer_norm = build_norm(spec.mixer_norm, rt)
        self.mixer = build_mixer(spec.mixer, layer, rt)
        self.conv = ShortConv(spec.mixer_conv, rt) if spec.mixer_conv is not None else None
        self.feed_forward = build_feed_forward(spec.feed_forward, layer, rt) if spec.feed_forward is not None else None

    def _named(self):
        """(part, the arguments of its plan / load / state) for every part that owns tensors."""
        s = self.spec
        sfx = s.names.get("suffix", ".weight")
        out = [(self.mixer_norm, (f"{s.prefix}{s.names['mixer_norm']}{sfx}",)), (self.mixer, (s.prefix, s.names))]
        if self.conv is not None:
            out.append((self.conv, (f"{s.prefix}{s.names['mixer_conv']}{sfx}",)))
        if self.feed_forward is not None:
            out.append((self.feed_forward, (s.prefix, s.names)))
        return out

    def plan(self) -> Dict[str, TensorSpec]:
        p: Dict[str, TensorSpec] = {}
        for part, args in self._named():
            p.update(part.plan(*args))
        return p

    def load(self, tensors) -> None:
        for part, args in self._named():
            part.load(tensors, *args)

    def state(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for part, args in self._named():
            if not hasattr(part, "state"):
                raise NotImplementedError(f"{type(part).__name__} of layer {self.layer} offers no state(): its tensors "
                                          f"cannot be given back by name")
            out.update(part.state(*args))
        return out

    def cache_requests(self, site: int) -> List[object]:
        reqs = list(self.mixer.cache_requests(site))
        if self.conv is not None:
            reqs += self.conv.cache_requests(site)
        return reqs

    def scratch_row(self) -> int:
        parts = [p for p in (self.mixer, self.feed_forward) if p is not None]
        return max(int(getattr(p, "scratch_row", lambda: 0)()) for p in parts)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p, _ in self._named())

    def nbytes(self) -> int:
        return sum(p.nbytes() for p, _ in self._named())

    def forward(self, x: torch.Tensor, batch, cache, site: int, info=None, next_norm=None):
        if info is not None and getattr(info, "norm", None) is self.mixer_norm and info.h is not None:
            h = info.h                                             # the rows came normalised already
        else:
            h = self.mixer_norm(x)
        if self.conv is None:
            u = h
        elif info is not None and getattr(info, "conv", None) is self.conv and info.u is not None:
            u = info.u                                             # ... and convolved, the state moved on
        else:
            u = self.conv.forward(h, batch, cache, site)
        self.mixer.forward(u, x, batch, cache, site)
        if self.feed_forward is not None:
            self.feed_forward.forward(h, x, batch)
        return None


class SandwichBlock:
    """x += m * post1(mixer(pre1(x))), then x += m * post2(feed_forward(pre2(x))): every sublayer stands between two
    norms, and what it adds to the stream is scaled by ``residual_mult``.  A sublayer adds its output into a zeroed
    float32 buffer (the parts' one interface: they add into the rows they are given) or, where it offers ``produce``,
    hands its output over as float32 rows of its own; the norm behind it reads those;
    where that norm is a Dynamic Tanh, it, the scaled residual sum and the norm in front of the next sublayer are one
    kernel.  Any registered norm serves; one without ``tensors`` runs as separate launches."""

    def __init__(self, spec, layer: int, rt):
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and (spec.ffn_norm is None or spec.ffn_post_norm is None)):
            raise ValueError(f"layer {layer}: a sandwich block needs a norm in front of and behind each of its sublayers")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.mult = float(spec.residual_mult)
        self.mixer_norm = build_norm(spec.mixer_norm, rt)
        self.mixer = build_mixer(spec.mixer, layer, rt)
        self.mixer_post = build_norm(spec.mixer_post_norm, rt)
        self.feed_forward = self.ffn_norm = self.ffn_post = None
        if spec.feed_forward is not None:
            self.ffn_norm = build_norm(spec.ffn_norm, rt)
            self.feed_forward = build_feed_forward(spec.feed_forward, layer, rt)
            self.ffn_post = build_norm(spec.ffn_post_norm, rt)

    def _named(self):
        s = self.spec
        sfx = s.names.get("suffix", ".weight")
        out = [(self.mixer_norm, (f"{s.prefix}{s.names['mixer_norm']}{sfx}",)), (self.mixer, (s.prefix, s.names)),
               (self.mixer_post, (f"{s.prefix}{s.names['mixer_post_norm']}{sfx}",))]
        if self.feed_forward is not None:
            out += [(self.ffn_norm, (f"{s.prefix}{s.names['ffn_norm']}{sfx}",)), (self.feed_forward, (s.prefix, s.names)),
                    (self.ffn_post, (f"{s.prefix}{s.names['ffn_post_norm']}{sfx}",))]
        return out

    def plan(self) -> Dict[str, TensorSpec]:
        p: Dict[str, TensorSpec] = {}
        for part, args in self._named():
            p.update(part.plan(*args))
        return p

    def load(self, tensors) -> None:
        for part, args in self._named():
            part.load(tensors, *args)

    def state(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for part, args in self._named():
            if not hasattr(part, "state"):
                raise NotImplementedError(f"{type(part).__name__} of layer {self.layer} offers no state(): its tensors "
                                          f"cannot be given back by name")
            out.update(part.state(*args))
        return out

    def cache_requests(self, site: int) -> List[object]:
        return list(self.mixer.cache_requests(site))

    def scratch_row(self) -> int:
        parts = [p for p in (self.mixer, self.feed_forward) if p is not None]
        return max(int(getattr(p, "scratch_row", lambda: 0)()) for p in parts) + 2 * self.spec.mixer.hidden

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p, _ in self._named())

    def nbytes(self) -> int:
        return sum(p.nbytes() for p, _ in self._named())

    def _close(self, x, y, post, next_norm):
        """x += m * post(y); returns what the norm that reads x next gives, when it ran in the same kernel."""
        K_ = self.rt.kernels
        if hasattr(post, "tensors") and hasattr(K_, "dyt_add"):
            if next_norm is not None and hasattr(next_norm, "tensors"):
                h = self.rt.empty(*x.shape)
                K_.dyt_add(x, y, post.tensors, self.mult, next_norm.tensors, h)
                return h
            K_.dyt_add(x, y, post.tensors, self.mult)
            return None
        p = post(y)
        if self.mult != 1.0:
            p = p * self.mult
        K_.add_residual(x, p)
        return None

    def forward(self, x: torch.Tensor, batch, cache, site: int, info=None, next_norm=None):
        from .norm import RowsInfo
        if info is not None and getattr(info, "norm", None) is self.mixer_norm and info.h is not None:
            h = info.h
        else:
            h = self.mixer_norm(x)
        if hasattr(self.mixer, "produce"):
            y = self.mixer.produce(h, batch, cache, site)
        else:
            y = torch.zeros_like(x)
            self.mixer.forward(h, y, batch, cache, site)
        if self.feed_forward is None:
            h = self._close(x, y, self.mixer_post, next_norm)
            return RowsInfo(norm=next_norm, h=h) if h is not None else None
        h = self._close(x, y, self.mixer_post, self.ffn_norm)
        if h is None:
            h = self.ffn_norm(x)
        if hasattr(self.feed_forward, "produce"):
            y = self.feed_forward.produce(h, batch)
        else:
            y.zero_()
            self.feed_forward.forward(h, y, batch)
        h = self._close(x, y, self.ffn_post, next_norm)
        return RowsInfo(norm=next_norm, h=h) if h is not None else None


class PostNormBlock:
    """x = norm1(a x + mixer(x)), then x = norm2(a x + feed_forward(x)) with ``stream_mult`` a: no norm in front of a
    sublayer, which reads the stream itself (in the activations' dtype), and one behind the sum.  A layer without
    feed-forward has the first line only.  The sublayers hand their output over as float32 rows (``produce``); the
    scaled stream, the sum, the norm and the rows the next sublayer reads are one kernel (the norm's ``close``).  The
    norm is any registered one that offers ``close(x, y, mult)``."""

    def __init__(self, spec, layer: int, rt):
        self.spec, self.layer, self.rt = spec, layer, rt
        self.mult = float(spec.stream_mult)
        self.mixer = build_mixer(spec.mixer, layer, rt)
        self.mixer_post = build_norm(spec.mixer_norm, rt)
        self.feed_forward = self.ffn_post = None
        if spec.feed_forward is not None:
            if spec.ffn_norm is None:
                raise ValueError(f"layer {layer}: a postnorm block with a feed-forward needs the norm behind it")
            self.feed_forward = build_feed_forward(spec.feed_forward, layer, rt)
            self.ffn_post = build_norm(spec.ffn_norm, rt)
        for part in (self.mixer, self.feed_forward):
            if part is not None and not hasattr(part, "produce"):
                raise ValueError(f"layer {layer}: {type(part).__name__} offers no produce(); a postnorm block needs a sublayer's "
                                 f"output as rows of its own")
        for norm in (self.mixer_post, self.ffn_post):
            if norm is not None and not hasattr(norm, "close"):
                raise ValueError(f"layer {layer}: {type(norm).__name__} offers no close(); a postnorm block needs the sum and "
                                 f"the norm as one step")

    def _named(self):
        s = self.spec
        sfx = s.names.get("suffix", ".weight")
        out = [(self.mixer, (s.prefix, s.names)), (self.mixer_post, (f"{s.prefix}{s.names['mixer_norm']}{sfx}",))]
        if self.feed_forward is not None:
            out += [(self.feed_forward, (s.prefix, s.names)), (self.ffn_post, (f"{s.prefix}{s.names['ffn_norm']}{sfx}",))]
        return out

    def plan(self) -> Dict[str, TensorSpec]:
        p: Dict[str, TensorSpec] = {}
        for part, args in self._named():
            p.update(part.plan(*args))
        return p

    def load(self, tensors) -> None:
        for part, args in self._named():
            part.load(tensors, *args)

    def state(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for part, args in self._named():
            if not hasattr(part, "state"):
                raise NotImplementedError(f"{type(part).__name__} of layer {self.layer} offers no state(): its tensors "
                                          f"cannot be given back by name")
            out.update(part.state(*args))
        return out

    def cache_requests(self, site: int) -> List[object]:
        return list(self.mixer.cache_requests(site))

    def scratch_row(self) -> int:
        parts = [p for p in (self.mixer, self.feed_forward) if p is not None]
        return max(int(getattr(p, "scratch_row", lambda: 0)()) for p in parts) + 2 * self.spec.mixer.hidden

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p, _ in self._named())

    def nbytes(self) -> int:
        return sum(p.nbytes() for p, _ in self._named())

    def forward(self, x: torch.Tensor, batch, cache, site: int, info=None, next_norm=None):
        from .norm import RowsInfo
        if info is not None and getattr(info, "norm", None) is STREAM_ROWS and info.h is not None:
            h = info.h                                             # the stream in the activations' dtype came along
        elif self.rt.full_precision:
            h = x
        else:
            h = self.rt.empty(*x.shape)
            self.rt.kernels.cast_rows(x, h)
        h = self.mixer_post.close(x, self.mixer.produce(h, batch, cache, site), self.mult)
        if self.feed_forward is not None:
            h = self.ffn_post.close(x, self.feed_forward.produce(h, batch), self.mult)
        return RowsInfo(norm=STREAM_ROWS, h=h)


class HyperConnection:
    """What ties one sublayer to the ``streams`` copies X_s of the stream: it reads u = sum_s a[s] X_s and, with its
    output y, X_t <- sum_s C[s, t] X_s + m b[t] y for all t at once.  a (``.in``), b (``.out``) [streams] and C (``.mix``)
    [streams, streams], indexed [from, to], are stored tensors under ``stem``; without a stem they are ones and the unit
    matrix.  They stay on the device as float32: a recorded step reads them there."""

    def __init__(self, streams: int, stem, rt):
        self.S, self.stem, self.rt = int(streams), stem, rt
        self.a = self.b = self.C = None

    def plan(self) -> Dict[str, TensorSpec]:
        if self.stem is None:
            return {}
        S = self.S
        return {f"{self.stem}.in": TensorSpec((S,), init="mean", std=0.1), f"{self.stem}.out": TensorSpec((S,), init="ones_normal", std=0.1),
                f"{self.stem}.mix": TensorSpec((S, S), init="eye_normal", std=0.1)}

    def load(self, tensors) -> None:
        rt, S = self.rt, self.S
        if self.stem is None:
            self.a = rt.vector(torch.ones(S))
            self.b = rt.vector(torch.ones(S))
            self.C = rt.vector(torch.eye(S))
            return
        self.a, self.b = rt.vector(tensors[f"{self.stem}.in"]), rt.vector(tensors[f"{self.stem}.out"])
        self.C = rt.vector(tensors[f"{self.stem}.mix"])

    def state(self) -> Dict[str, torch.Tensor]:
        if self.stem is None:
            return {}
        return {f"{self.stem}.in": self.a, f"{self.stem}.out": self.b, f"{self.stem}.mix": self.C}

    def nbytes(self) -> int:
        return (2 * self.S + self.S * self.S) * 4


class HyperBlock:
    """Hyper-connections: ``streams`` copies X_1 .. X_S of the stream, [rows, S, hidden] float32, instead of one.  For
    the mixer and then for the feed-forward (which may be absent), each with a ``HyperConnection`` (a, b, C) and a norm:
        u = sum_s a[s] X_s;   y = sublayer(norm(u));   X_t <- sum_s C[s, t] X_s + m b[t] y    (all t from the old X)
    with the spec's ``residual_mult`` m.  One stream with a = b = C = 1 is the pre-norm layer x += m sublayer(norm(x)).
    The sublayers hand their output over as float32 rows (``produce``).  One kernel (``hyper_connect``) writes a
    sublayer's output into the streams and forms the next reader's sum and norm from the new rows, so a layer is
    two such launches beside its sublayers'; the first reader of the first layer takes the streams from the embedding's
    rows in the same way."""

    def __init__(self, spec, layer: int, rt):
        if spec.streams < 1 or spec.streams > 8:
            raise ValueError(f"layer {layer}: {spec.streams} streams (1 to 8 are taken)")
        self.spec, self.layer, self.rt = spec, layer, rt
        self.S, self.mult = int(spec.streams), float(spec.residual_mult)
        self.mixer_norm = build_norm(spec.mixer_norm, rt)
        self.mixer = build_mixer(spec.mixer, layer, rt)
        stem = lambda key: f"{spec.prefix}{spec.names[key]}" if key in spec.names else None
        self.mixer_hc = HyperConnection(self.S, stem("mixer_hc"), rt)
        self.feed_forward = self.ffn_norm = self.ffn_hc = None
        if spec.feed_forward is not None:
            if spec.ffn_norm is None:
                raise ValueError(f"layer {layer}: a feed-forward needs the norm in front of it")
            self.ffn_norm = build_norm(spec.ffn_norm, rt)
            self.feed_forward = build_feed_forward(spec.feed_forward, layer, rt)
            self.ffn_hc = HyperConnection(self.S, stem("ffn_hc"), rt)
        for part in (self.mixer, self.feed_forward):
            if part is not None and not hasattr(part, "produce"):
                raise ValueError(f"layer {layer}: {type(part).__name__} offers no produce(); a hyper block needs a sublayer's "
                                 f"output as rows of its own")
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and (getattr(norm, "spec", None) is None or norm.spec.kind != "rmsnorm"):
                raise ValueError(f"layer {layer}: a hyper block's norms are of kind 'rmsnorm' (the kernel that sums the streams applies them)")

    def _named(self):
        s = self.spec
        sfx = s.names.get("suffix", ".weight")
        out = [(self.mixer_norm, (f"{s.prefix}{s.names['mixer_norm']}{sfx}",)), (self.mixer, (s.prefix, s.names)), (self.mixer_hc, ())]
        if self.feed_forward is not None:
            out += [(self.ffn_norm, (f"{s.prefix}{s.names['ffn_norm']}{sfx}",)), (self.feed_forward, (s.prefix, s.names)), (self.ffn_hc, ())]
        return out

    def plan(self) -> Dict[str, TensorSpec]:
        p: Dict[str, TensorSpec] = {}
        for part, args in self._named():
            p.update(part.plan(*args))
        return p

    def load(self, tensors) -> None:
        for part, args in self._named():
            part.load(tensors, *args)

    def state(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for part, args in self._named():
            if not hasattr(part, "state"):
                raise NotImplementedError(f"{type(part).__name__} of layer {self.layer} offers no state(): its tensors "
                                          f"cannot be given back by name")
            out.update(part.state(*args))
        return out

    def cache_requests(self, site: int) -> List[object]:
        return list(self.mixer.cache_requests(site))

    def scratch_row(self) -> int:
        parts = [p for p in (self.mixer, self.feed_forward) if p is not None]
        return max(int(getattr(p, "scratch_row", lambda: 0)()) for p in parts) + 2 * self.spec.mixer.hidden

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p, _ in self._named() if not isinstance(p, HyperConnection))

    def nbytes(self) -> int:
        return sum(p.nbytes() for p, _ in self._named())

    @property
    def reader(self):
        """(a, norm) of the block's first sublayer: what the kernel that last writes the streams needs to form its input."""
        return self.mixer_hc.a, self.mixer_norm

    def _connect(self, xs, y, hc, reader):
        """Write y through ``hc`` (None: nothing to write) and read for ``reader`` = (a, norm) (None: nothing to read);
        returns the reader's normed rows in the activations' dtype."""
        h = None
        if reader is not None:
            h = self.rt.empty(xs.shape[0], xs.shape[2])
        self.rt.kernels.hyper_connect(xs, y, hc.C if hc is not None else None, hc.b if hc is not None else None, self.mult,
                                      reader[0] if reader is not None else None, reader[1].weight if reader is not None else None,
                                      reader[1].spec.eps if reader is not None else 0.0, h)
        return h

    def forward(self, xs: torch.Tensor, batch, cache, site: int, info=None, next_reader=None):
        """``xs``: the streams [rows, S, hidden] float32, updated in place.  ``info``: a ``RowsInfo`` whose ``h`` holds this
        block's first input where the kernel before formed it.  ``next_reader``: (a, norm) of whatever reads the streams
        next (the next block's ``reader``, or ones and the final norm); its rows come back in a ``RowsInfo``."""
        from .norm import RowsInfo
        if xs.dim() != 3 or xs.shape[1] != self.S:
            raise ValueError(f"layer {self.layer}: the streams are {tuple(xs.shape)}, expected [rows, {self.S}, hidden]")
        if info is not None and getattr(info, "norm", None) is self.mixer_norm and info.h is not None:
            h = info.h
        else:
            h = self._connect(xs, None, None, self.reader)
        y = self.mixer.produce(h, batch, cache, site)
        if self.feed_forward is None:
            h = self._connect(xs, y, self.mixer_hc, next_reader)
        else:
            h = self._connect(xs, y, self.mixer_hc, (self.ffn_hc.a, self.ffn_norm))
            y = self.feed_forward.produce(h, batch)
            h = self._connect(xs, y, self.ffn_hc, next_reader)
        return RowsInfo(norm=next_reader[1], h=h) if next_reader is not None else None


STREAM_ROWS = object()      # a RowsInfo whose ``norm`` is this holds the stream itself in the activations' dtype


register_block("prenorm", PreNormBlock)
register_block("postnorm", PostNormBlock)
register_block("sandwich", SandwichBlock)
register_block("parallel", ParallelBlock)
register_block("hyper", HyperBlock)
