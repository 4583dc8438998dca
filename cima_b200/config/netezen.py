"""Typed configuration of the Netezen decoder, read from its own config.json keys.

A Netezen model is a stack of *pre-norm* layers whose sublayers' outputs are scaled by one factor m (``residual_mult``)
before they join the stream: x += m mixer(N(x)); x += m ff(N(x)), N an RMS norm whose stored weight w multiplies as
1 + w.  With ``streams`` S the model carries S copies of the stream (hyper-connections): a sublayer reads a weighted sum
of the copies and writes into every copy, through stored vectors and one S x S matrix a sublayer (``hc1`` the mixer's,
``hc2`` the feed-forward's); behind the last layer the copies are summed.  The head is the embedding table.

A layer's mixer is one of two kinds.  ``attention``: grouped-query softmax attention, rotary positions on the first
``rot.dims`` values of a head with neighbouring values paired, frequencies optionally rescaled by index
(``rot.scaling`` {factor, original, fast, slow}), a sliding window that keeps a sequence's first ``mask.keep_first``
positions visible.  ``latent_attention``: queries through a latent of ``q_rank`` values; keys and values projected from a
cached latent of ``kv_rank`` values beside one rotated key part of ``rot_dim`` values that all heads share; a sliding
window; a stored number a head in the softmax's denominator.  The feed-forward is ``dense`` (W_down relu(W_up h)^2),
``moe`` (softmax router, a stored correction where experts are chosen, clamped gated experts, optionally a shared expert
behind a sigmoid gate), or absent (``mlp: null``).

config.json gives ``vocab``, ``width``, ``norm`` {eps}, ``residual_mult``, ``streams`` and per entry of ``layers``:
``type``, ``mixer`` and ``mlp``:
  attention         mixer {heads, kv_heads, dim, vdim, scale, rot {dims, base[, scaling]}, mask {size[, keep_first]}}
  latent_attention  mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {dims, base}, mask {size}}
  mlp               {kind "dense", ff}  |  {kind "moe", expert {ff, limit}, router {experts, top}[, shared {ff, limit}]}
Tensor names: ``embed``, ``final.norm`` and under ``l<i>.``: ``norm1``, ``norm2``, ``hc1.{in,out,mix}``, ``hc2.*``,
``mix.{q,k,v,o}`` or ``mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,o}``, ``mlp.{up,down}`` or ``mlp.{router,correction,
e<j>.{gate,up,down},shared.{gate,up,down,sg}}``.  Whether a model has hyper-connection tensors, a router correction or a
sink is read off the stored tensors' names where a folder is given (``from_dict(cfg, shapes)``); a configuration
alone has them where ``streams`` is given, and always a correction and a sink.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .qwen2 import ConfigError
from .specs import BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
from .vunovik import _int, _num

MAX_POSITION = 1 << 20       # rotary positions have no end of their own


@dataclass(frozen=True)
class Rotation:
    dims: int                                   # 0 = nothing rotates
    base: float = 10000.0
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, original, fast, slow


@dataclass(frozen=True)
class GroupedMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation
    window: int                                 # 0 = every earlier position
    keep_first: int


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: Rotation
    window: int
    sink: bool


@dataclass(frozen=True)
class Experts:
    experts: int
    top: int
    ff: int
    limit: float
    correction: bool
    shared_ff: int                              # 0 = no shared expert
    shared_limit: float


@dataclass(frozen=True)
class NetezenLayer:
    kind: str                                   # "attention" | "latent_attention"
    grouped: Optional[GroupedMixer] = None
    latent: Optional[LatentMixer] = None
    dense_ff: int = 0                           # > 0: the dense feed-forward's middle
    moe: Optional[Experts] = None


def _rotation(rot: Any, where: str, limit: int) -> Rotation:
    if rot is None:
        return Rotation(dims=0)
    dims = _int(rot, "dims", where, least=0)
    if dims == 0:
        return Rotation(dims=0)
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}dims ({dims}) must be even and at most {limit}")
    base = _num(rot, "base", where)
    if base <= 1:
        raise ConfigError(f"config.json: {where}base ({base}) must be above 1")
    sc = rot.get("scaling")
    scaling = None
    if sc is not None:
        scaling = tuple(_num(sc, k, where + "scaling.") for k in ("factor", "original", "fast", "slow"))
        if min(scaling) <= 0:
            raise ConfigError(f"config.json: {where}scaling's factor, original, fast and slow must be positive")
    return Rotation(dims=dims, base=base, scaling=scaling)


def _window(m: Dict[str, Any], where: str):
    mask = m.get("mask")
    size = _int(mask, "size", where + "mask.", least=0) if mask is not None and mask.get("size") is not None else 0
    keep = _int(mask, "keep_first", where + "mask.", least=0) if mask is not None and mask.get("keep_first") is not None else 0
    return size, keep if size else 0


def _has(shapes, name: str, default: bool) -> bool:
    return default if shapes is None else name in shapes


@dataclass(frozen=True)
class NetezenConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    streams: int                                # copies of the stream
    learned_streams: bool                       # whether hc1.* / hc2.* are stored
    layers: Tuple[NetezenLayer, ...]

    ARCHITECTURE = "Netezen"

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any], shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "NetezenConfig":
        if cfg.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError(f"config.json: architecture {cfg.get('architecture')!r} is not '{cls.ARCHITECTURE}'")
        vocab, width = _int(cfg, "vocab", ""), _int(cfg, "width", "")
        eps = _num(cfg.get("norm"), "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps ({eps}) must be positive")
        streams = _int(cfg, "streams", "") if cfg.get("streams") is not None else 1
        if streams > 8:
            raise ConfigError(f"config.json: streams ({streams}) must be at most 8")
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]."
            kind = L.get("type") if isinstance(L, dict) else None
            m = L.get("mixer") if isinstance(L, dict) else None
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}mixer is missing")
            dense_ff, moe = 0, None
            f = L.get("mlp")
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"config.json: {where}mlp.kind {f.get('kind') if isinstance(f, dict) else f!r} is neither 'dense' nor 'moe'")
                if f["kind"] == "dense":
                    dense_ff = _int(f, "ff", where + "mlp.")
                else:
                    r, e, sh = f.get("router"), f.get("expert"), f.get("shared")
                    moe = Experts(experts=_int(r, "experts", where + "mlp.router."), top=_int(r, "top", where + "mlp.router."),
                                  ff=_int(e, "ff", where + "mlp.expert."), limit=_num(e, "limit", where + "mlp.expert."),
                                  correction=_has(shapes, f"l{i}.mlp.correction", True),
                                  shared_ff=_int(sh, "ff", where + "mlp.shared.") if sh is not None else 0,
                                  shared_limit=_num(sh, "limit", where + "mlp.shared.") if sh is not None else 0.0)
                    if moe.top > moe.experts:
                        raise ConfigError(f"config.json: {where}mlp.router.top ({moe.top}) exceeds its experts ({moe.experts})")
                    if moe.limit <= 0 or (moe.shared_ff and moe.shared_limit <= 0):
                        raise ConfigError(f"config.json: {where}mlp: the experts' limits must be positive")
            wm = where + "mixer."
            size, keep = _window(m, wm)
            heads, dim = _int(m, "heads", wm), _int(m, "dim", wm)
            vdim = _int(m, "vdim", wm) if m.get("vdim") is not None else dim
            if kind == "attention":
                g = GroupedMixer(heads=heads, kv_heads=_int(m, "kv_heads", wm) if m.get("kv_heads") is not None else heads, dim=dim,
                                 vdim=vdim, scale=_num(m, "scale", wm) if m.get("scale") is not None else dim ** -0.5,
                                 rot=_rotation(m.get("rot"), wm + "rot.", dim), window=size, keep_first=keep)
                if g.heads % g.kv_heads:
                    raise ConfigError(f"config.json: {wm}heads ({g.heads}) must be a multiple of kv_heads ({g.kv_heads})")
                layers.append(NetezenLayer(kind=kind, grouped=g, dense_ff=dense_ff, moe=moe))
            elif kind == "latent_attention":
                rd = _int(m, "rot_dim", wm, least=0) if m.get("rot_dim") is not None else 0
                rot = _rotation(dict(m.get("rot") or {}, dims=rd), wm + "rot.", max(rd, 0)) if rd else Rotation(dims=0)
                la = LatentMixer(heads=heads, dim=dim, rot_dim=rd, vdim=vdim, kv_rank=_int(m, "kv_rank", wm),
                                 q_rank=_int(m, "q_rank", wm, least=0) if m.get("q_rank") is not None else 0,
                                 scale=_num(m, "scale", wm) if m.get("scale") is not None else (dim + rd) ** -0.5,
                                 rot=rot, window=size, sink=_has(shapes, f"l{i}.mix.sink", True))
                layers.append(NetezenLayer(kind=kind, latent=la, dense_ff=dense_ff, moe=moe))
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is neither 'attention' nor 'latent_attention'")
        return cls(vocab=vocab, width=width, norm_eps=eps,
                   residual_mult=_num(cfg, "residual_mult", "") if cfg.get("residual_mult") is not None else 1.0,
                   streams=streams, learned_streams=_has(shapes, "l0.hc1.in", cfg.get("streams") is not None), layers=tuple(layers))

    @staticmethod
    def _rot_dict(r: Rotation) -> Dict[str, Any]:
        d: Dict[str, Any] = {"base": r.base, "dims": r.dims}
        if r.scaling is not None:
            d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), r.scaling))
        return d

    def to_dict(self) -> Dict[str, Any]:
        out = []
        for L in self.layers:
            if L.kind == "attention":
                g = L.grouped
                mixer: Dict[str, Any] = {"dim": g.dim, "heads": g.heads, "kv_heads": g.kv_heads, "scale": g.scale, "vdim": g.vdim}
                if g.window:
                    mixer["mask"] = {"keep_first": g.keep_first, "size": g.window}
                if g.rot.dims:
                    mixer["rot"] = self._rot_dict(g.rot)
            else:
                a = L.latent
                mixer = {"dim": a.dim, "heads": a.heads, "kv_rank": a.kv_rank, "q_rank": a.q_rank, "rot_dim": a.rot_dim, "scale": a.scale,
                         "vdim": a.vdim}
                if a.window:
                    mixer["mask"] = {"size": a.window}
                if a.rot_dim:
                    mixer["rot"] = self._rot_dict(a.rot)
            mlp: Optional[Dict[str, Any]] = None
            if L.dense_ff:
                mlp = {"ff": L.dense_ff, "kind": "dense"}
            elif L.moe is not None:
                e = L.moe
                mlp = {"expert": {"ff": e.ff, "limit": e.limit}, "kind": "moe", "router": {"experts": e.experts, "top": e.top}}
                if e.shared_ff:
                    mlp["shared"] = {"ff": e.shared_ff, "limit": e.shared_limit}
            out.append({"mixer": mixer, "mlp": mlp, "type": L.kind})
        d: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "layers": out, "norm": {"eps": self.norm_eps},
                             "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.learned_streams:
            d["streams"] = self.streams
        return d

    @staticmethod
    def _position(r: Rotation, head_dim: int) -> PositionSpec:
        if not r.dims:
            return PositionSpec(kind="none", head_dim=head_dim, rotary_dim=0, theta=0.0)
        params: Dict[str, Any] = {"interleaved": True}
        if r.scaling is not None:
            params["yarn"] = dict(zip(("factor", "original", "fast", "slow"), r.scaling))
        return PositionSpec(kind="rope", head_dim=head_dim, rotary_dim=r.dims, theta=r.base, params=params)

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = NormSpec(kind="rmsnorm", size=W, eps=eps, params={"offset": 1.0})
        blocks = []
        for i, L in enumerate(self.layers):
            names = {"mixer_norm": "norm1", "ffn_norm": "norm2", "up": "mlp.up", "down": "mlp.down", "experts": "mlp.", "suffix": ""}
            if self.learned_streams:
                names.update({"mixer_hc": "hc1", "ffn_hc": "hc2"})
            if L.kind == "attention":
                g = L.grouped
                mixer = MixerSpec(kind="attention", hidden=W, n_heads=g.heads, n_kv_heads=g.kv_heads, head_dim=g.dim, window=g.window,
                                  scale=g.scale, position=self._position(g.rot, g.dim), params={"v_dim": g.vdim, "keep_first": g.keep_first})
                names.update({k: f"mix.{k}" for k in ("q", "k", "v", "o")})
            else:
                a = L.latent
                mixer = MixerSpec(kind="latent_attention", hidden=W, n_heads=a.heads, n_kv_heads=1, head_dim=a.dim, window=a.window,
                                  scale=a.scale, position=self._position(a.rot, a.rot_dim) if a.rot_dim else None,
                                  params={"v_dim": a.vdim, "kv_rank": a.kv_rank, "latent_eps": eps, "rot_dim": a.rot_dim, "q_rank": a.q_rank,
                                          "head_sink": a.sink})
                names.update({"q_down": "mix.dq", "q_norm": "mix.dq.norm", "q": "mix.uq" if a.q_rank else "mix.q", "latent": "mix.dkv",
                              "latent_norm": "mix.dkv.norm", "k_up": "mix.uk", "v_up": "mix.uv", "sink": "mix.sink", "o": "mix.o"})
            ffn = None
            if L.dense_ff:
                ffn = FeedForwardSpec(kind="mlp", hidden=W, intermediate=L.dense_ff, activation="relu2")
            elif L.moe is not None:
                e = L.moe
                params: Dict[str, Any] = {"experts": e.experts, "top": e.top, "scoring": "softmax", "correction": e.correction, "limit": e.limit}
                if e.shared_ff:
                    params["shared"] = {"ff": e.shared_ff, "activation": "swish_clamped", "limit": e.shared_limit}
                    params["shared_gate"] = True
                ffn = FeedForwardSpec(kind="moe", hidden=W, intermediate=e.ff, activation="swish_clamped", params=params)
            blocks.append(BlockSpec(kind="hyper", mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=norm if ffn is not None else None,
                                    prefix=f"l{i}.", names=names, residual_mult=self.residual_mult, streams=self.streams))
        return ModelSpec(architecture=self.ARCHITECTURE, vocab=self.vocab, hidden=W, max_position=MAX_POSITION, layers=blocks,
                         schedule=list(range(len(blocks))), final_norm=norm, tie_head=True, embed_name="embed",
                         final_norm_name="final.norm", head_name="head", stream="hyper", streams=self.streams)
