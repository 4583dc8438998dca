"""Typed configuration of the Lipizen decoder, read from its own config.json keys.

A Lipizen model is a stack of *post-norm* layers: x = N(a x + mixer(x)), then x = N(a x + ff(x)) with one factor a
(``postln_alpha``) for the whole model; the sublayers read the stream itself.  N is an RMS norm in groups
(``norm.groups`` equal parts of the row, each divided by its own root mean square).  A layer's mixer is one of two
kinds.  ``attention``: differential attention (two softmax maps per head over the same values, subtracted with one
weight a layer), grouped key heads, a short causal convolution on q, k and v, a norm on q and k, rotary positions on
the first ``rot.dims`` values with every frequency divided by ``rot.scaling.factor``, a sliding window that keeps a
sequence's first ``mask.keep_first`` positions visible, a gate a head; with ``kv_from`` the layer reads another
layer's keys and values.  ``hgrn2``: a linear recurrence whose forget gate (with a learned lower bound) also decides
what is written.  The feed-forward is dense with a clamped gated activation, or absent (``mlp: null``).  The logits
pass a soft cap.

config.json gives: ``vocab``, ``width``, ``norm`` {eps, groups}, ``postln_alpha``, ``logit_softcap`` and per entry of
``layers``: ``type``, ``mixer`` and ``mlp``:
  attention   mixer {heads, kv_heads, dim, vdim, scale, diff, conv, rot {dims, base[, scaling {factor}]},
                     mask {size, keep_first}[, kv_from]}
  hgrn2       mixer {heads, dim, vdim}
  mlp         {kind "dense", ff, limit}
Tensor names: ``embed``, ``final.norm``, ``head`` and under ``l<i>.``: ``norm1``, ``norm2``, ``mix.*``,
``mlp.{gate,up,down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .qwen2 import ConfigError
from .specs import BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
from .vunovik import _int, _num

MAX_POSITION = 1 << 20       # rotary positions have no end of their own


@dataclass(frozen=True)
class DiffMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    conv: int                                   # taps of the convolution on q, k, v; 0 = none
    rot_dims: int                               # 0 = nothing rotates
    rot_base: float
    rot_factor: float                           # every frequency is divided by it
    window: int                                 # 0 = every earlier position
    keep_first: int
    kv_from: Optional[int]


@dataclass(frozen=True)
class GateMixer:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class DenseSpec:
    ff: int
    limit: float


@dataclass(frozen=True)
class LipizenLayer:
    kind: str                                   # "attention" | "hgrn2"
    attention: Optional[DiffMixer] = None
    gate: Optional[GateMixer] = None
    mlp: Optional[DenseSpec] = None


def _attention(m: Dict[str, Any], where: str) -> DiffMixer:
    rot = m.get("rot")
    dims, base, factor = 0, 10000.0, 1.0
    if rot is not None:
        dims = _int(rot, "dims", where + "rot.", least=0)
        if dims:
            base = _num(rot, "base", where + "rot.")
            sc = rot.get("scaling")
            if sc is not None:
                factor = _num(sc, "factor", where + "rot.scaling.")
                if factor <= 0:
                    raise ConfigError(f"config.json: {where}rot.scaling.factor ({factor}) must be positive")
    mask = m.get("mask")
    window = _int(mask, "size", where + "mask.", least=0) if mask is not None and mask.get("size") is not None else 0
    keep = _int(mask, "keep_first", where + "mask.", least=0) if mask is not None and mask.get("keep_first") is not None else 0
    dim = _int(m, "dim", where)
    a = DiffMixer(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where) if m.get("kv_heads") is not None else _int(m, "heads", where),
                  dim=dim, vdim=_int(m, "vdim", where) if m.get("vdim") is not None else dim,
                  scale=_num(m, "scale", where) if m.get("scale") is not None else dim ** -0.5, diff=_num(m, "diff", where),
                  conv=_int(m, "conv", where, least=0) if m.get("conv") is not None else 0, rot_dims=dims, rot_base=base,
                  rot_factor=factor, window=window, keep_first=keep if window else 0,
                  kv_from=_int(m, "kv_from", where, least=0) if m.get("kv_from") is not None else None)
    if a.heads % a.kv_heads:
        raise ConfigError(f"config.json: {where}heads ({a.heads}) must be a multiple of kv_heads ({a.kv_heads})")
    if a.rot_dims % 2 or a.rot_dims > a.dim:
        raise ConfigError(f"config.json: {where}rot.dims ({a.rot_dims}) must be even and at most dim ({a.dim})")
    if a.conv > 16:
        raise ConfigError(f"config.json: {where}conv ({a.conv}) must be at most 16 taps")
    return a


@dataclass(frozen=True)
class LipizenConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    alpha: float
    softcap: float                              # 0 = the logits as they are
    layers: Tuple[LipizenLayer, ...]

    ARCHITECTURE = "Lipizen"

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "LipizenConfig":
        if cfg.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError(f"config.json: architecture {cfg.get('architecture')!r} is not '{cls.ARCHITECTURE}'")
        vocab, width = _int(cfg, "vocab", ""), _int(cfg, "width", "")
        norm = cfg.get("norm")
        eps = _num(norm, "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps ({eps}) must be positive")
        groups = _int(norm, "groups", "norm.") if norm.get("groups") is not None else 1
        if width % groups:
            raise ConfigError(f"config.json: norm.groups ({groups}) must divide the width ({width})")
        softcap = _num(cfg, "logit_softcap", "") if cfg.get("logit_softcap") is not None else 0.0
        if softcap < 0:
            raise ConfigError(f"config.json: logit_softcap ({softcap}) must not be negative")
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
            mlp = None
            if L.get("mlp") is not None:
                f = L["mlp"]
                if not isinstance(f, dict) or f.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {f.get('kind') if isinstance(f, dict) else f!r} is not 'dense'")
                mlp = DenseSpec(ff=_int(f, "ff", where + "mlp."), limit=_num(f, "limit", where + "mlp."))
                if mlp.limit <= 0:
                    raise ConfigError(f"config.json: {where}mlp.limit ({mlp.limit}) must be positive")
            if kind == "attention":
                a = _attention(m, where + "mixer.")
                if a.kv_from is not None:
                    src = layers[a.kv_from].attention if a.kv_from < i and layers[a.kv_from].kind == "attention" else None
                    if src is None or src.kv_from is not None:
                        raise ConfigError(f"config.json: {where}mixer.kv_from ({a.kv_from}) must name an earlier attention layer "
                                          f"with keys and values of its own")
                    if (src.kv_heads, src.dim, src.vdim) != (a.kv_heads, a.dim, a.vdim):
                        raise ConfigError(f"config.json: {where}mixer reads layer {a.kv_from}'s keys and values but differs from it in "
                                          f"kv_heads, dim or vdim")
                layers.append(LipizenLayer(kind=kind, attention=a, mlp=mlp))
            elif kind == "hgrn2":
                layers.append(LipizenLayer(kind=kind, gate=GateMixer(heads=_int(m, "heads", where + "mixer."),
                                                                     dim=_int(m, "dim", where + "mixer."),
                                                                     vdim=_int(m, "vdim", where + "mixer.")), mlp=mlp))
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is neither 'attention' nor 'hgrn2'")
        return cls(vocab=vocab, width=width, norm_eps=eps, norm_groups=groups,
                   alpha=_num(cfg, "postln_alpha", "") if cfg.get("postln_alpha") is not None else 1.0, softcap=softcap,
                   layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        out = []
        for L in self.layers:
            if L.kind == "attention":
                a = L.attention
                mixer: Dict[str, Any] = {"conv": a.conv, "diff": a.diff, "dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads,
                                         "scale": a.scale, "vdim": a.vdim}
                if a.window:
                    mixer["mask"] = {"keep_first": a.keep_first, "size": a.window}
                if a.rot_dims:
                    mixer["rot"] = {"base": a.rot_base, "dims": a.rot_dims, "scaling": {"factor": a.rot_factor}}
                if a.kv_from is not None:
                    mixer["kv_from"] = a.kv_from
            else:
                g = L.gate
                mixer = {"dim": g.dim, "heads": g.heads, "vdim": g.vdim}
            mlp = {"ff": L.mlp.ff, "kind": "dense", "limit": L.mlp.limit} if L.mlp is not None else None
            out.append({"mixer": mixer, "mlp": mlp, "type": L.kind})
        d: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "layers": out, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                             "postln_alpha": self.alpha, "vocab": self.vocab, "width": self.width}
        if self.softcap:
            d["logit_softcap"] = self.softcap
        return d

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = NormSpec(kind="group_rmsnorm", size=W, eps=eps, params={"groups": self.norm_groups})
        blocks = []
        # what a layer's pages must keep: the widest mask among the layers that read them (itself and those that name it)
        keeps: Dict[int, int] = {}
        for i, L in enumerate(self.layers):
            if L.kind == "attention":
                a = L.attention
                src = i if a.kv_from is None else a.kv_from
                every = a.window == 0 or a.keep_first > 0
                keeps[src] = 0 if every or keeps.get(src, -1) == 0 else max(keeps.get(src, -1), a.window)
        for i, L in enumerate(self.layers):
            names = {"mixer_norm": "norm1", "ffn_norm": "norm2", "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down", "suffix": ""}
            if L.kind == "attention":
                a = L.attention
                pos = (PositionSpec(kind="rope", head_dim=a.dim, rotary_dim=a.rot_dims, theta=a.rot_base, params={"linear": a.rot_factor})
                       if a.rot_dims else PositionSpec(kind="none", head_dim=a.dim, rotary_dim=0, theta=0.0))
                mixer = MixerSpec(kind="diff_attention", hidden=W, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim,
                                  window=a.window, scale=a.scale, position=pos, cache_from=a.kv_from,
                                  params={"v_dim": a.vdim, "diff": a.diff, "taps": a.conv, "keep_first": a.keep_first, "eps": eps,
                                          "cache_window": keeps.get(i, 0)})
                names.update({k: f"mix.{k}" for k in ("q", "k", "v", "g", "o", "lq1", "lk1", "lq2", "lk2")})
            else:
                g = L.gate
                mixer = MixerSpec(kind="gated_recurrence", hidden=W, n_heads=g.heads, n_kv_heads=g.heads, head_dim=g.dim,
                                  params={"v_dim": g.vdim, "eps": eps})
                names.update({"q": "mix.q", "f": "mix.f", "f_bias": "mix.f.b", "lower": "mix.lower", "v": "mix.v", "norm": "mix.norm",
                              "o": "mix.o"})
            ffn = None
            if L.mlp is not None:
                ffn = FeedForwardSpec(kind="gated_mlp", hidden=W, intermediate=L.mlp.ff, activation="swish_clamped",
                                      params={"limit": L.mlp.limit})
            blocks.append(BlockSpec(kind="postnorm", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    ffn_norm=norm if ffn is not None else None, prefix=f"l{i}.", names=names, stream_mult=self.alpha))
        return ModelSpec(architecture=self.ARCHITECTURE, vocab=self.vocab, hidden=W, max_position=MAX_POSITION, layers=blocks,
                         schedule=list(range(len(blocks))), final_norm=norm, tie_head=False, embed_name="embed",
                         final_norm_name="final.norm", head_name="head", logit_softcap=self.softcap)
