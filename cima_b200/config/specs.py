"""Descriptions of a model as data: one spec per part, one per block, one per model.

An architecture's typed configuration (``qwen2.py``) turns its ``config.json``
keys into these specs; the parts (``cima_b200/parts``) are built from them and
know nothing else about the model they sit in.  Every size and constant is a
field here; none stands in the parts' code.

``kind`` selects the implementation from the part registries
(``cima_b200/parts/registry.py``); ``params`` carries what a kind needs beyond
the common fields, so that a kind defined outside the package needs no change
to these classes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    kind: str                    # "rmsnorm" (params["offset"] c: the stored weight w multiplies as c + w; default 0)
                                 # | "dyt" (tanh(alpha x) * w + b: no row statistics, eps unused)
                                 # | "group_rmsnorm" (params["groups"] equal parts of a row, each divided by its own root mean square)
    size: int
    eps: float
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class PositionSpec:
    kind: str                    # "rope" | "none"
    head_dim: int
    rotary_dim: int              # how many leading dims of a head rotate (<= head_dim, even)
    theta: float
    # "scaling": {"factor", "low", "high", "original"}: frequencies rescaled by their wavelength (see parts/position.py);
    # "linear": a factor every frequency is divided by;
    # "yarn": {"factor", "original", "fast", "slow"}: frequencies blended by their index between f and f / factor, sine and
    # cosine multiplied by 0.1 ln(factor) + 1;  "interleaved": True = neighbours (2i, 2i + 1) form a pair, not (i, i + rotary_dim / 2)
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class MixerSpec:
    """Only ``kind`` and ``hidden`` are every mixer's; the fields after them describe an attention and keep their
    defaults for a mixer that has no heads (a recurrence, a convolution), which puts its own sizes in ``params``."""
    kind: str                    # "attention"
    hidden: int
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = False
    out_bias: bool = False
    window: int = 0              # 0 = every earlier key; w > 0 = the last w keys
    scale: float = 0.0           # factor of q.k before the softmax
    position: Optional[PositionSpec] = None
    # Site (index into ModelSpec.schedule) whose keys and values this layer reads instead of
    # writing its own; None = own cache.
    cache_from: Optional[int] = None
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                    # "gated_mlp"
    hidden: int
    intermediate: int
    activation: str              # "silu"; "swish_clamped" takes params["limit"]
    bias: bool = False
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ShortConvSpec:
    """A causal convolution over time on each channel, added to its input: u_t = h_t + sum_j w[:, j] h_(t-taps+1+j),
    nothing before position 0.  A sequence carries its newest ``taps - 1`` inputs along as state."""
    channels: int
    taps: int


@dataclass(frozen=True)
class BigramSpec:
    """A second embedding table beside the token table, addressed by a hash of the token and the one before it:
    row (prev * mul_prev + tok * mul_cur) mod buckets, and row ``buckets`` (the table's last) for a sequence's first
    token.  The token before a step's first row travels with the sequence as state."""
    name: str
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class BlockSpec:
    kind: str                    # "prenorm": x += mixer(norm(x)); x += ffn(norm(x))
                                 # "parallel": h = norm(x); x += mixer(conv(h)) + ffn(h)
                                 # "sandwich": x += m * post(mixer(norm(x))); x += m * post(ffn(norm(x)))
                                 # "postnorm": x = norm(a x + mixer(x)); x = norm(a x + ffn(x)), a = stream_mult
                                 # "hyper": ``streams`` copies X_s of the stream; a sublayer reads norm(sum_s in[s] X_s) and
                                 #          X_t <- sum_s mix[s, t] X_s + m out[t] y for all t at once, m = residual_mult
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]      # None: the layer has no feed-forward ("parallel" only)
    mixer_norm: NormSpec
    ffn_norm: Optional[NormSpec]                 # None where one norm serves both sublayers
    prefix: str                  # tensor-name prefix of the layer, e.g. "model.layers.3."
    # tensor-name stems under the prefix, owned by the architecture's naming; a matrix or norm weight is
    # prefix + stem + names.get("suffix", ".weight")
    names: Dict[str, str] = field(default_factory=dict)
    # a short convolution in front of the mixer (its weight's stem is names["mixer_conv"]); None = none
    mixer_conv: Optional[ShortConvSpec] = None
    # "sandwich": the norms behind the sublayers (stems names["mixer_post_norm"], names["ffn_post_norm"]) and the
    # factor of what a sublayer adds to the stream
    mixer_post_norm: Optional[NormSpec] = None
    ffn_post_norm: Optional[NormSpec] = None
    residual_mult: float = 1.0
    # "postnorm": the factor of the stream in the sum that the norm behind a sublayer reads
    stream_mult: float = 1.0
    # "hyper": how many copies of the stream the model carries.  With names["mixer_hc"] / names["ffn_hc"] the vectors
    # <stem>.in, <stem>.out [streams] and the matrix <stem>.mix [streams, streams] (indexed [from, to]) of a sublayer are
    # stored tensors; without those names they are ones and the unit matrix (one stream: x += m * sublayer(norm(x)))
    streams: int = 1


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab: int
    hidden: int
    max_position: int
    layers: List[BlockSpec]
    # The order in which layers run: indices into ``layers``.  A layer may be named
    # twice; default is each layer once, in order.
    schedule: List[int]
    final_norm: NormSpec
    tie_head: bool
    embed_name: str
    final_norm_name: str
    head_name: str
    embed_scale: float = 1.0
    embed_bigram: Optional[BigramSpec] = None       # a hashed bigram table added to the token embedding
    logit_softcap: float = 0.0                      # c > 0: logits <- c * tanh(logits / c)
    # A checkpoint of an untied model that stores no head tensor: the table serves as the head
    # (the reference decides so, src/models/transformer.rs:810, and warns, :839-841).
    head_may_be_absent: bool = False
    # Prefixes of the tensor names above that a checkpoint may leave out (a bare backbone stores
    # "layers.0..." for "model.layers.0..."; the reference tries both, src/models/transformer.rs:472-488).
    optional_prefixes: Tuple[str, ...] = ()
    # What a layer reads.  "residual": the stream as the layer before left it.  "depth_average": with X_0 the
    # embedding's output and X_(s+1) the stream as site s leaves it, the next site (and the final norm) reads
    # sum_(j <= s+1) a_s[j] X_j; ``depth_names[s]`` names the vector a_s (s + 2 values) of site s.
    # "hyper": the step carries ``streams`` copies of the stream, all equal to the embedding's output at the start and
    # summed in front of the final norm; every layer is a block of kind "hyper" with as many streams.
    stream: str = "residual"
    depth_names: Tuple[str, ...] = ()
    streams: int = 1

    def describe(self) -> str:
        kinds = [f"{self.layers[i].mixer.kind}"
                 f"{'(w=%d)' % self.layers[i].mixer.window if self.layers[i].mixer.window else ''}"
                 f"+{self.layers[i].feed_forward.kind if self.layers[i].feed_forward else 'none'}" for i in self.schedule]
        return (f"{self.architecture}: vocab {self.vocab}, hidden {self.hidden}, "
                f"{len(self.layers)} layers, schedule {kinds}")
