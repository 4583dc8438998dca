"""A model put together from a ModelSpec: embedding, the blocks in the order of the schedule, final
norm and head; its cache; and the one step function that prefill, decoding, generation and trace
replay all go through.

The reference's counterparts: ``Transformer::build`` (src/models/transformer.rs:778-1002),
``forward_chunk_at`` (:1012-1321), ``project_logits`` (:1631-1652); one sequence there, a ragged
batch of sequences here.
"""
from __future__ import annotations

import dataclasses
import sys
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.kv import KVCache, StateRequest
from ..config.registry import lookup_architecture, read_config_json
from ..config.specs import ModelSpec
from ..parts import Linear, Runtime, build_block, build_norm
from ..parts.linear import FOLDED_NORM_ROWS
from ..parts.norm import RowsInfo
from ..weights.loader import TensorSpec, tensor_names
from .batch import StepBatch, StepEntry, build_batch, check_entries
from .fit import STEP_ROWS

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(d) -> torch.dtype:
    if d not in _DTYPES:
        raise ValueError(f"dtype {d!r} is not one of bfloat16, float32")
    return _DTYPES[d]


def build_plan(spec: ModelSpec, rt: Optional[Runtime] = None) -> Dict[str, TensorSpec]:
    """Every tensor the model reads, by name (needs no GPU: parts are built but not loaded)."""
    rt = rt or Runtime(kernels=None, dtype=torch.bfloat16, device="cpu")
    return Model(spec, rt).plan()


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec, self.rt = spec, rt
        for i in spec.schedule:
            if not (0 <= i < len(spec.layers)):
                raise ValueError(f"the schedule names layer {i}; the model has {len(spec.layers)}")
        self.blocks = [build_block(b, i, rt) for i, b in enumerate(spec.layers)]
        self.final_norm = build_norm(spec.final_norm, rt)
        if spec.stream not in ("residual", "depth_average", "hyper"):
            raise ValueError(f"the model's stream '{spec.stream}' is none of 'residual', 'depth_average', 'hyper'")
        if spec.stream == "hyper":
            for i, b in enumerate(spec.layers):
                if b.kind != "hyper" or b.streams != spec.streams:
                    raise ValueError(f"a model of {spec.streams} streams needs blocks of kind 'hyper' with as many; layer {i} is "
                                     f"'{b.kind}' with {b.streams}")
            if spec.final_norm.kind != "rmsnorm":
                raise ValueError("a model with several streams sums them in front of a final norm of kind 'rmsnorm'")
            self._ones = None                               # the final reader's weights: the streams are summed
        self.depth = None                                   # what a layer reads: the stream itself, or a depth average
        if spec.stream == "depth_average":
            from ..parts.depth_average import DepthAverage
            if len(spec.depth_names) != len(spec.schedule):
                raise ValueError(f"a depth average needs one vector per site: {len(spec.depth_names)} names for "
                                 f"{len(spec.schedule)} sites")
            self.depth = DepthAverage(spec.depth_names, rt)
        self.config = None                                  # set by load_model
        self.step_rows = STEP_ROWS                          # a step of more rows runs in parts
        self.embedding: Optional[torch.Tensor] = None
        self.bigram: Optional[torch.Tensor] = None          # the hashed bigram table, where the spec has one
        self.head: Optional[Linear] = None
        self.cache: Optional[KVCache] = None

    # ------------------------------------------------------------------ weights
    def plan(self) -> Dict[str, TensorSpec]:
        s = self.spec
        p: Dict[str, TensorSpec] = {s.embed_name: TensorSpec((s.vocab, s.hidden))}
        if s.embed_bigram is not None:
            p[s.embed_bigram.name] = TensorSpec((s.embed_bigram.buckets + 1, s.hidden))
        for b in self.blocks:
            p.update(b.plan())
        if self.depth is not None:
            p.update(self.depth.plan())
        p.update(self.final_norm.plan(s.final_norm_name))
        if not s.tie_head:
            p[s.head_name] = TensorSpec((s.vocab, s.hidden))
        return p

    def ignorable(self) -> List[str]:
        """Names a checkpoint may hold without the model reading them."""
        pats = ["*.rotary_emb.inv_freq"]
        if self.spec.tie_head:
            pats.append(self.spec.head_name)
        return pats

    def load(self, tensors) -> None:
        """``tensors``: name -> tensor, a dict or a ``TensorSource`` that fetches each tensor when it is asked for
        (every name of the plan is asked for once)."""
        s = self.spec
        table = tensors[s.embed_name]
        self.embedding = self.rt.matrix(table)
        if s.tie_head:
            self.head = Linear(self.embedding, None, self.rt)     # one copy on the device serves both
        del table
        if s.embed_bigram is not None:
            self.bigram = self.rt.matrix(tensors[s.embed_bigram.name]).to(self.embedding.dtype)
        for b in self.blocks:
            b.load(tensors)
        if self.depth is not None:
            self.depth.load(tensors)
        self.final_norm.load(tensors, s.final_norm_name)
        if not s.tie_head:
            self.head = Linear(tensors[s.head_name], None, self.rt)

    def state_dict(self) -> Dict[str, torch.Tensor]:
        """Every tensor of the plan by its name, as it is kept on the device (matrices in the model's precision or
        the 32 bits they were stored in, vectors in float32); stacked matrices come back as views of their rows."""
        s = self.spec
        out: Dict[str, torch.Tensor] = {s.embed_name: self.embedding}
        if self.bigram is not None:
            out[s.embed_bigram.name] = self.bigram
        for b in self.blocks:
            out.update(b.state())
        if self.depth is not None:
            out.update(self.depth.state())
        out.update(self.final_norm.state(s.final_norm_name))
        if not s.tie_head:
            out[s.head_name] = self.head.weight
        return out

    @property
    def short_context(self) -> int:
        """The bound of the context class for which decode steps are recorded apart: the smallest that a mixer
        names (``mixer.short_context``), 0 if none does."""
        named = [int(getattr(b.mixer, "short_context", 0) or 0) for b in self.blocks if hasattr(b, "mixer")]
        named = [n for n in named if n > 0]
        return min(named) if named else 0

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step may be recorded as a CUDA graph: every layer's parts and the final norm say so."""
        return (all(getattr(b, "graph_safe", False) for b in self.blocks) and getattr(self.final_norm, "graph_safe", False)
                and (self.depth is None or self.depth.graph_safe))

    def weight_bytes(self, rows: int = 1) -> int:
        """Bytes a decode step of ``rows`` sequences reads of the weights: every block, final norm and head once
        (embedding rows excluded unless the head shares the table); of a routed feed-forward the experts that
        ``rows`` tokens can reach (``extra_bytes(rows)`` of a part, beyond what one token reads)."""
        extra = 0
        if rows > 1:
            for b in self.blocks:
                ff = getattr(b, "feed_forward", None)
                if ff is not None and hasattr(ff, "extra_bytes"):
                    extra += ff.extra_bytes(rows)
        return (sum(b.nbytes() for b in self.blocks) + self.final_norm.nbytes() + self.head.nbytes()
                + (self.depth.nbytes() if self.depth is not None else 0) + extra)

    # ------------------------------------------------------------------ cache
    def make_cache(self, max_tokens: int, max_seqs: Optional[int] = None, page_size: int = 64,
                   extra_state: Sequence[StateRequest] = ()) -> KVCache:
        # storage belongs to a *site* (an entry of the schedule), weights to a layer: a layer that
        # runs twice keeps the keys and values of each run apart
        sched = self.spec.schedule
        shares = {site: self.spec.layers[layer].mixer.cache_from for site, layer in enumerate(sched)
                  if self.spec.layers[layer].mixer.cache_from is not None}
        self.cache = KVCache(self._cache_requests(),
                             max_tokens, self.spec.max_position,
                             self.rt.dtype, self.rt.device, page_size=page_size, max_seqs=max_seqs,
                             shares=shares, extra_state=extra_state)
        return self.cache

    BIGRAM_STATE = "embed.bigram_prev"

    def _cache_requests(self):
        """What every site asks of the cache; the token before a sequence's next one (the bigram embedding's state,
        one int32 a slot) is asked for with the first site, as state that belongs to a sequence's end."""
        reqs = [list(self.blocks[layer].cache_requests(site)) for site, layer in enumerate(self.spec.schedule)]
        if self.spec.embed_bigram is not None:
            if not reqs:
                reqs.append([])
            reqs[0].append(StateRequest(self.BIGRAM_STATE, (), torch.int32))
        return reqs

    def forecast(self, max_tokens: int, max_seqs: Optional[int] = None, page_size: int = 64,
                 extra_state: Sequence[StateRequest] = ()):
        """Bytes that the weights, a cache of ``max_tokens`` positions and a step's scratch will take."""
        from .fit import forecast
        sched = self.spec.schedule
        shares = [site for site, layer in enumerate(sched) if self.spec.layers[layer].mixer.cache_from is not None]
        widest = max([int(getattr(b, "scratch_row", lambda: 0)()) for b in self.blocks] + [self.spec.hidden])
        return forecast(self.plan(), self._cache_requests(),
                        self.rt.dtype, max_tokens, self.spec.hidden, self.spec.vocab, widest, page_size, shares,
                        extra_state, max_seqs or 0,
                        streams=len(sched) + 2 if self.depth is not None else (self.spec.streams + 1 if self.spec.stream == "hyper" else 1))

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the tokens the entries bring, from the cache earlier steps left; float32 logits
        ``[wanted, vocab]`` in the order of the entries and of their ``want``."""
        cache = self.cache
        if cache is None:
            raise RuntimeError("the model has no cache yet: call make_cache first")
        entries = list(entries)
        for e in entries:
            if not cache.slots.is_held(e.slot):
                raise ValueError(f"slot {e.slot} is not open")
        starts = [cache.length(e.slot) for e in entries]
        # the whole step fits or nothing is taken: a step that fails leaves the cache as it found it
        cache.must_fit([(e.slot, s + len(e.tokens)) for e, s in zip(entries, starts)])
        if sum(len(e.tokens) for e in entries) > self.step_rows:
            return self._step_in_parts(entries)
        return self._step_within_bound(entries, starts)

    def _step_within_bound(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> torch.Tensor:
        cache = self.cache
        limit = cache.most_tokens_going_on()
        if limit is not None and any(starts) and max(len(e.tokens) for e in entries) > limit:
            return self._step_in_rounds(entries, limit)
        batch = build_batch(entries, starts, self.spec.vocab, self.rt.device)
        for e, s in zip(entries, starts):
            cache.reserve(e.slot, s + len(e.tokens))
        cache.flush()
        logits = self.forward(batch)
        for e, s in zip(entries, starts):
            cache.commit(e.slot, s + len(e.tokens))
        return logits

    def _step_in_parts(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A step of more rows than ``step_rows`` (the number the forecast of a step's scratch counts on) as several:
        its sequences in their order, as many at a time as stay within the bound; a sequence that alone exceeds it
        in rounds of ``step_rows`` tokens (its later rounds go on from the cache).  Sequences do not depend on one
        another and a sequence's logits not on how its tokens are cut, so the logits are the step's own, in the
        order of the entries and of their ``want``.  With a window's ring of pages a prompt that starts is left
        whole however long (it reads its own rows, while rounds that go on may add a page at most)."""
        check_entries(entries, self.spec.vocab)
        cache = self.cache
        ring = cache.most_tokens_going_on() is not None
        parts, group, rows = [], [], 0

        def run_group():
            nonlocal group, rows
            if group:
                parts.append(self._step_within_bound(group, [cache.length(e.slot) for e in group]))
            group, rows = [], 0

        for e in entries:
            n = len(e.tokens)
            if n > self.step_rows:
                run_group()
                if ring and cache.length(e.slot) == 0:
                    group = [e]
                    run_group()
                else:
                    parts.append(self._step_in_rounds([e], self.step_rows))
                continue
            if rows + n > self.step_rows:
                run_group()
            group.append(e)
            rows += n
        run_group()
        return torch.cat(parts)

    def _step_in_rounds(self, entries: Sequence[StepEntry], most: int) -> torch.Tensor:
        """The same step as rounds of at most ``most`` tokens a sequence (see ``KVCache.most_tokens_going_on``);
        the logits come back in the order of the entries and of their ``want``, as from one step."""
        for i, e in enumerate(entries):
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise ValueError(f"entry {i}: wanted place {w} is outside its {len(e.tokens)} tokens")
        parts, place = [], {}                                 # (entry, index in its want) -> row among all rounds' logits
        done_rows = 0
        for lo in range(0, max(len(e.tokens) for e in entries), most):
            sub = []
            for i, e in enumerate(entries):
                if lo >= len(e.tokens):
                    continue
                want = []
                for k, w in enumerate(e.want):
                    if lo <= w < lo + most:
                        place[(i, k)] = done_rows + sum(len(x.want) for x in sub) + len(want)
                        want.append(w - lo)
                sub.append(StepEntry(e.slot, e.tokens[lo:lo + most], want))
            parts.append(self.step(sub))
            done_rows += parts[-1].shape[0]
        order = [place[(i, k)] for i, e in enumerate(entries) for k in range(len(e.want))]
        logits = torch.cat(parts)
        return logits[torch.as_tensor(order, dtype=torch.long, device=logits.device)] if order else logits

    def check_device(self) -> None:
        """Raise if a bounded wait inside a kernel ran out since the last check (synchronises)."""
        k = self.rt.kernels
        if hasattr(k, "device_errors") and k.device_errors():
            raise RuntimeError("a kernel's bounded wait ran out (TMA or tensor-core pipeline): results are invalid")

    def forward(self, batch: StepBatch) -> torch.Tensor:
        K_, s = self.rt.kernels, self.spec
        if self.depth is not None:
            return self._forward_depth_average(batch)
        if s.stream == "hyper":
            return self._forward_hyper(batch)
        x = self.rt.empty(batch.n_rows, s.hidden, dtype=torch.float32)
        # What a kernel leaves behind about the rows it wrote travels along as a RowsInfo, so that norms are
        # folded into the products around them (few rows) or run together with the residual add (many rows).
        info = None
        order = [self.blocks[layer] for layer in s.schedule]
        if s.embed_bigram is not None:
            g = s.embed_bigram
            K_.embed_bigram(batch, self.embedding, self.bigram, x, s.embed_scale, g.buckets, g.mul_prev, g.mul_cur,
                            self.cache.state[self.BIGRAM_STATE])
        elif batch.n_rows <= FOLDED_NORM_ROWS and not self.rt.full_precision:
            ssq = self.rt.empty(batch.n_rows, 1, dtype=torch.float32)
            first = getattr(order[0], "mixer_norm", None) if order else self.final_norm
            if (getattr(first, "weight", None) is not None and first.spec.kind == "rmsnorm"
                    and first.spec.size == s.hidden):
                xw = self.rt.empty(batch.n_rows, s.hidden)
                K_.embed(batch.tokens, self.embedding, x, s.embed_scale, ssq, first.weight, xw)
                info = RowsInfo(ssq=ssq, xw=xw, xw_norm=first)
            else:
                K_.embed(batch.tokens, self.embedding, x, s.embed_scale, ssq)
                info = RowsInfo(ssq=ssq)
        else:
            K_.embed(batch.tokens, self.embedding, x, s.embed_scale)
        for site, block in enumerate(order):
            if site + 1 < len(order):
                nxt = getattr(order[site + 1], "mixer_norm", None)
            else:
                nxt = self.final_norm if batch.want_all_in_order else None
            info = block.forward(x, batch, self.cache, site, info, nxt)
        return self.project(x, batch, info)

    def _forward_depth_average(self, batch: StepBatch) -> torch.Tensor:
        """The same loop where a layer reads a depth average: the step keeps every stream (``DepthAverage``), site s
        adds into plane s + 1, and the average that follows it, with the next norm, is one kernel."""
        K_, s = self.rt.kernels, self.spec
        order = [self.blocks[layer] for layer in s.schedule]
        stack = self.depth.begin(batch.n_rows, s.hidden)
        K_.embed(batch.tokens, self.embedding, stack[0], s.embed_scale)
        x, info = self.depth.start(stack), None
        for site, block in enumerate(order):
            block.forward(x, batch, self.cache, site, info, None)
            conv = None
            if site + 1 < len(order):
                nxt = getattr(order[site + 1], "mixer_norm", None)
                if getattr(order[site + 1], "conv", None) is not None:
                    conv = (order[site + 1].conv, batch, self.cache, site + 1)
            else:
                nxt = self.final_norm if batch.want_all_in_order else None
            x, info = self.depth.after(stack, site, nxt, conv)
        return self.project(x, batch, info)

    def _forward_hyper(self, batch: StepBatch) -> torch.Tensor:
        """The same loop over several copies of the stream (``HyperBlock``): the embedding's rows become every copy and
        the first block's input in one launch; each block's last launch forms the next block's input; behind the last
        block the copies are summed and normed, for every row where all are wanted, else for the wanted rows only."""
        K_, s = self.rt.kernels, self.spec
        from ..parts.norm import RowsInfo
        S, T = s.streams, batch.n_rows
        order = [self.blocks[layer] for layer in s.schedule]
        if self._ones is None:
            self._ones = self.rt.vector(torch.ones(S))
        last = (self._ones, self.final_norm)
        e = self.rt.empty(T, s.hidden, dtype=torch.float32)
        K_.embed(batch.tokens, self.embedding, e, s.embed_scale)
        xs = self.rt.empty(T, S, s.hidden, dtype=torch.float32)
        first = order[0].reader if order else (last if batch.want_all_in_order else None)
        h = self.rt.empty(T, s.hidden) if first is not None else None
        K_.hyper_connect(xs, e, None, None, 1.0, first[0] if first else None, first[1].weight if first else None,
                         first[1].spec.eps if first else 0.0, h, spread=True)
        info = RowsInfo(norm=first[1], h=h) if first is not None else None
        for site, block in enumerate(order):
            if site + 1 < len(order):
                nxt = order[site + 1].reader
            else:
                nxt = last if batch.want_all_in_order else None
            info = block.forward(xs, batch, self.cache, site, info, nxt)
        if batch.n_want == 0:
            return torch.empty((0, s.vocab), dtype=torch.float32, device=self.rt.device)
        if info is not None and info.norm is self.final_norm and info.h is not None:
            logits = self.head.logits(info.h)
        else:
            flat = xs.view(T, S * s.hidden)
            if not batch.want_all_in_order:
                picked = self.rt.empty(batch.n_want, S * s.hidden, dtype=torch.float32)
                K_.gather_rows(flat, batch.want_rows, picked)
                flat = picked
            h = self.rt.empty(flat.shape[0], s.hidden)
            K_.hyper_connect(flat.view(flat.shape[0], S, s.hidden), None, None, None, 1.0, last[0], self.final_norm.weight,
                             self.final_norm.spec.eps, h)
            logits = self.head.logits(h)
        if s.logit_softcap > 0 and logits.shape[0] > 0:
            K_.softcap(logits, s.logit_softcap)
        return logits

    def project(self, x: torch.Tensor, batch: StepBatch, info=None) -> torch.Tensor:
        """Final norm and head at the wanted rows only; the logits capped softly where the spec says so."""
        logits = self._project(x, batch, info)
        if self.spec.logit_softcap > 0 and logits.shape[0] > 0:
            self.rt.kernels.softcap(logits, self.spec.logit_softcap)
        return logits

    def _project(self, x: torch.Tensor, batch: StepBatch, info=None) -> torch.Tensor:
        if batch.n_want == 0:
            return torch.empty((0, self.spec.vocab), dtype=torch.float32, device=self.rt.device)
        if not batch.want_all_in_order:
            picked = self.rt.empty(batch.n_want, self.spec.hidden, dtype=torch.float32)
            self.rt.kernels.gather_rows(x, batch.want_rows, picked)
            x, info = picked, None
        if info is not None and getattr(info, "norm", None) is self.final_norm and info.h is not None:
            return self.head.logits(info.h)
        if hasattr(self.final_norm, "lazy"):
            ssq = getattr(info, "ssq", None) if info is not None else None
            xw = info.xw if (info is not None and getattr(info, "xw_norm", None) is self.final_norm) else None
            return self.head.logits(self.final_norm.lazy(x, ssq, xw))
        return self.head.logits(self.final_norm(x))


def settle_head(spec: ModelSpec, stored: Sequence[str], warn=None) -> ModelSpec:
    """The spec with the head tied to the table if the architecture allows a checkpoint without a head
    tensor and this one has none (src/models/transformer.rs:810: tied = the flag, or no lm_head.weight)."""
    names = [spec.head_name] + [spec.head_name[len(p):] for p in spec.optional_prefixes if spec.head_name.startswith(p)]
    if spec.tie_head or not spec.head_may_be_absent or any(n in stored for n in names):
        return spec
    if warn is not None:
        warn(f"{spec.head_name} absent: the embedding table serves as the head")
    return dataclasses.replace(spec, tie_head=True)


def load_model(folder: Optional[str] = None, dtype="bfloat16", max_tokens: int = 4096, max_seqs: Optional[int] = None,
               device="cuda:0", kernels=None, verbose: bool = True, config=None, seed: int = 0,
               draw: str = "cpu") -> Model:
    """A model from a folder with config.json and model.safetensors, or, without a folder, from ``config`` (a
    config.json dict or the architecture's typed configuration) with random weights drawn from ``seed``; its
    class is chosen by the configuration either way, and both go through the same steps: the fit check, the parts'
    ``load`` from a source that hands out one tensor at a time, the cache.  ``draw``: where the random values are
    drawn, "cpu" (the values that ``write_random_model`` stores for this seed) or "device" (the device's own
    generator: other values, seconds instead of a minute for a 7B shape).  The reference's in-memory stand-in for
    a checkpoint takes the same road as a file (src/selftest.rs:23-159)."""
    from ..kernels import Kernels
    from ..weights.loader import CheckpointTensors, RandomTensors
    if (folder is None) == (config is None):
        raise ValueError("load_model takes a model folder or a configuration, one of the two")
    if folder is not None:
        raw = read_config_json(folder)
    else:
        raw = config.to_dict() if hasattr(config, "to_dict") else dict(config)
    entry = lookup_architecture(raw)
    if folder is not None and entry.parse_with_shapes is not None:
        from ..weights.loader import tensor_shapes
        typed = entry.parse_with_shapes(raw, tensor_shapes(folder))      # sizes that only the tensors' shapes give
    else:
        typed = entry.parse(raw)
    spec = entry.spec(typed)
    if folder is not None:
        spec = settle_head(spec, tensor_names(folder),
                           warn=(lambda m: print(f"[cima_b200] {m}", file=sys.stderr, flush=True)) if verbose else None)
    rt = Runtime(kernels=kernels if kernels is not None else Kernels(verbose=verbose),
                 dtype=parse_dtype(dtype), device=device)
    model = Model(spec, rt)
    model.config = typed                                    # the architecture's typed configuration, as parsed
    from ..sampling.sampler import sampler_state
    from .fit import check_fit
    check_fit(model.forecast(max_tokens, max_seqs, extra_state=sampler_state()), device)     # before anything is allocated
    if folder is not None:
        source = CheckpointTensors(folder, model.plan(), ignore=model.ignorable(), optional_prefixes=spec.optional_prefixes)
    else:
        if draw not in ("cpu", "device"):
            raise ValueError(f"draw '{draw}' is neither 'cpu' nor 'device'")
        source = RandomTensors(model.plan(), seed, torch.bfloat16, device if draw == "device" else "cpu")
    with source:
        model.load(source)
    model.load_peak_host_bytes = source.peak_bytes          # most bytes of fetched tensors alive at once while loading
    model.make_cache(max_tokens, max_seqs, extra_state=sampler_state())
    return model
