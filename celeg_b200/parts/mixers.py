"""Mixer parts. Interface of a mixer:

    Mixer(params, weights, parts, rt)       parts: built nested parts (e.g. {"position": ...})
    cache_need() -> PagedNeed | StateNeed | None
    bind_cache(binding)                     PagedBinding or StateBinding from the cache storage
    forward(x, out, step)                   x: normed activations [T, hidden]; writes the
                                            mixer's output (to be added to the residual) to out
    takes_split_norm(step) -> bool          optional: True if forward() hands x to the runtime's products
                                            only, which can apply a row scale that x still lacks (then x
                                            may be a kernels.SplitNorm instead of a tensor)
    ends_with_product = True                optional: the last thing forward() does to ``out`` is
                                            rt.linear(..., out, ...); the runtime may then add that product
                                            to the residual stream itself and leave ``out`` unwritten

A mixer does not know which model or layer it is in; everything it needs about the step is
in the StepContext, everything about its cache in the binding.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Mapping, Optional

import torch

from .. import kernels
from ..cache.manager import PagedNeed, StateNeed
from .registry import register_part
from .runtime import Runtime, StepContext


@dataclass
class PagedBinding:
    """Where a paged mixer's keys and values live: one layer of a group's storage,
    [pages, kv_heads, page_tokens, head_dim] each; ``owner`` False = read only (the cache
    belongs to an earlier layer of the run order)."""
    group: int
    k: torch.Tensor
    v: torch.Tensor
    page_tokens: int
    owner: bool = True


@dataclass
class StateBinding:
    """Where a fixed-state mixer's state lives: ``state`` is a view [slots, elements] of the
    slot slab; ``slot_stride`` floats separate one slot from the next."""
    state: torch.Tensor
    slot_stride: int
    owner: bool = True


# Blocks of the decode attention that a B200 holds at a time at a head size of 64 (148 SMs x 5): what the times
# of its launches at 1 to 256 requests and 2 k to 130 k keys fit (see decode_split). A mixer asks the kernel
# library for the number of its own head size on its own device.
DECODE_RESIDENT_BLOCKS = 740


def decode_split(tokens: int, kv_heads: int, context_bucket: int, window: Optional[int], max_context: int,
                 resident_blocks: int = DECODE_RESIDENT_BLOCKS):
    """How the decode attention splits the keys of a step of ``tokens`` requests: (chunk, max_splits,
    cap_splits). Every request's keys are cut into chunks of ``chunk`` (a multiple of 64); ``max_splits`` chunks
    cover the step's context bucket and ``cap_splits`` >= max_splits is what the scratch is sized for, a
    number that depends only on the longest context the runtime allows.

    Few requests with short contexts: enough splits for about one and a half blocks per SM, chunks of at most
    1,024 keys. Where that limit binds (many requests or long contexts) the chunk grows up to 4,096 keys: fewer
    blocks start and fewer partial results are merged. The launch's blocks (requests x kv heads x splits) run
    in rounds of ``resident_blocks``. If one round can hold them, about half a round is asked for: the
    times fall off sharply just above a whole round (2 requests at 65 k keys: 60 us with 720 blocks, 75 us with
    816) and are flat or a little better towards half of one (1 request at 130 k: 70 us with 712 blocks, 63 us
    with 368; at 65 k 41 us with 360 to 408). Otherwise, of 1,024 / 2,048 / 4,096 keys the largest chunk within a
    twentieth of the most even filling of the rounds is taken (a count like 1,024 blocks, 1.4 rounds, was the
    slowest choice wherever it was measured). Measured on B200, 32 query heads on 8 kv heads of 64, microseconds
    a layer at chunks of 1,024 / 2,048 / 4,096 keys: 64 requests at 8 k keys 173 / 168 / 196, 16 at 32 k
    179 / 171 / 194, 8 at 65 k 188 / 175 / 200, 32 at 65 k 654 / 636 / 631, 8 at 130 k 360 / 337 / 326."""
    bucket = context_bucket
    if window:
        bucket = min(bucket, 1 << max(8, (window - 1).bit_length()))
    longest = max_context if not window else min(max_context, 2 * window)
    cap_splits = max(32, -(-longest // 1024) * 2)
    blocks_wanted = 224
    items = max(1, tokens * kv_heads)
    splits = max(1, min(bucket // 128, -(-blocks_wanted // items), cap_splits))
    chunk = min(-(-bucket // splits), 1024)
    chunk = (chunk + 63) // 64 * 64
    if chunk == 1024:
        if items * -(-bucket // 4096) < resident_blocks:
            # one round holds the launch: about half a round of blocks, in chunks of 1,024 to 4,096 keys
            splits = max(1, resident_blocks // 2 // items)
            chunk = min(max((-(-bucket // splits) + 63) // 64 * 64, 1024), 4096)
        else:
            def evenness(candidate: int) -> float:
                blocks = items * -(-bucket // candidate)
                rounds = -(-blocks // resident_blocks)
                return blocks / (rounds * resident_blocks)
            candidates = (1024, 2048, 4096)
            best = max(evenness(c) for c in candidates)
            chunk = max(c for c in candidates if evenness(c) >= best - 0.05)
    max_splits = -(-bucket // chunk)
    if max_splits > cap_splits:             # a bucket beyond the longest context: cannot come from a valid step
        raise ValueError(f"a context bucket of {context_bucket} keys needs {max_splits} splits, the scratch holds "
                         f"{cap_splits} (longest context {max_context})")
    return chunk, max_splits, cap_splits


class PagedAttentionKernels:
    """The choice among the attention kernels for a step's queries over a paged cache, shared by the mixers that
    attend over one. A mixer that inherits it has ``rt``, ``heads``, ``kv_heads``, ``head_dim``, ``window``, ``scale``,
    ``sinks`` (or None), ``distance_bias`` (absent, None, or a float32 table [heads, n + 1] of score biases by distance
    back to the key), ``binding``, the queries in ``qkv`` (head h of a row at h * head_dim, rows ``qkv_width``
    apart), the output buffer ``attended`` [tokens, heads * head_dim] and ``_resident_blocks = None``.
    ``_value_cache()`` names the tensor the values are read from: the binding's own, or the keys themselves for a
    mixer whose values are a leading part of what it caches as keys."""

    def _value_cache(self) -> torch.Tensor:
        return self.binding.v

    def _mask(self) -> Optional[int]:
        """What the tensor-core kernels get as ``window``: the window, or for a mixer with a chunked mask
        (``chunk`` positions a chunk) minus the chunk's size, which they read as "the keys of the query's own
        chunk"."""
        chunk = getattr(self, "chunk", None)
        return -int(chunk) if chunk else self.window

    def _decode_split(self, step: StepContext, tokens: Optional[int] = None):
        """One query token per request: how the keys are split so that few requests still fill the GPU,
        and the scratch of the split (chunk, max_splits, partial outputs, maxima and sums, counters)."""
        rt = self.rt
        if self._resident_blocks is None:
            self._resident_blocks = kernels.attention_decode_resident_blocks(self.head_dim) or DECODE_RESIDENT_BLOCKS
        # (a chunked mask shows a query at most a chunk's keys, as a window of that size would)
        chunk, max_splits, cap_splits = decode_split(tokens or step.tokens, self.kv_heads, step.context_bucket,
                                                     getattr(self, "chunk", None) or self.window, rt.max_context,
                                                     self._resident_blocks)
        rows = rt.max_requests * self.heads * cap_splits
        partial_o = rt.flat_scratch("attention.partial_o", rows * self.head_dim, torch.float32)
        partial_ml = rt.flat_scratch("attention.partial_ml", rows * 2, torch.float32)
        counters = rt.flat_scratch("attention.counters", rt.max_requests * self.kv_heads, torch.int32, zero=True)
        return chunk, max_splits, partial_o, partial_ml, counters

    def _decodes(self, step: StepContext) -> bool:
        """Whether the step goes to the split-key decode kernel (one query token per request)."""
        rt = self.rt
        return (step.max_span == 1 and step.tokens <= rt.max_requests and
                kernels.attention_decode_supported(self.heads, self.kv_heads, self.head_dim, rt.act_dtype))

    def attend(self, step: StepContext, table: torch.Tensor) -> None:
        """Attention of the step's queries (normalised, rotated, in ``self.qkv``) over the cache, which holds the
        step's own keys and values already. A step that is all single tokens goes to the split-key decode
        kernel. A step that begins with single-token spans and goes on with prompt portions (the order the
        scheduler plans: decoding requests first) is served by both: the decode kernel shares a request's keys
        among the query heads of a group and splits long contexts, where a prompt kernel would walk the whole
        context once per query head for one row of a 128-row tile."""
        rt = self.rt
        if self._values_differ():
            self._attend_general(step, table, 0)
            return
        if self._decodes(step):
            self._attend_single_tokens(step, table, step.tokens)
            return
        single = step.leading_single_tokens
        if (0 < single < step.tokens and single <= rt.max_requests and step.host_span_lengths is not None
                and kernels.attention_decode_supported(self.heads, self.kv_heads, self.head_dim, rt.act_dtype)):
            self._attend_single_tokens(step, table, single)
            self._attend_portions(step, table, single)
            return
        self._attend_portions(step, table, 0)

    def _attend_single_tokens(self, step: StepContext, table: torch.Tensor, count: int) -> None:
        """The first ``count`` tokens of the step, each the only token of its span."""
        b = self.binding
        chunk, max_splits, partial_o, partial_ml, counters = self._decode_split(step, count)
        kernels.attention_decode(self.qkv, self.qkv_width, self.attended, b.k, self._value_cache(), step.positions,
                                 step.token_span, table, count, self.heads, self.kv_heads,
                                 self.head_dim, b.page_tokens, self._mask(), self.scale, chunk, max_splits,
                                 partial_o, partial_ml, counters, step.error_flag, sinks=self.sinks,
                                 distance_bias=getattr(self, "distance_bias", None))

    def _attend_portions(self, step: StepContext, table: torch.Tensor, skip: int) -> None:
        """The spans from ``skip`` on (the spans before it have one token each, so span ``skip`` begins at token
        ``skip``). The kernels take token indices from ``span_begin`` and table rows by span, so a later part of
        both arrays addresses the same buffers."""
        b = self.binding
        rt = self.rt
        values = self._value_cache()
        spans = step.spans - skip
        span_begin = step.span_begin[skip:]
        span_table = table[skip:]
        lengths = step.host_span_lengths[skip:] if step.host_span_lengths is not None else None
        if (lengths is not None and rt.tcgen05_attention and kernels.attention_prefill_tcgen05_supported(
                self.heads, self.kv_heads, self.head_dim, b.page_tokens, rt.act_dtype)):
            # head size 64: S and O' in tensor memory, Q/K/V by TMA
            tiles = step.prompt_tile_bound or sum((length + 127) // 128 for length in lengths)
            kernels.attention_prefill_tcgen05(self.qkv, self.qkv_width, self.attended, b.k, values, step.positions,
                                              span_begin, span_table, step.tokens, spans, tiles, self.heads,
                                              self.kv_heads, self.head_dim, b.page_tokens, self._mask(), self.scale,
                                              step.error_flag, sinks=self.sinks,
                                              distance_bias=getattr(self, "distance_bias", None))
            return
        if kernels.attention_prefill_supported(self.heads, self.kv_heads, self.head_dim, rt.act_dtype):
            kernels.attention_prefill(self.qkv, self.qkv_width, self.attended, b.k, values, step.positions,
                                      span_begin, span_table, step.tokens, spans, self.heads, self.kv_heads,
                                      self.head_dim, b.page_tokens, self._mask(), self.scale, step.error_flag,
                                      sinks=self.sinks, distance_bias=getattr(self, "distance_bias", None))
            return
        self._attend_general(step, table, skip)

    def _values_differ(self) -> bool:
        """Values of another size than the keys: only the general kernel reads those."""
        return getattr(self, "value_dim", None) not in (None, self.head_dim)

    def _attend_general(self, step: StepContext, table: torch.Tensor, skip: int) -> None:
        """The tokens from ``skip`` on through the general kernel: a warp a (token, query head), any sizes, a window
        or a chunked mask (``chunk``), values of their own size (``value_dim``)."""
        b = self.binding
        kernels.attention_generic(self.qkv[skip:], self.qkv_width, self.attended[skip:], b.k, self._value_cache(),
                                  step.positions[skip:], step.token_span[skip:], table, step.tokens - skip,
                                  self.heads, self.kv_heads, self.head_dim, b.page_tokens, self.window, self.scale,
                                  step.error_flag, sinks=self.sinks, value_dim=getattr(self, "value_dim", None),
                                  chunk=getattr(self, "chunk", None), distance_bias=getattr(self, "distance_bias", None))


@register_part("mixer", "attention")
class AttentionMixer(PagedAttentionKernels):
    """Causal grouped-query attention over the paged cache with optional per-head q/k RMSNorm (or one over
    the whole projection: ``whole_qk_norm``), a position encoding, an optional window, an optional sink per
    query head, values that are the unrotated keys (``values_are_keys``: no value projection), and softmax
    scale given by the configuration.
    Order of operations as in celeg (src/backend/cpu/operators/attention_token.cpp:151-204;
    src/backend/cuda/packed/operators.cu:66-99, 101-246, 494-529): fused q|k|v projection,
    norm, rotation, cache write, attention, output projection."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window = params.get("window")
        self.scale = float(params.get("softmax_scale", self.head_dim ** -0.5))
        self.eps = float(params.get("qk_norm_eps", 1e-6))
        self.reads_only = bool(params.get("reads_cache_only", False))
        # q and k normalised over the whole projection (weights as wide as the projections) instead of per head
        self.whole_qk_norm = bool(params.get("whole_qk_norm", False))
        # no value projection: a key as projected (before norm and rotation) is its own value
        self.values_are_keys = bool(params.get("values_are_keys", False))
        if (self.whole_qk_norm or self.values_are_keys) and self.reads_only:
            raise ValueError("whole_qk_norm and values_are_keys are for mixers that own their cache")
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are not a multiple of {self.kv_heads} kv heads")
        self.position = parts.get("position")
        q_width = self.heads * self.head_dim
        kv_width = self.kv_heads * self.head_dim
        if self.reads_only:
            self.stored_kv_heads = 0
            fused = weights["q_proj"]
        elif self.values_are_keys:
            self.stored_kv_heads = self.kv_heads
            fused = torch.cat([weights["q_proj"], weights["k_proj"]], dim=0)
        else:
            self.stored_kv_heads = self.kv_heads
            fused = torch.cat([weights["q_proj"], weights["k_proj"], weights["v_proj"]], dim=0)
        self.qkv_width = q_width + (1 if self.values_are_keys else 2) * self.stored_kv_heads * self.head_dim
        self.w_qkv = rt.matrix(fused)
        self.w_out = rt.matrix(weights["out_proj"])
        self.q_norm = rt.vector(weights["q_norm"]) if "q_norm" in weights else None
        self.k_norm = rt.vector(weights["k_norm"]) if "k_norm" in weights else None
        # a learned score per query head that enters the softmax's denominator once: no key, no value, not scaled
        self.sinks = rt.vector(weights["sinks"]) if "sinks" in weights else None
        if self.sinks is not None and self.sinks.shape != (self.heads,):
            raise ValueError(f"attention sinks have shape {tuple(self.sinks.shape)}, expected ({self.heads},)")
        if self.values_are_keys and not self.whole_qk_norm and (self.q_norm is not None or self.k_norm is not None):
            raise ValueError("values_are_keys with per-head q/k norms is not built; use whole_qk_norm or no norms")
        self.row_scales = (rt.flat_scratch("attention.row_scales", 2 * rt.max_tokens, torch.float32)
                           if self.whole_qk_norm or self.values_are_keys else None)
        self.binding: Optional[PagedBinding] = None
        self._resident_blocks: Optional[int] = None      # (asked of the kernel library at the first decode step)
        self.qkv = rt.scratch("attention.qkv", self.qkv_width)
        self.attended = rt.scratch("attention.out", q_width)
        assert kv_width >= 0

    def cache_need(self):
        return PagedNeed(kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def bind_cache(self, binding: PagedBinding) -> None:
        if binding.owner and self.reads_only:
            raise ValueError("an attention mixer without k/v projections cannot own a cache")
        self.binding = binding

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def takes_split_norm(self, step: StepContext) -> bool:
        return self.rt.takes_split_norm(step.tokens, self.w_qkv)

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, b, t = self.rt, self.binding, step.tokens
        rt.linear(x, self.w_qkv, self.qkv, t)
        table = step.block_tables[b.group]
        fused = self.position.fused() if self.position is not None else {"inv_freq": None, "rotary_dim": 0}
        store = b.owner and not self.reads_only
        if self.whole_qk_norm or self.values_are_keys:
            if fused is None or not store:
                raise ValueError("whole_qk_norm / values_are_keys need a position part with fused() tables and a "
                                 "cache of the mixer's own")
            kernels.qk_whole_norm_rope_store(self.qkv, self.q_norm, self.k_norm, fused["inv_freq"], step.positions,
                                             step.token_span, table, b.k, b.v, t, self.heads, self.kv_heads,
                                             self.head_dim, fused["rotary_dim"], b.page_tokens, self.eps,
                                             self.values_are_keys, self.row_scales, step.error_flag)
            self.attend(step, table)
            rt.linear(self.attended, self.w_out, out, t)
            return
        if (fused is not None and store and rt.fuse_decode_qk and self.sinks is None and self._decodes(step)):
            # one token per request: norm, rotation and cache write happen inside the attention kernel
            chunk, max_splits, partial_o, partial_ml, counters = self._decode_split(step)
            kernels.attention_decode_fused(self.qkv, self.qkv_width, self.attended, b.k, b.v, step.positions,
                                           step.token_span, table, t, self.heads, self.kv_heads, self.head_dim,
                                           b.page_tokens, self.window, self.scale, chunk, max_splits, partial_o,
                                           partial_ml, counters, step.error_flag, self.q_norm, self.k_norm,
                                           fused["inv_freq"], fused["rotary_dim"], self.eps)
            rt.linear(self.attended, self.w_out, out, t)
            return
        if fused is not None:
            kernels.qk_norm_rope_store(self.qkv, self.q_norm, self.k_norm, fused["inv_freq"], step.positions,
                                       step.token_span, table, b.k, b.v, t, self.heads, self.stored_kv_heads,
                                       self.head_dim, fused["rotary_dim"], b.page_tokens, self.eps, store,
                                       step.error_flag)
        else:
            # unfused: normalise in place, let the position part rewrite q and k, then store
            kernels.qk_norm_rope_store(self.qkv, self.q_norm, self.k_norm, None, step.positions, step.token_span,
                                       table, b.k, b.v, t, self.heads, self.stored_kv_heads, self.head_dim, 0,
                                       b.page_tokens, self.eps, 2 if self.stored_kv_heads else 0, step.error_flag)
            rows = self.qkv[:t]
            q_width = self.heads * self.head_dim
            kv_width = self.stored_kv_heads * self.head_dim
            q_view = rows[:, :q_width].unflatten(1, (self.heads, self.head_dim))
            k_view = rows[:, q_width:q_width + kv_width].unflatten(1, (self.stored_kv_heads, self.head_dim))
            self.position.apply(q_view, k_view, step.positions[:t], t)
            if store:
                kernels.qk_norm_rope_store(self.qkv, None, None, None, step.positions, step.token_span, table,
                                           b.k, b.v, t, self.heads, self.stored_kv_heads, self.head_dim, 0,
                                           b.page_tokens, self.eps, True, step.error_flag)
        self.attend(step, table)
        rt.linear(self.attended, self.w_out, out, t)


def distance_bucket(distance: int, buckets: int, far: float) -> int:
    """The row of a table of ``buckets`` learned score biases that stands for a key ``distance`` positions back: the
    first buckets // 2 rows stand for one distance each, the others divide the distances from buckets // 2 up to
    ``far`` evenly in the logarithm, the last row takes everything farther (the bucketing of relative positions in
    Raffel et al., "Exploring the Limits of Transfer Learning with a Unified Text-to-Text Transformer", 2020, for one
    direction)."""
    exact = buckets // 2
    if distance < exact:
        return distance
    stretched = exact + int(math.floor(math.log(distance / exact) / math.log(far / exact) * (buckets - exact)))
    return min(buckets - 1, stretched)


def distance_bias_table(table: torch.Tensor, far: int) -> torch.Tensor:
    """A stored table [buckets, heads] as the attention kernels read it: float32 [heads, far + 1], entry [h, n] the bias
    of a key n positions back (``far`` and everything farther share the last entry, whose bucket is the last)."""
    buckets = int(table.shape[0])
    if buckets < 2 or far <= buckets // 2:
        raise ValueError(f"a distance table of {buckets} rows up to distance {far}: needs 2 rows or more and a "
                         f"farthest distance beyond {buckets // 2}")
    rows = torch.tensor([distance_bucket(n, buckets, float(far)) for n in range(far + 1)], dtype=torch.long)
    return table.to(torch.float32)[rows].t().contiguous()


@register_part("mixer", "prepared_attention")
class PreparedAttentionMixer(PagedAttentionKernels):
    """Causal grouped-query softmax attention whose q, k and v leave one fused projection as float32 sums and are
    made ready for the paged attention kernels by one launch. Everything but the four matrices is optional:

    * biases on the projections (tensors ``q_bias``, ``k_bias``, ``v_bias``, ``out_bias``);
    * ``whole_qk_norm``: one RMS norm over the whole q projection and one over the whole k projection (tensors
      ``q_norm``, ``k_norm`` as wide as the projections, ``eps``);
    * a nested part ``position`` that rotates pairs (i, i + half) of the heads' leading dimensions;
    * ``temperature`` = {coef, every}: q times 1 + coef ln(floor((position + 1) / every) + 1);
    * ``distance_far`` with the tensor ``distance_table`` [buckets, heads]: a learned number per head and distance
      bucket (:func:`distance_bucket`) added to the scaled scores;
    * ``value_mix``: "first" notes the layer's values of the step's tokens for later layers, "blend" replaces v by
      (1 - lam) v + lam v_first with lam the stored number ``value_mix`` (what is cached is the blended v);
    * ``output_gate``: the heads' results times sigmoid(W_g h), element by element (tensor ``gate``);
    * values of a size ``vdim`` of their own, a softmax scale given by the configuration, a sink per head (tensor
      ``sinks``), and a mask: ``window`` = w lets a query at position i read key j when 0 <= i - j < w, ``chunk`` = c
      when floor(i / c) = floor(j / c) (chunks counted from position 0 of the sequence, so the mask does not depend
      on how a prompt was cut into steps). Query head h reads key/value head h // (heads / kv_heads).

    On the bfloat16 path, when keys and values differ in size and the tensor-core kernels take the larger size, both
    are stored at that size (the tails zero: a zero adds nothing to a score, and a zero value column gives a zero
    result column, which meets zero columns of the output projection); otherwise heads are stored as they are and
    the general kernel reads values of their own size."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.kv_heads = int(params.get("kv_heads") or self.heads)
        self.dim = int(params["dim"])
        self.vdim = int(params.get("vdim") or self.dim)
        self.scale = float(params.get("scale", self.dim ** -0.5))
        chunk = params.get("chunk")
        self.chunk = int(chunk) if chunk else None
        if self.chunk is not None and self.chunk < 1:
            raise ValueError(f"attention: a chunk of {self.chunk} positions")
        window = params.get("window")
        self.window = int(window) if window else None
        if self.window is not None and (self.window < 1 or self.chunk is not None):
            raise ValueError(f"attention: a window of {self.window} positions (beside a chunk: {self.chunk})")
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are not a multiple of {self.kv_heads} kv heads")
        self.sinks = rt.vector(weights["sinks"]) if "sinks" in weights else None
        if self.sinks is not None and self.sinks.shape != (self.heads,):
            raise ValueError(f"attention sinks have shape {tuple(self.sinks.shape)}, expected ({self.heads},)")
        self.output_gate = bool(params.get("output_gate", False))
        # sizes of a stored head: what the kernels see as head size (keys, queries) and value size
        self.head_dim = self.value_dim = None
        larger = max(self.dim, self.vdim)
        if self.dim == self.vdim or (rt.act_dtype == torch.bfloat16 and not self.output_gate
                                     and self._fast_kernels_take(larger)):
            self.head_dim = self.value_dim = larger
        else:
            self.head_dim, self.value_dim = self.dim, self.vdim
        q_width, k_width, v_width = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.q_width, self.k_width, self.v_width = q_width, k_width, v_width
        stacked = [weights["q"], weights["k"], weights["v"]]
        if self.output_gate:
            stacked.append(weights["gate"])
        self.w_qkv = rt.matrix(torch.cat(stacked, dim=0))
        self.gate_width = self.heads * self.vdim if self.output_gate else 0
        biases = [weights.get("q_bias"), weights.get("k_bias"), weights.get("v_bias")]
        if any(b is not None for b in biases):
            widths = (q_width, k_width, v_width)
            self.bias = rt.vector(torch.cat([b.float() if b is not None else torch.zeros(w) for b, w in zip(biases, widths)]))
        else:
            self.bias = None
        # what the plain store (biases only) cannot do goes through the general preparation
        self.whole_qk_norm = bool(params.get("whole_qk_norm", False))
        self.eps = float(params.get("eps", 1e-6))
        self.q_norm = self.k_norm = None
        if self.whole_qk_norm:
            self.q_norm, self.k_norm = rt.vector(weights["q_norm"]), rt.vector(weights["k_norm"])
            if self.q_norm.shape != (q_width,) or self.k_norm.shape != (k_width,):
                raise ValueError(f"whole-projection norm weights of shapes {tuple(self.q_norm.shape)} / "
                                 f"{tuple(self.k_norm.shape)}, expected ({q_width},) / ({k_width},)")
        position = parts.get("position")
        fused = position.fused() if position is not None else None
        self.frequencies, self.rotary_dim = None, 0
        if fused is not None and fused.get("rotary_dim"):
            if fused.get("interleaved") or fused["rotary_dim"] > self.dim:
                raise ValueError("attention: the position part must rotate pairs (i, i + half) of at most dim dimensions")
            self.frequencies, self.rotary_dim = fused["inv_freq"], int(fused["rotary_dim"])
        elif position is not None and fused is None:
            raise ValueError("attention: the position part must offer fused() tables")
        temperature = params.get("temperature")
        self.temperature = (float(temperature["coef"]), int(temperature["every"])) if temperature else None
        if self.temperature is not None and self.temperature[1] < 1:
            raise ValueError(f"attention: a query temperature every {self.temperature[1]} positions")
        self.distance_bias = None
        if "distance_table" in weights:
            table = weights["distance_table"]
            if table.dim() != 2 or table.shape[1] != self.heads:
                raise ValueError(f"a distance table of shape {tuple(table.shape)}, expected (buckets, {self.heads})")
            self.distance_bias = rt.vector(distance_bias_table(table, int(params["distance_far"])))
        mix = params.get("value_mix")
        if mix not in (None, "first", "blend"):
            raise ValueError(f"attention: value_mix {mix!r}; known: first, blend")
        self.blend = {None: 0, "first": 1, "blend": 2}[mix]
        self.lam = float(weights["value_mix"].to(torch.float32).reshape(-1)[0]) if self.blend == 2 else 0.0
        # the first marked layer's values of the step's tokens: float32 rows that every marked layer of a model shares
        self.first_values = rt.scratch("attention.first_values", v_width, torch.float32) if self.blend else None
        self.prepares = bool(self.whole_qk_norm or self.frequencies is not None or self.temperature or self.blend)
        w_out = weights["out"]
        if self.value_dim != self.vdim:          # zero columns where the attention's result has its zero tail
            padded = torch.zeros((w_out.shape[0], self.heads, self.value_dim), dtype=w_out.dtype)
            padded[:, :, :self.vdim] = w_out.reshape(w_out.shape[0], self.heads, self.vdim)
            w_out = padded.reshape(w_out.shape[0], self.heads * self.value_dim)
        self.w_out = rt.matrix(w_out)
        self.out_bias = rt.vector(weights["out_bias"]) if "out_bias" in weights else None
        self.ends_with_product = self.out_bias is None       # forward() then writes `out` last, with rt.linear
        self.binding: Optional[PagedBinding] = None
        self._resident_blocks: Optional[int] = None
        self.projected = rt.scratch("prepared_attention.proj", q_width + k_width + v_width + self.gate_width, torch.float32)
        self.qkv_width = self.heads * self.head_dim
        self.qkv = rt.scratch("prepared_attention.q", self.qkv_width)
        self.attended = rt.scratch("prepared_attention.out", self.heads * self.value_dim)
        self.unbiased = rt.scratch("prepared_attention.unbiased", self.hidden, torch.float32) if self.out_bias is not None else None

    def _fast_kernels_take(self, size: int) -> bool:
        return (kernels.attention_prefill_supported(self.heads, self.kv_heads, size, torch.bfloat16)
                and kernels.attention_decode_supported(self.heads, self.kv_heads, size, torch.bfloat16))

    def cache_need(self):
        return PagedNeed(kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window,
                         value_head_dim=None if self.value_dim == self.head_dim else self.value_dim)

    def bind_cache(self, binding: PagedBinding) -> None:
        if not binding.owner:
            raise ValueError("this attention writes its keys and values: it cannot read another position's cache")
        self.binding = binding

    def _attend(self, x: torch.Tensor, step: StepContext) -> None:
        rt, b, t = self.rt, self.binding, step.tokens
        rt.linear(x, self.w_qkv, self.projected, t)
        table = step.block_tables[b.group]
        if self.prepares:
            kernels.qkv_prepare(self.projected, self.bias, self.qkv, step.positions, step.token_span, table, b.k, b.v, t,
                                self.heads, self.kv_heads, self.dim, self.vdim, self.head_dim, self.value_dim,
                                b.page_tokens, step.error_flag, q_norm=self.q_norm, k_norm=self.k_norm,
                                norm_eps=self.eps, frequencies=self.frequencies, rotary_dim=self.rotary_dim,
                                temperature=self.temperature, blend=self.blend, lam=self.lam,
                                first_values=self.first_values)
        else:
            kernels.bias_store_kv(self.projected, self.bias, self.qkv, step.positions, step.token_span, table, b.k, b.v,
                                  t, self.heads, self.kv_heads, self.dim, self.vdim, self.head_dim, self.value_dim,
                                  b.page_tokens, step.error_flag)
        self.attend(step, table)
        if self.output_gate:
            kernels.sigmoid_gate(self.attended, self.projected[:, self.q_width + self.k_width + self.v_width:], t,
                                 self.gate_width)

    def forward_without_bias(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> Optional[torch.Tensor]:
        """forward() into a float32 ``out`` without the output projection's bias, which is returned (or None) for a
        caller that adds it in a pass of its own."""
        self._attend(x, step)
        self.rt.linear(self.attended, self.w_out, out, step.tokens)
        return self.out_bias

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        if self.out_bias is None:
            self._attend(x, step)
            self.rt.linear(self.attended, self.w_out, out, step.tokens)
            return
        self.forward_without_bias(x, self.unbiased, step)
        kernels.scaled_sum(self.unbiased, None, self.out_bias, 1.0, 0.0, out, step.tokens)


@register_part("mixer", "chunked_attention")
class ChunkedAttentionMixer(PreparedAttentionMixer):
    """The prepared attention as a design names it that uses it for its chunked mask: no position encoding, biases on
    the four projections, values of a size of their own, ``chunk`` positions a chunk."""


@register_part("mixer", "side_by_side")
class SideBySideMixer:
    """Two mixers (nested parts ``left`` and ``right``) that read the same rows; the result is
    left_scale * left + right_scale * right. Each child leaves its result as float32 rows (its last product's sums);
    one launch scales, adds (a child's output bias too, if it hands one over) and rounds once. A child that holds
    a cache gets its own: the children are named to the model under ``children``."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.left_scale = float(params.get("left_scale", 1.0))
        self.right_scale = float(params.get("right_scale", 1.0))
        if parts.get("left") is None or parts.get("right") is None:
            raise ValueError("side_by_side: needs the nested mixers 'left' and 'right'")
        self.left, self.right = parts["left"], parts["right"]
        self.children = {"left": self.left, "right": self.right}
        self.left_out = rt.scratch("side_by_side.left", self.hidden, torch.float32)
        self.right_out = rt.scratch("side_by_side.right", self.hidden, torch.float32)

    @staticmethod
    def _run(child, x, out, step):
        without = getattr(child, "forward_without_bias", None)
        if without is not None:
            return without(x, out, step)
        child.forward(x, out, step)
        return None

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        left_bias = self._run(self.left, x, self.left_out, step)
        right_bias = self._run(self.right, x, self.right_out, step)
        if right_bias is not None and left_bias is None:
            kernels.scaled_sum(self.right_out, self.left_out, right_bias, self.right_scale, self.left_scale, out, step.tokens)
            return
        if right_bias is not None:
            kernels.scaled_sum(self.right_out, None, right_bias, 1.0, 0.0, self.right_out, step.tokens)
        kernels.scaled_sum(self.left_out, self.right_out, left_bias, self.left_scale, self.right_scale, out, step.tokens)


@register_part("mixer", "short_conv")
class ShortConvMixer:
    """Gated short convolution: [B|C|X] = in_proj(x); conv over B*X with a depthwise causal
    kernel of ``taps`` taps; out_proj(C * conv). Per-request state: the last taps-1 values of
    B*X per channel, float32 (celeg src/backend/cpu/kernels/convolution.cpp:7-28;
    src/backend/cuda/packed/operators.cu:31-62)."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.taps = int(params["taps"])
        self.w_in = rt.matrix(weights["in_proj"])
        self.w_out = rt.matrix(weights["out_proj"])
        self.kernel = rt.vector(weights["conv"].reshape(self.hidden, self.taps))
        self.binding: Optional[StateBinding] = None
        self.projected = rt.scratch("short_conv.proj", 3 * self.hidden)
        self.gated = rt.scratch("short_conv.out", self.hidden)

    def cache_need(self):
        return StateNeed(elements=(self.taps - 1) * self.hidden)

    def bind_cache(self, binding: StateBinding) -> None:
        self.binding = binding

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def takes_split_norm(self, step: StepContext) -> bool:
        return self.rt.takes_split_norm(step.tokens, self.w_in)

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t = self.rt, step.tokens
        if not rt.linear_short_conv(x, self.w_in, self.kernel, self.taps, self.binding, self.gated, step):
            rt.linear(x, self.w_in, self.projected, t)
            kernels.short_conv(self.projected, self.kernel, self.binding.state, self.binding.slot_stride,
                               self.gated, step.token_span, step.span_begin, step.span_slot, t, step.spans,
                               self.hidden, self.taps, step.max_span)
        rt.linear(self.gated, self.w_out, out, t)
