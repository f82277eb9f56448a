"""Mixers whose cache is a matrix per head that every token rewrites (kernels: csrc/recurrent_scan.cu).
The state is float32 on both precision paths and lives in the request's state slot; gates, unit norms,
decays and every sum of the recurrence are float32; the projections run in the path's matrix type and leave
float32 results.

    mlstm         S' = a S + b k v^T, n' = a n + b k with exponential gates kept in range by a running maximum;
                  read-out S'^T q over max(|n'.q|, exp(-m')) (Beck et al., "xLSTM: Extended Long Short-Term
                  Memory", 2024, the matrix-memory cell)
    gated_delta   S' = g S + k (beta (v - (g S)^T k))^T, read-out S'^T q, after short causal convolutions with
                  SiLU on q, k, v and unit-length q, k (Yang, Kautz, Hatamizadeh, "Gated Delta Networks:
                  Improving Mamba2 with Delta Rule", 2024)
    retention     S' = d S + k v^T with a constant decay d per head, read-out S'^T q, no softmax and no denominator
                  (Sun et al., "Retentive Network: A Successor to Transformer for Large Language Models", 2023)
    lightning_attention   the same recurrence with SiLU on q, k and v and no factor on the keys; the heads' read-outs
                  are normalised together, as one vector, and gated by a sigmoid
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from .. import kernels
from ..cache.manager import StateNeed
from .mixers import StateBinding
from .registry import register_part
from .runtime import Runtime, StepContext


@register_part("mixer", "mlstm")
class MlstmMixer:
    """q = W_q x / sqrt(dim), k = W_k x (heads x dim), v = W_v x (heads x vdim); per head a log input gate
    cap tanh((W_i x + b_i) / cap) and a log forget gate logsigmoid(cap tanh((W_f x + b_f) / cap)). Each head's
    read-out is divided by its root mean square, scaled by ``norm`` (all heads' width), gated by sigmoid(W_g x)
    and projected by W_o. The running maximum of a new request is 0."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.cap = float(params["gate_cap"])
        self.eps = float(params["eps"])
        if self.dim > kernels.SCAN_MAX_DIM:
            raise ValueError(f"mlstm: a key size of {self.dim} exceeds {kernels.SCAN_MAX_DIM}")
        self.qk_width = self.heads * self.dim
        self.v_width = self.heads * self.vdim
        fused = torch.cat([weights["q"], weights["k"], weights["v"], weights["gate"], weights["input_gate"],
                           weights["forget_gate"]], dim=0)
        self.w_in = rt.matrix(fused)
        self.w_out = rt.matrix(weights["out"])
        self.bias_i = rt.vector(weights["input_gate_bias"])
        self.bias_f = rt.vector(weights["forget_gate_bias"])
        self.norm = rt.vector(weights["norm"])
        self.proj_width = int(fused.shape[0])
        self.binding: Optional[StateBinding] = None
        self.projected = rt.scratch("recurrent.proj", self.proj_width, torch.float32)
        self.gates = rt.scratch("recurrent.gates", 2 * self.heads, torch.float32)
        self.read = rt.scratch("recurrent.read", self.v_width, torch.float32)
        self.gated = rt.scratch("recurrent.gated", self.v_width)

    def cache_need(self):
        return StateNeed(elements=self.heads * self.dim * self.vdim + self.heads * self.dim + self.heads)

    def bind_cache(self, binding: StateBinding) -> None:
        self.binding = binding

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t, b = self.rt, step.tokens, self.binding
        rt.linear(x, self.w_in, self.projected, t)
        rows = self.projected
        at = 0
        q = rows[:, at:at + self.qk_width]; at += self.qk_width
        k = rows[:, at:at + self.qk_width]; at += self.qk_width
        v = rows[:, at:at + self.v_width]; at += self.v_width
        gate = rows[:, at:at + self.v_width]; at += self.v_width
        pre_i = rows[:, at:at + self.heads]; at += self.heads
        pre_f = rows[:, at:at + self.heads]
        if step.max_span == 1 and step.spans == t:
            # every request brings one token: gates, state update, read-out, norm and output gate in one launch
            width = self.qk_width
            offsets = (0, width, 2 * width, 2 * width + self.v_width, 2 * width + 2 * self.v_width,
                       2 * width + 2 * self.v_width + self.heads)
            kernels.recurrent_decode(kernels.SCAN_MLSTM, rows, offsets, None, None, 0, 0, self.bias_i, self.bias_f,
                                     self.cap, self.norm, True, self.eps, 0.0, b.state, b.slot_stride, step.span_begin,
                                     step.span_slot, t, self.heads, self.heads, self.dim, self.vdim, self.dim ** -0.5,
                                     self.gated)
            rt.linear(self.gated, self.w_out, out, t)
            return
        kernels.mlstm_gates(pre_i, pre_f, self.bias_i, self.bias_f, self.cap, self.gates, t, self.heads)
        kernels.recurrent_scan(kernels.SCAN_MLSTM, q, k, v, self.gates, self.read, b.state, b.slot_stride,
                               step.span_begin, step.span_slot, step.spans, self.heads, self.heads, self.dim,
                               self.vdim, self.dim ** -0.5)
        kernels.gated_head_norm(self.read, gate, self.norm, True, self.gated, t, self.heads, self.vdim, self.eps,
                                kernels.GATE_SIGMOID)
        rt.linear(self.gated, self.w_out, out, t)


@register_part("mixer", "gated_delta")
class GatedDeltaMixer:
    """q = W_q x, k = W_k x (kv_heads x dim), v = W_v x (heads x vdim), each through a depthwise causal
    convolution of ``taps`` taps and SiLU; q and k per head divided by sqrt(sum of squares + 1e-6), q also by
    sqrt(dim); beta = sigmoid(W_b x) and decay g = exp(-exp(A_log) softplus(W_a x + dt_bias)) per head. Head h
    reads q/k head h // (heads / kv_heads). Each head's read-out is divided by its root mean square, scaled by
    ``norm`` (vdim, shared by the heads), gated by SiLU(W_g x) and projected by W_o. Per-request state: S per
    head, then the last taps - 1 inputs of the convolutions."""

    UNIT_EPS = 1e-6

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.kv_heads = int(params["kv_heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.taps = int(params["taps"])
        self.eps = float(params["eps"])
        if self.heads % self.kv_heads:
            raise ValueError(f"gated_delta: {self.heads} heads are not a multiple of {self.kv_heads} q/k heads")
        if self.dim > kernels.SCAN_MAX_DIM or not 1 <= self.taps <= 16:
            raise ValueError(f"gated_delta: key size {self.dim} (at most {kernels.SCAN_MAX_DIM}) or {self.taps} taps "
                             f"(1 to 16) is out of range")
        self.qk_width = self.kv_heads * self.dim
        self.v_width = self.heads * self.vdim
        self.channels = 2 * self.qk_width + self.v_width
        fused = torch.cat([weights["q"], weights["k"], weights["v"], weights["gate"], weights["beta"],
                           weights["decay"]], dim=0)
        self.w_in = rt.matrix(fused)
        self.w_out = rt.matrix(weights["out"])
        self.kernel = rt.vector(torch.cat([weights["q_conv"].reshape(self.qk_width, self.taps),
                                           weights["k_conv"].reshape(self.qk_width, self.taps),
                                           weights["v_conv"].reshape(self.v_width, self.taps)], dim=0))
        self.a_log = rt.vector(weights["a_log"])
        self.dt_bias = rt.vector(weights["dt_bias"])
        self.norm = rt.vector(weights["norm"])
        self.proj_width = int(fused.shape[0])
        self.state_elements = self.heads * self.dim * self.vdim
        self.binding: Optional[StateBinding] = None
        self.carried: Optional[torch.Tensor] = None
        self.projected = rt.scratch("recurrent.proj", self.proj_width, torch.float32)
        self.convolved = rt.scratch("recurrent.conv", self.channels, torch.float32)
        self.gates = rt.scratch("recurrent.gates", 2 * self.heads, torch.float32)
        self.read = rt.scratch("recurrent.read", self.v_width, torch.float32)
        self.gated = rt.scratch("recurrent.gated", self.v_width)

    def cache_need(self):
        return StateNeed(elements=self.state_elements + (self.taps - 1) * self.channels)

    def bind_cache(self, binding: StateBinding) -> None:
        self.binding = binding
        self.carried = binding.state[:, self.state_elements:]

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t, b = self.rt, step.tokens, self.binding
        rt.linear(x, self.w_in, self.projected, t)
        rows = self.projected
        at = self.channels
        gate = rows[:, at:at + self.v_width]; at += self.v_width
        pre_beta = rows[:, at:at + self.heads]; at += self.heads
        pre_a = rows[:, at:at + self.heads]
        if step.max_span == 1 and step.spans == t:
            # every request brings one token: convolutions, unit norms, gates, state update, read-out, norm and
            # output gate in one launch, the carried inputs in a second
            offsets = (0, self.qk_width, 2 * self.qk_width, self.channels, self.channels + self.v_width,
                       self.channels + self.v_width + self.heads)
            kernels.recurrent_decode(kernels.SCAN_DELTA, rows, offsets, self.kernel, self.carried, self.taps,
                                     self.channels, self.a_log, self.dt_bias, 0.0, self.norm, False, self.eps,
                                     self.UNIT_EPS, b.state, b.slot_stride, step.span_begin, step.span_slot, t,
                                     self.heads, self.kv_heads, self.dim, self.vdim, self.dim ** -0.5, self.gated)
            rt.linear(self.gated, self.w_out, out, t)
            return
        kernels.delta_prepare(rows, self.kernel, self.carried, b.slot_stride, step.token_span, step.span_begin,
                              step.span_slot, self.convolved, pre_beta, pre_a, self.a_log, self.dt_bias, self.gates,
                              t, step.spans, self.channels, self.taps, self.kv_heads, self.dim, self.heads,
                              self.UNIT_EPS)
        conv = self.convolved
        q = conv[:, :self.qk_width]
        k = conv[:, self.qk_width:2 * self.qk_width]
        v = conv[:, 2 * self.qk_width:]
        kernels.recurrent_scan(kernels.SCAN_DELTA, q, k, v, self.gates, self.read, b.state, b.slot_stride,
                               step.span_begin, step.span_slot, step.spans, self.heads, self.kv_heads, self.dim,
                               self.vdim, self.dim ** -0.5)
        kernels.gated_head_norm(self.read, gate, self.norm, False, self.gated, t, self.heads, self.vdim, self.eps,
                                kernels.GATE_SILU)
        rt.linear(self.gated, self.w_out, out, t)


@register_part("mixer", "retention")
class RetentionMixer:
    """q = W_q x, k = W_k x / sqrt(dim) (heads x dim), v = W_v x (heads x vdim); per head S <- decay_h S + k v^T
    and the read-out S^T q, with ``decay`` one constant a head. Each head's read-out is divided by its root mean
    square (no weight), the heads are gated by SiLU(W_g x) and projected by W_o. Per-request state: S per head,
    float32, zero for a new request."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.eps = float(params["eps"])
        decay = [float(d) for d in params["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"retention: {len(decay)} decays for {self.heads} heads")
        if self.dim > kernels.SCAN_MAX_DIM:
            raise ValueError(f"retention: a key size of {self.dim} exceeds {kernels.SCAN_MAX_DIM}")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=rt.device)
        self.qk_width = self.heads * self.dim
        self.v_width = self.heads * self.vdim
        fused = torch.cat([weights["q"], weights["k"], weights["v"], weights["gate"]], dim=0)
        self.w_in = rt.matrix(fused)
        self.w_out = rt.matrix(weights["out"])
        self.proj_width = int(fused.shape[0])
        self.binding: Optional[StateBinding] = None
        self.projected = rt.scratch("recurrent.proj", self.proj_width, torch.float32)
        self.read = rt.scratch("recurrent.read", self.v_width, torch.float32)
        self.gated = rt.scratch("recurrent.gated", self.v_width)
        # long prompts: segments of SEGMENT tokens scanned side by side (the decay is a constant, so a segment's
        # state and read-outs from a zero state are corrected afterwards by what was carried into it)
        self.max_segments = rt.max_tokens // self.SEGMENT + rt.max_requests + 16
        elements = self.heads * self.dim * self.vdim
        self.segment_states = rt.flat_scratch("retention.segments", 2 * self.max_segments * elements, torch.float32)
        self.segment_plan = rt.flat_scratch("retention.plan", 2 * self.max_segments + 8, torch.int32, zero=True)
        self.segment_numbers = torch.arange(self.max_segments, dtype=torch.int32, device=rt.device)

    SEGMENT = 128               # tokens a segment
    SEGMENTED_FROM = 384        # steps of at least this many tokens are scanned in segments

    def cache_need(self):
        return StateNeed(elements=self.heads * self.dim * self.vdim)

    def bind_cache(self, binding: StateBinding) -> None:
        self.binding = binding

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t, b = self.rt, step.tokens, self.binding
        rt.linear(x, self.w_in, self.projected, t)
        rows = self.projected
        width = self.qk_width
        if step.max_span == 1 and step.spans == t:
            # every request brings one token: state update, read-out, head norm and output gate in one launch
            offsets = (0, width, 2 * width, 2 * width + self.v_width, 0, 0)
            kernels.recurrent_decode(kernels.SCAN_RETENTION, rows, offsets, None, None, 0, 0, self.decay, self.decay,
                                     0.0, None, False, self.eps, 0.0, b.state, b.slot_stride, step.span_begin,
                                     step.span_slot, t, self.heads, self.heads, self.dim, self.vdim, self.dim ** -0.5,
                                     self.gated)
            rt.linear(self.gated, self.w_out, out, t)
            return
        q = rows[:, :width]
        k = rows[:, width:2 * width]
        v = rows[:, 2 * width:2 * width + self.v_width]
        gate = rows[:, 2 * width + self.v_width:]
        segments = t // self.SEGMENT + step.spans
        if t >= self.SEGMENTED_FROM and segments <= self.max_segments and segments + step.spans + 2 <= self.segment_plan.numel():
            kernels.retention_segmented(q, k, v, self.decay, self.read, b.state, b.slot_stride, step.span_begin,
                                        step.span_slot, step.spans, t, self.heads, self.dim, self.vdim, self.dim ** -0.5,
                                        self.SEGMENT, segments, self.segment_states, self.segment_plan, self.segment_numbers)
        else:
            kernels.recurrent_scan(kernels.SCAN_RETENTION, q, k, v, self.decay, self.read, b.state, b.slot_stride,
                                   step.span_begin, step.span_slot, step.spans, self.heads, self.heads, self.dim,
                                   self.vdim, self.dim ** -0.5)
        kernels.gated_head_norm(self.read, gate, None, False, self.gated, t, self.heads, self.vdim, self.eps,
                                kernels.GATE_SILU)
        rt.linear(self.gated, self.w_out, out, t)


@register_part("mixer", "lightning_attention")
class LightningAttentionMixer(RetentionMixer):
    """q = SiLU(W_q x), k = SiLU(W_k x) (heads x dim), v = SiLU(W_v x) (heads x vdim); per head S <- decay_h S + k v^T
    and the read-out S^T q, with ``decay`` one constant a head and no other factor. The heads' read-outs side by side
    are divided by their common root mean square (one over all heads), scaled by ``norm`` (all heads' width), gated by
    sigmoid(W_g x) and projected by W_o. Per-request state: S per head, float32, zero for a new request.

    The recurrence is the retention's: its scan, its segmented form for long portions and its decoding kernel are
    used with a key factor of 1. The activations are applied to the projection's float32 results (in place for
    portions, as the values are read when decoding), and because the norm runs over all heads, which no block of the
    decoding launch sees together, that launch leaves the raw read-outs and the norm and gate follow in one more."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        super().__init__(params, weights, parts, rt)
        self.norm = rt.vector(weights["norm"])
        if self.norm.shape != (self.v_width,):
            raise ValueError(f"lightning_attention: the norm's weight has shape {tuple(self.norm.shape)}, expected "
                             f"({self.v_width},)")

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t, b = self.rt, step.tokens, self.binding
        rt.linear(x, self.w_in, self.projected, t)
        rows = self.projected
        width = self.qk_width
        gate = rows[:, 2 * width + self.v_width:]
        if step.max_span == 1 and step.spans == t:
            kernels.retention_decode_raw(rows, (0, width, 2 * width), self.decay, b.state, b.slot_stride, step.span_slot,
                                         t, self.heads, self.dim, self.vdim, 1.0, kernels.ACT_SILU, self.read)
        else:
            kernels.activation_columns(rows, 2 * width + self.v_width, t, kernels.ACT_SILU)
            q = rows[:, :width]
            k = rows[:, width:2 * width]
            v = rows[:, 2 * width:2 * width + self.v_width]
            segments = t // self.SEGMENT + step.spans
            if (t >= self.SEGMENTED_FROM and segments <= self.max_segments
                    and segments + step.spans + 2 <= self.segment_plan.numel()):
                kernels.retention_segmented(q, k, v, self.decay, self.read, b.state, b.slot_stride, step.span_begin,
                                            step.span_slot, step.spans, t, self.heads, self.dim, self.vdim, 1.0,
                                            self.SEGMENT, segments, self.segment_states, self.segment_plan,
                                            self.segment_numbers)
            else:
                kernels.recurrent_scan(kernels.SCAN_RETENTION, q, k, v, self.decay, self.read, b.state, b.slot_stride,
                                       step.span_begin, step.span_slot, step.spans, self.heads, self.heads, self.dim,
                                       self.vdim, 1.0)
        # one norm over all heads: a single "head" as wide as all of them
        kernels.gated_head_norm(self.read, gate, self.norm, True, self.gated, t, 1, self.v_width, self.eps,
                                kernels.GATE_SIGMOID)
        rt.linear(self.gated, self.w_out, out, t)


@register_part("mixer", "gated_linear_recurrence")
class GatedLinearRecurrenceMixer:
    """The recurrent block of De et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient
    Language Models" (2024), with its real-gated linear recurrent unit. Two branches of ``width`` channels:
    y = gelu_tanh(W_y x + b_y) and u = conv(W_x x + b_x) + b_c, a causal convolution per channel over ``taps``
    inputs (the last tap meets the token itself, zeros before a sequence's start). The channels are cut into
    ``blocks`` equal parts; in part b, r = sigmoid(A_b u_b + a_b) and i = sigmoid(I_b u_b + i_b) with square matrices.
    Per channel a = exp(-gate_factor r softplus(lam)), S <- a S + sqrt(1 - a^2) i u from S = 0 (the first token is no
    special case), and the result is W_o (S y).

    Per-request state, float32, zero for a new request: the last taps - 1 inputs W_x x + b_x of the convolution
    (oldest first), then S. One fused [y | x] projection leaves float32 sums; everything between it and W_o is
    float32 on both precision paths (biases, activations, convolution, the gates' products as FFMA sums, decays,
    the recurrence), and S y is rounded once for W_o. Tensors: ``y``, ``x``, ``conv`` [width, taps],
    ``recurrence_gate`` and ``input_gate`` [blocks, width / blocks, width / blocks], ``lam`` [width], ``out``, and the
    optional biases ``y_bias``, ``x_bias``, ``conv_bias``, ``recurrence_gate_bias``, ``input_gate_bias``."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.width = int(params["width"])
        self.blocks = int(params["blocks"])
        self.taps = int(params["taps"])
        self.gate_factor = float(params.get("gate_factor", 8.0))
        if self.width % self.blocks:
            raise ValueError(f"gated_linear_recurrence: {self.width} channels are not a multiple of {self.blocks} blocks")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"gated_linear_recurrence: {self.taps} taps; 1 to 16 are built")
        part = self.width // self.blocks
        if 3 * part * 4 > 48 * 1024:
            raise ValueError(f"gated_linear_recurrence: a part of {part} channels exceeds the decoding kernel's 4,096")
        width = self.width
        self.w_in = rt.matrix(torch.cat([weights["y"], weights["x"]], dim=0))
        self.w_out = rt.matrix(weights["out"])

        def pair(first, second, size):
            if first not in weights and second not in weights:
                return None
            halves = [weights[name].float().reshape(-1) if name in weights else torch.zeros(size) for name in (first, second)]
            return rt.vector(torch.cat(halves))

        self.bias = pair("y_bias", "x_bias", width)
        self.conv = rt.vector(weights["conv"])
        if self.conv.shape != (width, self.taps):
            raise ValueError(f"gated_linear_recurrence: the convolution has shape {tuple(self.conv.shape)}, expected "
                             f"({width}, {self.taps})")
        self.conv_bias = rt.vector(weights["conv_bias"]) if "conv_bias" in weights else None
        gates = torch.stack([weights["recurrence_gate"].float(), weights["input_gate"].float()])
        if gates.shape != (2, self.blocks, part, part):
            raise ValueError(f"gated_linear_recurrence: the gates' matrices have shape {tuple(gates.shape[1:])}, expected "
                             f"({self.blocks}, {part}, {part})")
        self.gate_w = rt.vector(gates)                                   # [2, blocks, part, part]
        self.gate_bias = pair("recurrence_gate_bias", "input_gate_bias", width)
        self.lam = rt.vector(weights["lam"].reshape(-1))
        self.binding: Optional[StateBinding] = None
        self.projected = rt.scratch("linear_recurrence.proj", 2 * width, torch.float32)
        self.branch = rt.scratch("linear_recurrence.y", width, torch.float32)
        self.conved = rt.scratch("linear_recurrence.u", width, torch.float32)
        self.gates = rt.scratch("linear_recurrence.gates", 2 * width, torch.float32)
        self.result = rt.scratch("linear_recurrence.out", width)

    def cache_need(self):
        return StateNeed(elements=self.taps * self.width)

    def bind_cache(self, binding: StateBinding) -> None:
        self.binding = binding
        self.carried = binding.state                                       # [taps - 1, width] at the slot's start
        self.state = binding.state[:, (self.taps - 1) * self.width:]      # [width] behind them

    ends_with_product = True

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t, b, width = self.rt, step.tokens, self.binding, self.width
        rt.linear(x, self.w_in, self.projected, t)
        if step.max_span == 1 and step.spans == t:
            kernels.lru_decode(self.projected, self.bias, self.conv, self.conv_bias, self.carried, self.state,
                               b.slot_stride, step.span_slot, self.gate_w, self.gate_bias, self.lam, self.gate_factor,
                               self.result, t, width, self.taps, self.blocks)
        else:
            kernels.lru_prepare(self.projected, self.bias, self.conv, self.conv_bias, self.carried, b.slot_stride,
                                step.token_span, step.span_begin, step.span_slot, self.branch, self.conved, t,
                                step.spans, width, self.taps)
            part = width // self.blocks
            kernels.block_diagonal_product(self.conved, self.blocks, self.gate_w.view(2 * self.blocks, part, part),
                                           self.gates, t)
            kernels.lru_scan(self.gates, self.conved, self.gate_bias, self.lam, self.gate_factor, self.branch,
                             self.result, self.state, b.slot_stride, step.span_begin, step.span_slot, t, step.spans,
                             width)
        rt.linear(self.result, self.w_out, out, t)
