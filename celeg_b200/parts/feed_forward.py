"""Feed-forward parts. Interface:

    FeedForward(params, weights, parts, rt)
    forward(x, out, step)     x: normed activations [T, hidden]; writes the output to out
    takes_split_norm(step)    optional, as for mixers
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import kernels
from .registry import register_part
from .runtime import Runtime, StepContext


ACTIVATIONS = {"gelu": kernels.ACT_GELU_ERF, "gelu_tanh": kernels.ACT_GELU_TANH, "silu": kernels.ACT_SILU,
               "relu2": kernels.ACT_RELU_SQUARED, "relu": kernels.ACT_RELU}


@register_part("feed_forward", "swiglu")
class SwiGluFeedForward:
    """down(silu(gate(x)) * up(x)); gate and up are one fused projection [2I, H] (gate rows
    first), as celeg concatenates w1 and w3 (src/backend/cpu/weights_loader.cpp:93-99;
    src/backend/cuda/packed/operators.cu:531-596). ``activation`` names another function of the gate (a gated
    linear unit with ReLU, a GELU, ...): in the weight-streaming product's epilogue for steps of few rows, else as the
    product and an element-wise kernel."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.inner = int(params["intermediate_size"])
        name = params.get("activation", "silu")
        if name not in ACTIVATIONS:
            raise ValueError(f"gated feed-forward: unknown activation {name!r}; known: {', '.join(ACTIVATIONS)}")
        self.activation = ACTIVATIONS[name]
        self.w_gate_up = rt.matrix(torch.cat([weights["gate"], weights["up"]], dim=0))
        self.w_down = rt.matrix(weights["down"])
        self.gate_up = rt.scratch("swiglu.gate_up", 2 * self.inner)
        self.activated = rt.scratch("swiglu.act", self.inner)

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def takes_split_norm(self, step: StepContext) -> bool:
        return self.rt.takes_split_norm(step.tokens, self.w_gate_up)

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t = self.rt, step.tokens
        rt.linear_swiglu(x, self.w_gate_up, self.gate_up, self.activated, t, self.inner, self.activation)
        rt.linear(self.activated, self.w_down, out, t)


@register_part("feed_forward", "dense")
class DenseFeedForward:
    """down(act(up(x))) with act one of ``gelu`` (exact, by erf), ``gelu_tanh``, ``silu`` or ``relu2`` (the square of
    ReLU); the activation in float32, rounded once."""

    ACTIVATIONS = ACTIVATIONS

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.inner = int(params["intermediate_size"])
        name = params.get("activation", "gelu")
        if name not in self.ACTIVATIONS:
            raise ValueError(f"dense feed-forward: unknown activation {name!r}; known: {', '.join(self.ACTIVATIONS)}")
        self.activation = self.ACTIVATIONS[name]
        self.w_up = rt.matrix(weights["up"])
        self.w_down = rt.matrix(weights["down"])
        self.raised = rt.scratch("dense.up", self.inner)

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t = self.rt, step.tokens
        rt.linear_activation(x, self.w_up, self.raised, t, self.activation)
        rt.linear(self.raised, self.w_down, out, t)


@register_part("feed_forward", "moe")
class MoeFeedForward:
    """A mixture of ``experts`` small feed-forwards down_e(act(up_e(x))) of which each token uses ``top``:
    s = softmax(W_router x) over all experts (float32 sums and softmax), the experts with the largest s + ``correction`` are
    chosen, their weights are their s divided by the sum of the chosen s (+ 1e-20), and the output is the weighted
    sum of their outputs. A nested part ``shared`` (any feed-forward) runs for every token and is added, times
    sigmoid(w_shared_gate . x) when the tensor ``shared_gate`` is given. A tensor ``router_bias`` is added to the
    router's logits. Without a correction the choice falls on the largest logits and the weights are the softmax over
    the chosen logits alone (s_e / sum of the chosen s is that softmax). With ``gated_experts`` an expert is a gated
    linear unit down_e(act(gate_e(x)) * up_e(x)): gate_e and up_e are stacked into one matrix, the first product
    leaves [gate | up] rows and an element-wise kernel makes the inner rows.

    Steps of few tokens stream the chosen experts' matrices once per (token, choice) pair; larger steps order the
    pairs by expert on the device and run both products tile by tile over a table the device makes, on a grid
    sized for the worst case, so that nothing on the host depends on the routing (kernels: csrc/moe.cu). On the
    bfloat16 path those two products are the grouped form of the tcgen05 product (csrc/gemm_tcgen05.cu: TMA boxes
    of 128 rows out of the rows gathered in expert order and out of the experts' stacked matrices, the activation
    in the epilogue), where the shapes allow it."""

    FEW_TOKENS = 16

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.inner = int(params["intermediate_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        name = params.get("activation", "relu2")
        if name not in DenseFeedForward.ACTIVATIONS:
            raise ValueError(f"moe: unknown activation {name!r}; known: {', '.join(DenseFeedForward.ACTIVATIONS)}")
        self.activation = DenseFeedForward.ACTIVATIONS[name]
        if not 0 < self.top <= self.experts:
            raise ValueError(f"moe: top {self.top} of {self.experts} experts")
        # the router's matrix, with the shared expert's gate as one more row: one product with float32 sums gives both
        self.gated = "shared_gate" in weights and parts.get("shared") is not None
        rows = [weights["router"]] + ([weights["shared_gate"].reshape(1, -1)] if self.gated else [])
        self.w_router = rt.matrix(torch.cat(rows, dim=0))
        self.logits = rt.scratch("moe.logits", int(self.w_router.shape[0]), torch.float32)
        self.correction = rt.vector(weights["correction"]) if "correction" in weights else None
        self.router_bias = rt.vector(weights["router_bias"]) if "router_bias" in weights else None
        self.gated_experts = bool(params.get("gated_experts", False))
        if self.gated_experts:                                                                        # [E, 2 inner, hidden]
            self.w_up = rt.matrix(torch.stack([torch.cat([weights[f"e{e}.gate"], weights[f"e{e}.up"]], dim=0)
                                               for e in range(self.experts)]))
        else:
            self.w_up = rt.matrix(torch.stack([weights[f"e{e}.up"] for e in range(self.experts)]))    # [E, inner, hidden]
        self.w_down = rt.matrix(torch.stack([weights[f"e{e}.down"] for e in range(self.experts)]))    # [E, hidden, inner]
        self.shared = parts.get("shared")
        pairs = rt.max_tokens * self.top
        self.max_pairs = pairs
        self.chosen = rt.flat_scratch("moe.chosen", pairs, torch.int32)
        self.weights = rt.flat_scratch("moe.weights", pairs, torch.float32)
        self.shared_gate = rt.flat_scratch("moe.shared_gate", rt.max_tokens, torch.float32)
        self.place = rt.flat_scratch("moe.place", pairs, torch.int32)
        self.source = rt.flat_scratch("moe.source", pairs, torch.int32)
        self.table = rt.flat_scratch("moe.table", 4 + 3 * kernels.moe_max_tiles(pairs, self.experts), torch.int32, zero=True)
        self.gathered = rt.flat_scratch("moe.gathered", pairs * self.hidden, rt.act_dtype).view(pairs, self.hidden)
        self.raised = rt.flat_scratch("moe.raised", pairs * self.inner, rt.act_dtype).view(pairs, self.inner)
        # gated experts: the first product's [gate | up] rows, before the element-wise kernel
        self.paired = (rt.flat_scratch("moe.paired", pairs * 2 * self.inner, rt.act_dtype).view(pairs, 2 * self.inner)
                       if self.gated_experts else None)
        self.lowered = rt.flat_scratch("moe.lowered", pairs * self.hidden, rt.act_dtype).view(pairs, self.hidden)
        self.shared_out = rt.scratch("moe.shared_out", self.hidden) if self.shared is not None else None

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        t, top = step.tokens, self.top
        pairs = t * top
        gated = self.gated
        self.rt.linear(x, self.w_router, self.logits, t)
        kernels.moe_route(self.logits, self.experts, self.correction, self.experts if gated else None, self.chosen,
                          self.weights, self.shared_gate if gated else None, t, top, bias=self.router_bias)
        if self.shared is not None:
            self.shared.forward(x, self.shared_out, step)
        # what the first product writes and which activation its epilogue applies
        first_out, first_act = (self.paired, -1) if self.gated_experts else (self.raised, self.activation)
        if t <= self.FEW_TOKENS:
            kernels.expert_rows(x, top, self.chosen, self.w_up, first_out, pairs, first_act)
            if self.gated_experts:
                kernels.glu(self.paired, self.raised, pairs, self.inner, self.activation)
            kernels.expert_rows(self.raised, 1, self.chosen, self.w_down, self.lowered, pairs, -1)
            place = None
        elif (self.rt.tensor_core_products != "none" and kernels.expert_product_tcgen05_supported(self.gathered, self.w_up)
              and kernels.expert_product_tcgen05_supported(self.raised, self.w_down)):
            kernels.moe_group(self.chosen, t, self.experts, top, self.place, self.source, self.table, tile_rows=128)
            tiles = kernels.moe_max_tiles(pairs, self.experts, 128)
            kernels.moe_gather_rows(x, self.source, self.gathered, pairs)
            kernels.expert_product_tcgen05(self.gathered, self.w_up, first_out, self.table, tiles, first_act,
                                           self.rt.error_flag)
            if self.gated_experts:
                kernels.glu(self.paired, self.raised, pairs, self.inner, self.activation)
            kernels.expert_product_tcgen05(self.raised, self.w_down, self.lowered, self.table, tiles, -1, self.rt.error_flag)
            place = self.place
        else:
            kernels.moe_group(self.chosen, t, self.experts, top, self.place, self.source, self.table)
            tiles = kernels.moe_max_tiles(pairs, self.experts)
            kernels.expert_product(x, self.source, self.w_up, first_out, self.table, tiles, first_act)
            if self.gated_experts:
                kernels.glu(self.paired, self.raised, pairs, self.inner, self.activation)
            kernels.expert_product(self.raised, None, self.w_down, self.lowered, self.table, tiles, -1)
            place = self.place
        kernels.moe_combine(self.lowered, place, self.weights, self.shared_out, self.shared_gate if gated else None,
                            out, t, top)
