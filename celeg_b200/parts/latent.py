"""The latent-attention mixer (kernels: csrc/latent_attention.cu and the attention kernels of the paged cache).

Per position the cache holds one vector [c | r]: c = rms_norm(W_down h)[:rank] * w, from which head h's key
U_h c and value V_h c would be up-projected, and r, a rotated key part shared by all heads. A head's score
q_h . (U_h c) + q_rot_h . r equals (U_h^T q_h) . c + q_rot_h . r, so the query is taken to the latent space once
per token, the attention kernels see ONE key head of size rank + rot shared by all query heads whose values are
the keys themselves (only their first ``rank`` elements are used afterwards), and each head's result is
up-projected by V_h and multiplied by its output gate sigmoid(W_g h)_h. Keys and values per head are never
materialised, in prompts or in decoding (DeepSeek-AI, "DeepSeek-V2: A Strong, Economical, and Efficient
Mixture-of-Experts Language Model", 2024, describes the absorption).
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from .. import kernels
from ..cache.manager import PagedNeed
from .mixers import PagedAttentionKernels, PagedBinding
from .registry import register_part
from .runtime import Runtime, StepContext


@register_part("mixer", "latent_attention")
class LatentAttentionMixer(PagedAttentionKernels):
    """q = W_q h laid out head by head as [dim unrotated | rot_dim rotated]; W_down h = [rank latent | rot_dim shared
    rotated key part]; scores (q_unrotated . U_h c + q_rotated . r) * scale, causal softmax; head outputs V_h (sum p c)
    times sigmoid(W_g h)_h; W_o on the concatenated heads. The nested part ``position`` gives the rotation's
    frequencies and the factor of its cos and sin; it pairs neighbouring dimensions (``rope_interleaved``) or dimensions
    i and i + half (``rope_split_half``).

    Optional: the queries through a latent vector of their own (tensors ``q_down``, ``q_down_norm``; then ``q`` is the
    up-projection of rms_norm(W_q_down h) * w); ``window`` = w lets position i read j when 0 <= i - j < w; a sink per
    head in the softmax's denominator (tensor ``sinks``); ``gate_per_element``: the gate matrix has a row for every
    element of every head's result instead of one per head."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.rot = int(params["rot_dim"])
        self.vdim = int(params["vdim"])
        self.rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["eps"])
        window = params.get("window")
        self.window = int(window) if window else None
        self.sinks = rt.vector(weights["sinks"]) if "sinks" in weights else None
        if self.sinks is not None and self.sinks.shape != (self.heads,):
            raise ValueError(f"latent_attention: sinks of shape {tuple(self.sinks.shape)}, expected ({self.heads},)")
        self.gate_per_element = bool(params.get("gate_per_element", False))
        self.kv_heads = 1
        self.head_dim = self.rank + self.rot                 # what the attention kernels see as the head size
        if self.head_dim > 512:
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {self.head_dim} exceeds 512")
        position = parts.get("position")
        fused = position.fused() if position is not None else None
        if fused is None or not fused.get("rotary_dim") or fused["rotary_dim"] > self.rot:
            raise ValueError("latent_attention needs a position part that rotates pairs of at most rot_dim dimensions")
        self.halves = not fused.get("interleaved", False)
        self.rotary_dim = int(fused["rotary_dim"])
        self.frequencies = fused["inv_freq"]
        self.magnitude = float(fused.get("magnitude", 1.0))
        self.q_width = self.heads * (self.dim + self.rot)
        self.down_width = self.rank + self.rot
        # with a query latent the fused projection leaves [q latent | down | gate] and q follows from the normed latent
        self.q_rank = int(weights["q_down"].shape[0]) if "q_down" in weights else 0
        self.first_width = self.q_rank or self.q_width
        fused_in = torch.cat([weights["q_down"] if self.q_rank else weights["q"], weights["down"], weights["gate"]], dim=0)
        self.proj_width = int(fused_in.shape[0])
        self.w_in = rt.matrix(fused_in)
        if self.q_rank:
            self.w_q_up = rt.matrix(weights["q"])               # [heads * (dim + rot), q_rank]
            self.q_down_norm = rt.vector(weights["q_down_norm"])
            self.q_latent = rt.scratch("latent.q_latent", self.q_rank)
            self.q_rows = rt.scratch("latent.q", self.q_width)
        self.w_up_keys = rt.matrix(weights["up_keys"])         # [heads * dim, rank]
        self.w_up_values = rt.matrix(weights["up_values"])     # [heads * vdim, rank]
        self.w_out = rt.matrix(weights["out"])
        self.down_norm = rt.vector(weights["down_norm"])
        self.binding: Optional[PagedBinding] = None
        self._resident_blocks: Optional[int] = None
        self.projected = rt.scratch("latent.proj", self.proj_width)
        self.qkv = rt.scratch("latent.query", self.heads * self.head_dim)          # absorbed queries
        self.qkv_width = self.heads * self.head_dim
        self.attended = rt.scratch("latent.attended", self.heads * self.head_dim)
        self.values = rt.scratch("latent.values", self.heads * self.vdim)

    def cache_need(self):
        return PagedNeed(kv_heads=1, head_dim=self.head_dim, window=self.window, value_head_dim=0)

    def bind_cache(self, binding: PagedBinding) -> None:
        self.binding = binding

    def _value_cache(self) -> torch.Tensor:
        return self.binding.k

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, b, t = self.rt, self.binding, step.tokens
        rt.linear(x, self.w_in, self.projected, t)
        rows = self.projected
        down = rows[:, self.first_width:self.first_width + self.down_width]
        gate = rows[:, self.first_width + self.down_width:]
        if self.q_rank:
            kernels.rmsnorm_strided(rows[:, :self.q_rank], self.q_down_norm, self.q_latent, self.eps, t)
            rt.linear(self.q_latent, self.w_q_up, self.q_rows, t)
            q = self.q_rows
        else:
            q = rows[:, :self.q_width]
        table = step.block_tables[b.group]
        kernels.latent_prepare(q, down, self.down_norm, self.frequencies, self.magnitude, self.eps, step.positions,
                               step.token_span, table, b.k, b.page_tokens, self.qkv, t, self.heads, self.dim,
                               self.rot, self.rotary_dim, self.rank, step.error_flag, halves=self.halves)
        library = rt.act_dtype == torch.bfloat16 and not rt.small_batch(t)
        # the query in the latent space: (U_h^T q_h) for every head, beside its rotated part
        if library:
            # many bfloat16 rows: one batched library product over the heads (views, nothing is copied)
            torch.bmm(q[:t].unflatten(1, (self.heads, self.dim + self.rot))[:, :, :self.dim].transpose(0, 1),
                      self.w_up_keys.view(self.heads, self.dim, self.rank),
                      out=self.qkv[:t].unflatten(1, (self.heads, self.head_dim))[:, :, :self.rank].transpose(0, 1))
        else:
            kernels.head_project(q, self.dim + self.rot, self.w_up_keys, True, self.qkv, self.head_dim, t, self.heads,
                                 self.rank, self.dim)
        self.attend(step, table)
        # V_h (sum p c) times the head's gate
        if library:
            torch.bmm(self.attended[:t].unflatten(1, (self.heads, self.head_dim))[:, :, :self.rank].transpose(0, 1),
                      self.w_up_values.view(self.heads, self.vdim, self.rank).transpose(1, 2),
                      out=self.values[:t].unflatten(1, (self.heads, self.vdim)).transpose(0, 1))
            if self.gate_per_element:
                kernels.head_gate(self.values, 1, gate, t, self.heads * self.vdim)
            else:
                kernels.head_gate(self.values, self.vdim, gate, t, self.heads)
        else:
            kernels.head_project(self.attended, self.head_dim, self.w_up_values, False, self.values, self.vdim, t,
                                 self.heads, self.vdim, self.rank, gate=gate, gate_per_element=self.gate_per_element)
        rt.linear(self.values, self.w_out, out, t)
