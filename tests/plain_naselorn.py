"""A plain, slow Naselorn model: whole sequences, no cache, float64, one function a mechanism.

Naselorn is a decoder-only model of pre-norm blocks: x <- x + Mixer(Norm(x)), then x <- x + FeedForward(Norm(x)), the
norm an RMS norm whose stored weight w stands for the scale 1 + w. Token rows are the embedding rows times a constant
plus a sinusoidal vector of the position. Two kinds of mixers: ``lightning`` (linear attention with SiLU on q, k and v,
a fixed decay per head, one RMS norm over all heads together, a sigmoid gate) and ``parallel`` (two mixers of the same
input side by side, their results added with two constants: a softmax attention without rotation whose queries see only
the keys of their own chunk of positions, with biases on every projection, and a gated linear recurrent unit behind a
short causal convolution, with block-diagonal gates). Feed-forward: a gated one with ReLU, or a mixture of SiLU-gated
experts (the largest router logits choose, softmax over the chosen logits weighs) plus a shared expert. This file shares
no code with the ``celeg_b200`` package: it takes the configuration as the dict that config.json holds and the weights as
a dict of arrays.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np


def as_float64(tensors) -> Dict[str, np.ndarray]:
    """{name: torch tensor} -> {name: float64 array}."""
    import torch
    return {name: value.to(torch.float64).numpy() for name, value in tensors.items()}


# ------------------------------------------------------------------------- small functions
def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def relu(x):
    return np.maximum(x, 0.0)


def softplus(x):
    return np.logaddexp(0.0, x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_scaled(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x: np.ndarray, stored: np.ndarray, eps: float) -> np.ndarray:
    """The blocks' norm: the stored weight lies around zero and stands for 1 + itself."""
    return rms_scaled(x, eps) * (1.0 + stored)


# ------------------------------------------------------------------------------ the input
def sinusoid(positions: Sequence[int], width: int) -> np.ndarray:
    """[positions, width]: entry 2i is sin(p f_i), entry 2i + 1 cos(p f_i), f_i = 10000^(-2i / width)."""
    out = np.zeros((len(positions), width), dtype=np.float64)
    for row, p in enumerate(positions):
        for i in range((width + 1) // 2):
            angle = p * 10000.0 ** (-2.0 * i / width)
            out[row, 2 * i] = math.sin(angle)
            if 2 * i + 1 < width:
                out[row, 2 * i + 1] = math.cos(angle)
    return out


def embed(config: dict, tensors, tokens: Sequence[int]) -> np.ndarray:
    rows = tensors["embed"][np.asarray(tokens)] * float(config["embedding"]["scale"])
    return rows + sinusoid(range(len(tokens)), int(config["width"]))


# --------------------------------------------------------------------------------- mixers
def lightning(tensors, base: str, mixer: dict, h: np.ndarray, eps: float) -> np.ndarray:
    """Per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; the heads' read-outs side by side are RMS-normed as
    one vector with a plain weight, gated by sigmoid(W_g h) and projected."""
    heads, dim, vdim = int(mixer["heads"]), int(mixer["dim"]), int(mixer["vdim"])
    tokens = h.shape[0]
    q = silu(h @ tensors[base + "q"].T).reshape(tokens, heads, dim)
    k = silu(h @ tensors[base + "k"].T).reshape(tokens, heads, dim)
    v = silu(h @ tensors[base + "v"].T).reshape(tokens, heads, vdim)
    read = np.zeros((tokens, heads, vdim), dtype=np.float64)
    for head in range(heads):
        state = np.zeros((dim, vdim), dtype=np.float64)
        decay = float(mixer["decay"][head])
        for t in range(tokens):
            state = decay * state + np.outer(k[t, head], v[t, head])
            read[t, head] = state.T @ q[t, head]
    normed = rms_scaled(read.reshape(tokens, heads * vdim), eps) * tensors[base + "norm"]
    gated = normed * sigmoid(h @ tensors[base + "g"].T)
    return gated @ tensors[base + "o"].T


def chunked_attention(tensors, base: str, mixer: dict, h: np.ndarray) -> np.ndarray:
    """Softmax attention without any rotation; query i sees key j <= i only when both lie in the same chunk of
    ``mask.size`` positions counted from position 0. Query head n reads key/value head n // (heads / kv_heads)."""
    heads, groups = int(mixer["heads"]), int(mixer["kv_heads"])
    dim, vdim = int(mixer["dim"]), int(mixer["vdim"])
    size = int(mixer["mask"]["size"]) if mixer.get("mask") else None
    scale = float(mixer["scale"])
    tokens = h.shape[0]
    q = (h @ tensors[base + "q"].T + tensors[base + "q.b"]).reshape(tokens, heads, dim)
    k = (h @ tensors[base + "k"].T + tensors[base + "k.b"]).reshape(tokens, groups, dim)
    v = (h @ tensors[base + "v"].T + tensors[base + "v.b"]).reshape(tokens, groups, vdim)
    out = np.zeros((tokens, heads, vdim), dtype=np.float64)
    for head in range(heads):
        group = head // (heads // groups)
        for i in range(tokens):
            first = 0 if size is None else (i // size) * size
            scores = (k[first:i + 1, group] @ q[i, head]) * scale
            weights = np.exp(scores - scores.max())
            weights /= weights.sum()
            out[i, head] = weights @ v[first:i + 1, group]
    return out.reshape(tokens, heads * vdim) @ tensors[base + "o"].T + tensors[base + "o.b"]


def causal_conv(x: np.ndarray, taps: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """x [tokens, channels], taps [channels, n]: the last tap meets the current token, zeros before the start."""
    tokens, n = x.shape[0], taps.shape[1]
    out = np.tile(bias, (tokens, 1)).astype(np.float64)
    for t in range(tokens):
        for j in range(n):
            source = t - (n - 1 - j)
            if source >= 0:
                out[t] += taps[:, j] * x[source]
    return out


def gated_recurrent_unit(tensors, base: str, mixer: dict, h: np.ndarray) -> np.ndarray:
    """Two branches of ``width`` channels: y = gelu_tanh(W_y h + b) and u = conv(W_x h + b). In each of ``blocks`` equal
    parts of the channels r = sigmoid(A_b u_b + a_b) and i = sigmoid(I_b u_b + i_b); a = exp(-8 r softplus(lam));
    S_t = a S_(t-1) + sqrt(1 - a^2) i u from S = 0, also at the first token; out = W_o (S y)."""
    width, blocks = int(mixer["width"]), int(mixer["blocks"])
    tokens = h.shape[0]
    y = gelu_tanh(h @ tensors[base + "y"].T + tensors[base + "y.b"])
    u = causal_conv(h @ tensors[base + "x"].T + tensors[base + "x.b"], tensors[base + "conv"], tensors[base + "conv.b"])
    part = width // blocks
    r = np.zeros_like(u)
    i = np.zeros_like(u)
    for b in range(blocks):
        cut = slice(b * part, (b + 1) * part)
        r[:, cut] = sigmoid(u[:, cut] @ tensors[base + "ra"][b].T + tensors[base + "ra.b"][b])
        i[:, cut] = sigmoid(u[:, cut] @ tensors[base + "ri"][b].T + tensors[base + "ri.b"][b])
    a = np.exp(-8.0 * r * softplus(tensors[base + "lam"]))
    state = np.zeros(width, dtype=np.float64)
    states = np.zeros((tokens, width), dtype=np.float64)
    for t in range(tokens):
        state = a[t] * state + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        states[t] = state
    return (states * y) @ tensors[base + "o"].T


def side_by_side(tensors, base: str, mixer: dict, h: np.ndarray) -> np.ndarray:
    left = chunked_attention(tensors, base + "left.", mixer["left"], h)
    right = gated_recurrent_unit(tensors, base + "right.", mixer["right"], h)
    return float(mixer["left_scale"]) * left + float(mixer["right_scale"]) * right


# ----------------------------------------------------------------------------- feed-forward
def gated_feed_forward(tensors, base: str, h: np.ndarray, act) -> np.ndarray:
    return (act(h @ tensors[base + "gate"].T) * (h @ tensors[base + "up"].T)) @ tensors[base + "down"].T


def route(tensors, base: str, mlp: dict, h: np.ndarray):
    """(chosen [tokens, top], weights [tokens, top]): the largest logits choose; softmax over the chosen logits."""
    top = int(mlp["router"]["top"])
    logits = h @ tensors[base + "router"].T + tensors[base + "router.b"]
    chosen = np.argsort(-logits, axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(logits, chosen, axis=-1)
    weights = np.exp(picked - picked.max(axis=-1, keepdims=True))
    return chosen, weights / weights.sum(axis=-1, keepdims=True)


def mixture_of_experts(tensors, base: str, mlp: dict, h: np.ndarray) -> np.ndarray:
    chosen, weights = route(tensors, base, mlp, h)
    out = np.zeros((h.shape[0], tensors[base + "e0.down"].shape[0]), dtype=np.float64)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * gated_feed_forward(tensors, f"{base}e{int(e)}.", h[t:t + 1], silu)[0]
    if mlp.get("shared"):
        out += gated_feed_forward(tensors, base + "shared.", h, silu)
    return out


def feed_forward(tensors, base: str, mlp: Optional[dict], h: np.ndarray):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return gated_feed_forward(tensors, base, h, relu)
    if mlp["kind"] == "moe":
        return mixture_of_experts(tensors, base, mlp, h)
    raise ValueError(mlp["kind"])


def mixer_of(tensors, base: str, layer: dict, h: np.ndarray, eps: float) -> np.ndarray:
    if layer["type"] == "lightning":
        return lightning(tensors, base, layer["mixer"], h, eps)
    if layer["type"] == "parallel":
        return side_by_side(tensors, base, layer["mixer"], h)
    raise ValueError(layer["type"])


# ------------------------------------------------------------------------------- the model
def streams(config: dict, tensors: Dict[str, np.ndarray], tokens: Sequence[int]) -> List[np.ndarray]:
    """The stream after every block, [tokens, width] each."""
    eps = float(config["norm"]["eps"])
    x = embed(config, tensors, tokens)
    out = []
    for index, layer in enumerate(config["layers"]):
        base = f"l{index}."
        x = x + mixer_of(tensors, base + "mix.", layer, offset_norm(x, tensors[base + "norm1"], eps), eps)
        if layer.get("mlp") is not None:
            x = x + feed_forward(tensors, base + "mlp.", layer["mlp"], offset_norm(x, tensors[base + "norm2"], eps))
        out.append(x)
    return out


def logits(config: dict, tensors: Dict[str, np.ndarray], tokens: Sequence[int]) -> np.ndarray:
    x = streams(config, tensors, tokens)[-1]
    return offset_norm(x, tensors["final.norm"], float(config["norm"]["eps"])) @ tensors["head"].T
