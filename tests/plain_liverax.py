"""A plain, slow Liverax model: whole sequences, no cache, float64, one function a mechanism.

Liverax is a decoder-only model of pre-norm blocks, x <- x + Mixer(N(x)) and then, where the layer has a feed-forward,
x <- x + FeedForward(N'(x)); N is a layer norm with a weight and no bias. Three kinds of mixers, all softmax attention:

* ``attention``: grouped queries, a rotation of the leading dimensions of every q and k head in pairs (i, i + half) whose
  frequencies may be divided by a constant, a window of recent positions;
* ``attention_2``: biases on q, k and v, one RMS norm over the whole q projection and one over the whole k projection,
  no rotation, a query factor that grows with the logarithm of the position, a learned number per (head, distance
  bucket) added to the scaled scores, every earlier position visible, a sigmoid gate on the heads' results;
* ``latent_attention``: the queries through a normed latent vector, keys and values up-projected from one normed latent
  vector per position plus one rotated key part that all heads share, a window, a learned sink per head in the softmax's
  denominator, a sigmoid gate.

In layers marked for it the values are blended with the values that the first marked layer made of the same token.
The feed-forward is gated with the tanh form of GELU; the logits are capped smoothly. This file shares no code with the
``celeg_b200`` package: it takes the configuration as the dict that config.json holds and the weights as a dict of arrays.
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_scaled(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """(x - mean) / sqrt(mean of squared deviations + eps) * weight over the last axis; no bias."""
    centred = x - np.mean(x, axis=-1, keepdims=True)
    return centred / np.sqrt(np.mean(centred * centred, axis=-1, keepdims=True) + eps) * weight


# ------------------------------------------------------------------------------ positions
def rotate_halves(x: np.ndarray, positions: Sequence[int], dims: int, base: float, divide_by: float = 1.0) -> np.ndarray:
    """x: [T, heads, size]. Of every head the first ``dims`` entries are turned: entry i and entry i + dims/2 form a
    pair that is rotated by the angle position * base^(-2i / dims) / divide_by; entries from ``dims`` on stay."""
    half = dims // 2
    out = x.copy()
    frequencies = base ** (-2.0 * np.arange(half) / dims) / divide_by
    angles = np.asarray(positions, dtype=np.float64)[:, None] * frequencies[None, :]          # [T, half]
    cos, sin = np.cos(angles)[:, None, :], np.sin(angles)[:, None, :]
    first, second = x[..., :half], x[..., half:dims]
    out[..., :half] = first * cos - second * sin
    out[..., half:dims] = second * cos + first * sin
    return out


def query_temperature(position: int, coef: float, every: int) -> float:
    """1 + coef * ln(floor((position + 1) / every) + 1)."""
    return 1.0 + coef * math.log((position + 1) // every + 1)


def distance_bucket(distance: int, buckets: int, far: float) -> int:
    """The row of a layer's distance table for a key ``distance`` positions back. The first half of the rows stand for
    one distance each; the others split the distances from buckets/2 to ``far`` evenly in the logarithm; the last row
    takes everything farther."""
    exact = buckets // 2
    if distance < exact:
        return distance
    stretched = exact + int(math.floor(math.log(distance / exact) / math.log(far / exact) * (buckets - exact)))
    return min(buckets - 1, stretched)


# -------------------------------------------------------------------------------- softmax
def masked_softmax_rows(scores: np.ndarray, window: Optional[int], sink: Optional[float] = None) -> np.ndarray:
    """scores: [T, T] of one head, query i over key j. Key j is visible to query i when j <= i and, with a window w,
    i - j < w. A sink adds exp(sink) to the denominator and nothing else."""
    count = scores.shape[0]
    weights = np.zeros_like(scores)
    for i in range(count):
        first = 0 if window is None else max(0, i - window + 1)
        row = scores[i, first:i + 1]
        top = row.max() if sink is None else max(row.max(), sink)
        e = np.exp(row - top)
        denominator = e.sum() + (0.0 if sink is None else math.exp(sink - top))
        weights[i, first:i + 1] = e / denominator
    return weights


# --------------------------------------------------------------------------------- mixers
def blend_values(v: np.ndarray, first_values: Optional[np.ndarray], lam: float) -> np.ndarray:
    """(1 - lam) v + lam v_first; the first marked layer (no ``first_values`` yet) keeps its own."""
    if first_values is None:
        return v
    return (1.0 - lam) * v + lam * first_values


def grouped_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: Optional[int],
                      bias_of=None, sinks: Optional[np.ndarray] = None) -> np.ndarray:
    """q: [T, H, d], k: [T, G, d], v: [T, G, dv]; query head h reads key/value head h // (H / G).
    ``bias_of(h)`` gives a [T, T] matrix added to the scaled scores of head h. Returns [T, H * dv]."""
    tokens, heads, _ = q.shape
    group = heads // k.shape[1]
    out = np.zeros((tokens, heads, v.shape[2]))
    for h in range(heads):
        g = h // group
        scores = q[:, h, :] @ k[:, g, :].T * scale
        if bias_of is not None:
            scores = scores + bias_of(h)
        weights = masked_softmax_rows(scores, window, None if sinks is None else float(sinks[h]))
        out[:, h, :] = weights @ v[:, g, :]
    return out.reshape(tokens, -1)


def rotary_attention(h: np.ndarray, positions: Sequence[int], m: dict, w: Dict[str, np.ndarray], prefix: str,
                     shared: dict) -> np.ndarray:
    """The ``attention`` mixer. ``shared`` carries the first marked layer's values through the model."""
    tokens = h.shape[0]
    heads, groups = m["heads"], m.get("kv_heads") or m["heads"]
    q = (h @ w[prefix + "q"].T).reshape(tokens, heads, m["dim"])
    k = (h @ w[prefix + "k"].T).reshape(tokens, groups, m["dim"])
    v = (h @ w[prefix + "v"].T).reshape(tokens, groups, m["vdim"])
    rot = m.get("rot")
    if rot:
        divide = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate_halves(q, positions, rot["dims"], rot["base"], divide)
        k = rotate_halves(k, positions, rot["dims"], rot["base"], divide)
    if m.get("v_mix"):
        v = blend_values(v, shared.get("first_values"), float(w[prefix + "vmix"]))
        shared.setdefault("first_values", v)
    window = (m.get("mask") or {}).get("size")
    return grouped_attention(q, k, v, m["scale"], window) @ w[prefix + "o"].T


def distance_attention(h: np.ndarray, positions: Sequence[int], m: dict, w: Dict[str, np.ndarray], prefix: str,
                       eps: float, shared: dict) -> np.ndarray:
    """The ``attention_2`` mixer."""
    tokens = h.shape[0]
    heads, groups = m["heads"], m.get("kv_heads") or m["heads"]
    q = h @ w[prefix + "q"].T + w[prefix + "q.b"]
    k = h @ w[prefix + "k"].T + w[prefix + "k.b"]
    v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).reshape(tokens, groups, m["vdim"])
    q = rms_scaled(q, eps) * w[prefix + "q.norm"]            # one norm over all heads' rows together
    k = rms_scaled(k, eps) * w[prefix + "k.norm"]
    temperature = m.get("q_temp")
    if temperature:
        factors = np.array([query_temperature(p, temperature["coef"], temperature["every"]) for p in positions])
        q = q * factors[:, None]
    q = q.reshape(tokens, heads, m["dim"])
    k = k.reshape(tokens, groups, m["dim"])
    if m.get("v_mix"):
        v = blend_values(v, shared.get("first_values"), float(w[prefix + "vmix"]))
        shared.setdefault("first_values", v)
    table = w[prefix + "rel"]                                   # [buckets, heads]
    buckets = table.shape[0]
    where = np.asarray(positions, dtype=np.int64)
    row_of = np.array([distance_bucket(n, buckets, m["bias_max"]) for n in range(int(where.max()) + 1)], dtype=np.int64)
    rows = row_of[np.clip(where[:, None] - where[None, :], 0, None)]          # (keys after the query are never read)
    mixed = grouped_attention(q, k, v, m["scale"], None, bias_of=lambda head: table[rows, head])
    gate = sigmoid(h @ w[prefix + "g"].T)
    return (mixed * gate) @ w[prefix + "o"].T


def latent_attention(h: np.ndarray, positions: Sequence[int], m: dict, w: Dict[str, np.ndarray], prefix: str,
                     eps: float) -> np.ndarray:
    """The ``latent_attention`` mixer, nothing absorbed: every head's keys and values are built."""
    tokens = h.shape[0]
    heads, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    latent_q = rms_scaled(h @ w[prefix + "dq"].T, eps) * w[prefix + "dq.norm"]
    q = (latent_q @ w[prefix + "uq"].T).reshape(tokens, heads, dim + rot_dim)
    down = h @ w[prefix + "dkv"].T
    c = rms_scaled(down[:, :rank], eps) * w[prefix + "dkv.norm"]
    shared_key = down[:, rank:].reshape(tokens, 1, rot_dim)
    base = m["rot"]["base"]
    divide = float((m["rot"].get("scaling") or {}).get("factor", 1.0))
    q_rotated = rotate_halves(q[:, :, dim:], positions, rot_dim, base, divide)
    shared_key = rotate_halves(shared_key, positions, rot_dim, base, divide)
    keys = np.concatenate([(c @ w[prefix + "uk"].T).reshape(tokens, heads, dim),
                           np.repeat(shared_key, heads, axis=1)], axis=2)
    queries = np.concatenate([q[:, :, :dim], q_rotated], axis=2)
    values = (c @ w[prefix + "uv"].T).reshape(tokens, heads, vdim)
    window = (m.get("mask") or {}).get("size")
    sinks = w.get(prefix + "sink")
    mixed = grouped_attention(queries, keys, values, m["scale"], window, sinks=sinks)
    gate = sigmoid(h @ w[prefix + "g"].T)
    return (mixed * gate) @ w[prefix + "o"].T


# --------------------------------------------------------------------------- feed-forward
def gated_feed_forward(h: np.ndarray, w: Dict[str, np.ndarray], prefix: str) -> np.ndarray:
    return (gelu_tanh(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


# ------------------------------------------------------------------------------ the model
def forward(config: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], *, keep_layers: bool = False):
    """Logits [T, vocab] of one whole sequence from position 0; with ``keep_layers`` also the stream after every
    layer, [layers, T, width]."""
    eps = float(config["norm"]["eps"])
    positions = list(range(len(tokens)))
    x = w["embed"][np.asarray(tokens, dtype=np.int64)]
    shared: dict = {}
    kept: List[np.ndarray] = []
    for index, layer in enumerate(config["layers"]):
        base = f"l{index}."
        h = layer_norm(x, w[base + "norm1"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            x = x + rotary_attention(h, positions, m, w, base + "mix.", shared)
        elif kind == "attention_2":
            x = x + distance_attention(h, positions, m, w, base + "mix.", eps, shared)
        elif kind == "latent_attention":
            x = x + latent_attention(h, positions, m, w, base + "mix.", eps)
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        if layer.get("mlp") is not None:
            x = x + gated_feed_forward(layer_norm(x, w[base + "norm2"], eps), w, base + "mlp.")
        if keep_layers:
            kept.append(x.copy())
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    if keep_layers:
        return logits, np.stack(kept)
    return logits


def greedy(config: dict, w: Dict[str, np.ndarray], prompt: Sequence[int], new_tokens: int) -> List[int]:
    """Greedy continuation, the whole sequence recomputed for every token."""
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(np.argmax(forward(config, w, tokens)[-1])))
    return tokens[len(prompt):]
