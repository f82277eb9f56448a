"""Small Liverax configurations with weights of the tests' own making, written as model folders.

The sizes differ from one configuration to the next in every respect that the design leaves open (widths, head
counts and groupings, key and value sizes, how much of a head is rotated, rotation bases with and without a divisor,
windows, with and without a mask, latent ranks, numbers of distance buckets and the farthest distance, the query
factor's constants, which layers blend their values and which kind comes first among them, layers without a
feed-forward, with and without capped logits). Weights come from a numpy generator and are rounded to bfloat16, so the
float64 plain model and the engine read the same numbers. ``sharpen`` scales the query and key projections (softmax close
to one-hot, so a single key shows).
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Dict, Optional

import numpy as np
import torch


def attention(heads, kv_heads, dim, vdim, scale=None, rot_dims=None, base=10000.0, divide=None, window=None, v_mix=False):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale,
             "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}, "v_mix": v_mix}
    if divide is not None:
        mixer["rot"]["scaling"] = {"factor": divide}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer, "buckets": 0}


def attention_2(heads, kv_heads, dim, vdim, buckets, far, scale=None, temp=None, v_mix=False):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale,
             "bias_max": far, "v_mix": v_mix}
    if temp is not None:
        mixer["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention_2", "mixer": mixer, "buckets": buckets}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale=None, base=10000.0, window=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": (dim + rot_dim) ** -0.5 if scale is None else scale, "rot": {"base": base, "dims": rot_dim}}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "buckets": 0}


def with_mlp(layer, ff):
    layer = copy.deepcopy(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return layer


def config(vocab, width, layers, eps=1e-5, cap=25.0):
    """``layers`` carry the rows of their distance tables under ``buckets``; the written config.json does not (the
    checkpoint's shapes say it)."""
    raw = {"architecture": "Liverax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if cap is not None:
        raw["logit_softcap"] = cap
    return raw


def for_disk(raw: dict) -> dict:
    out = copy.deepcopy(raw)
    for layer in out["layers"]:
        layer.pop("buckets", None)
    return out


# every kind twice; two key heads; heads rotated in part, with and without a divisor; values blended in four layers, the
# first of them of the rotary kind; windows of 24 and 33 (no multiple of a page) and a latent window of 20
MIXED = config(160, 64, [
    with_mlp(attention(4, 2, 16, 16, rot_dims=8, divide=4.0, window=24, v_mix=True), 96),
    with_mlp(latent(4, 16, 8, 24, 40, 32, window=20, base=5000.0), 80),
    with_mlp(attention_2(4, 2, 16, 16, 8, 48, scale=0.3, temp=(0.5, 16), v_mix=True), 72),
    with_mlp(attention(8, 2, 8, 16, window=33, v_mix=True), None),
    with_mlp(latent(2, 8, 16, 8, 24, 16), 64),
    with_mlp(attention_2(2, 2, 32, 16, 12, 100, temp=(0.2, 7), v_mix=True), 48),
])

# sizes that fit no vector width: a width of 36, keys of 12 with values of 7, seventeen query heads on one key head, an
# odd number of buckets, a window of 1 (a token sees itself only) and of 7, the first blended layer of the distance
# kind, a distance layer without the query factor, no capped logits
ODD = config(50, 36, [
    with_mlp(attention_2(3, 3, 12, 7, 5, 9, v_mix=True), 20),
    with_mlp(attention(3, 3, 12, 7, rot_dims=6, base=77.0, window=7, v_mix=True), None),
    with_mlp(latent(5, 6, 4, 5, 10, 7, window=1), 44),
    with_mlp(attention(17, 1, 10, 10, rot_dims=2, divide=1.5), 12),
    with_mlp(latent(3, 10, 2, 3, 6, 9, base=300.0), None),
    with_mlp(attention_2(6, 3, 6, 7, 4, 300, temp=(1.0, 1), v_mix=True), 30),
], eps=1e-6, cap=None)

# heads of 64 and of 128 (the tensor-core kernels' sizes), windows of 160 and 70, a latent vector of 64 + 64, thirty-two
# buckets up to distance 512
WIDE = config(200, 128, [
    with_mlp(attention(8, 1, 64, 64, scale=0.11, window=160, divide=2.5, v_mix=True), 160),
    with_mlp(attention_2(4, 2, 64, 64, 32, 512, temp=(0.3, 64), v_mix=False), 96),
    with_mlp(latent(6, 48, 64, 40, 64, 48, window=70), None),
    with_mlp(attention_2(2, 1, 128, 64, 6, 40, scale=0.05, v_mix=True), 64),
    with_mlp(attention(4, 4, 128, 128, rot_dims=64, base=500000.0), 200),
])

CONFIGS = {"mixed": (MIXED, 11), "odd": (ODD, 15), "wide": (WIDE, 13)}


def single_layer(layer, ff=None, vocab=96, width=48, cap=None):
    """A model of one layer, to look at one mechanism alone."""
    return config(vocab, width, [with_mlp(layer, ff)], cap=cap)


def _round(values) -> torch.Tensor:
    return torch.from_numpy(np.asarray(values, dtype=np.float32)).to(torch.bfloat16)


def make_tensors(raw: dict, seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    rng = np.random.default_rng(seed)
    width, vocab = raw["width"], raw["vocab"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = _round(rng.normal(0.0, gain / math.sqrt(cols), size=(rows, cols)))

    def vector(name, size, mean=0.0, std=0.3):
        out[name] = _round(rng.normal(mean, std, size=(size,)))

    out["embed"] = _round(rng.normal(0.0, 1.0, size=(vocab, width)))
    for index, layer in enumerate(raw["layers"]):
        base = f"l{index}."
        mix, m = base + "mix.", layer["mixer"]
        vector(base + "norm1", width, 1.0, 0.2)
        heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "latent_attention":
            rot, rank, q_rank = m["rot_dim"], m["kv_rank"], m["q_rank"]
            matrix(mix + "dq", q_rank, width)
            vector(mix + "dq.norm", q_rank, 1.0, 0.2)
            matrix(mix + "uq", heads * (dim + rot), q_rank, gain=sharpen)
            matrix(mix + "dkv", rank + rot, width, gain=sharpen)
            vector(mix + "dkv.norm", rank, 1.0, 0.2)
            matrix(mix + "uk", heads * dim, rank)
            matrix(mix + "uv", heads * vdim, rank)
            vector(mix + "sink", heads, 0.0, 1.0)
            matrix(mix + "g", heads * vdim, width)
            matrix(mix + "o", width, heads * vdim)
        else:
            groups = m["kv_heads"]
            matrix(mix + "q", heads * dim, width, gain=sharpen)
            matrix(mix + "k", groups * dim, width, gain=sharpen)
            matrix(mix + "v", groups * vdim, width)
            matrix(mix + "o", width, heads * vdim)
            if m.get("v_mix"):
                out[mix + "vmix"] = _round(rng.uniform(0.2, 0.8))
            if layer["type"] == "attention_2":
                vector(mix + "q.b", heads * dim)
                vector(mix + "k.b", groups * dim)
                vector(mix + "v.b", groups * vdim)
                vector(mix + "q.norm", heads * dim, sharpen, 0.2)
                vector(mix + "k.norm", groups * dim, sharpen, 0.2)
                out[mix + "rel"] = _round(rng.normal(0.0, 1.0, size=(layer["buckets"], heads)))
                matrix(mix + "g", heads * vdim, width)
        if layer.get("mlp") is None:
            continue
        vector(base + "norm2", width, 1.0, 0.2)
        inner = layer["mlp"]["ff"]
        matrix(base + "mlp.gate", inner, width)
        matrix(base + "mlp.up", inner, width)
        matrix(base + "mlp.down", width, inner)
    vector("final.norm", width, 1.0, 0.2)
    matrix("head", vocab, width)
    return out


def write_model(folder: str, raw: dict, seed: int, sharpen: float = 1.0,
                tensors: Optional[Dict[str, torch.Tensor]] = None):
    """Writes ``folder`` and returns (config as written, {name: bfloat16 tensor})."""
    from safetensors.torch import save_file
    tensors = tensors if tensors is not None else make_tensors(raw, seed, sharpen)
    os.makedirs(folder, exist_ok=True)
    disk = for_disk(raw)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(disk, handle, indent=1)
    save_file({name: value.contiguous() for name, value in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return disk, tensors
