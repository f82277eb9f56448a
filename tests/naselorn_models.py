"""Small Naselorn configurations with weights of the tests' own making, written as model folders.

The sizes differ from one configuration to the next in every respect that the design leaves open (widths, head
counts, key and value sizes, chunk sizes, with and without a chunked mask, decays, channels, blocks and taps of the
recurrent unit, the two constants of the side-by-side mixer, numbers of experts and choices, with and without a
shared expert, layers without a feed-forward, which mixer comes first). Weights come from a numpy generator and are
rounded to bfloat16, so the float64 plain model and the engine read the same numbers. Router matrices are drawn
large so that no choice of experts is a close call; ``sharpen`` scales the attention's query and key projections
(softmax close to one-hot, so a single key shows).
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Dict, Optional

import numpy as np
import torch


def lightning(heads, dim, vdim, decay=None):
    decay = decay if decay is not None else [1.0 - 2.0 ** -(2 + 2 * h) for h in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def parallel(heads, kv_heads, dim, vdim, chunk, width, blocks, taps, scale=None, left_scale=1.0, right_scale=1.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if chunk is not None:
        left["mask"] = {"size": chunk}
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": taps},
                                          "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def with_mlp(layer, mlp):
    layer = copy.deepcopy(layer)
    layer["mlp"] = mlp
    return layer


def config(vocab, width, layers, eps=1e-5, scale=None):
    return {"architecture": "Naselorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": math.sqrt(width) if scale is None else scale}, "layers": layers}


# both mixers twice, both feed-forwards; keys of 16 with values of 32 (stored at one size on the bfloat16 path) and
# keys of 24 with values of 8; chunks of 16 (a page) and of 40 (no multiple of a page or a tile); one choice and three
MIXED = config(160, 64, [
    with_mlp(parallel(4, 2, 16, 32, 16, 48, 3, 4, left_scale=1.25, right_scale=0.75), moe(8, 3, 32, shared=48)),
    with_mlp(lightning(2, 16, 24, [0.9, 0.99]), dense(96)),
    with_mlp(parallel(6, 3, 24, 8, 40, 80, 2, 3, scale=0.3, left_scale=0.5, right_scale=1.5), dense(80)),
    with_mlp(lightning(4, 8, 8), moe(6, 1, 40)),
])

# sizes that fit no vector width: a width of 36, seventeen query heads on one key head (more than the split-key kernel
# groups), keys of 12 and values of 7, a chunk of 7, 35 channels in 5 blocks with 2 taps and 18 in one block with one
# tap (no carried inputs), five experts all chosen, forty experts (more than a warp), a layer without a feed-forward,
# an attention without a mask, a decay of exactly one
ODD = config(50, 36, [
    with_mlp(parallel(17, 1, 12, 7, 7, 35, 5, 2, left_scale=2.0, right_scale=-1.0), moe(5, 5, 20, shared=12)),
    with_mlp(lightning(3, 24, 7, [0.5, 0.875, 1.0]), None),
    with_mlp(parallel(2, 2, 10, 10, None, 18, 1, 1), moe(40, 3, 8)),
    with_mlp(lightning(1, 12, 20, [0.96875]), dense(44)),
], eps=1e-6, scale=1.0)

# heads of 64 and of 128 (the tensor-core kernels' sizes), chunks of 160 and of 128, a key size of 136 in the lightning
# mixer (several lanes a column), 256 channels in 2 blocks with 4 taps
WIDE = config(200, 128, [
    with_mlp(parallel(8, 1, 64, 128, 160, 256, 2, 4, scale=0.11, left_scale=0.8, right_scale=1.1), dense(160)),
    with_mlp(lightning(2, 136, 24), moe(12, 4, 48, shared=64)),
    with_mlp(lightning(2, 32, 64), None),
    with_mlp(parallel(8, 4, 64, 64, 128, 64, 8, 5), moe(4, 2, 72, shared=24)),
    with_mlp(lightning(1, 64, 128, [0.999]), dense(96)),
])

CONFIGS = {"mixed": (MIXED, 11), "odd": (ODD, 15), "wide": (WIDE, 13)}


def single_layer(layer, mlp=None, vocab=96, width=48, scale=None):
    """A model of one layer, to look at one mechanism alone."""
    return config(vocab, width, [with_mlp(layer, mlp)], scale=scale)


def _round(values: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.asarray(values, dtype=np.float32)).to(torch.bfloat16)


def make_tensors(raw: dict, seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    rng = np.random.default_rng(seed)
    width, vocab = raw["width"], raw["vocab"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        out[name] = _round(rng.normal(0.0, gain / math.sqrt(cols), size=(rows, cols)))

    def vector(name, size, mean=0.0, std=0.3):
        out[name] = _round(rng.normal(mean, std, size=(size,)))

    def gated(name, inner):
        matrix(name + "gate", inner, width)
        matrix(name + "up", inner, width)
        matrix(name + "down", width, inner)

    out["embed"] = _round(rng.normal(0.0, 1.0 / math.sqrt(width), size=(vocab, width)))
    for index, layer in enumerate(raw["layers"]):
        base = f"l{index}."
        mix, m = base + "mix.", layer["mixer"]
        vector(base + "norm1", width, 0.0, 0.2)
        if layer["type"] == "lightning":
            heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
            matrix(mix + "q", heads * dim, width)
            matrix(mix + "k", heads * dim, width)
            matrix(mix + "v", heads * vdim, width)
            matrix(mix + "g", heads * vdim, width)
            vector(mix + "norm", heads * vdim, 1.0, 0.2)
            matrix(mix + "o", width, heads * vdim)
        else:
            left, right = m["left"], m["right"]
            at = mix + "left."
            heads, groups, dim, vdim = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
            matrix(at + "q", heads * dim, width, gain=sharpen)
            matrix(at + "k", groups * dim, width, gain=sharpen)
            matrix(at + "v", groups * vdim, width)
            matrix(at + "o", width, heads * vdim)
            vector(at + "q.b", heads * dim)
            vector(at + "k.b", groups * dim)
            vector(at + "v.b", groups * vdim)
            vector(at + "o.b", width)
            at = mix + "right."
            channels, blocks, taps = right["width"], right["blocks"], right["conv"]
            part = channels // blocks
            matrix(at + "y", channels, width)
            matrix(at + "x", channels, width)
            vector(at + "y.b", channels)
            vector(at + "x.b", channels)
            out[at + "conv"] = _round(rng.normal(0.0, 0.5, size=(channels, taps)))
            vector(at + "conv.b", channels)
            out[at + "ra"] = _round(rng.normal(0.0, 1.0 / math.sqrt(part), size=(blocks, part, part)))
            out[at + "ri"] = _round(rng.normal(0.0, 1.0 / math.sqrt(part), size=(blocks, part, part)))
            out[at + "ra.b"] = _round(rng.normal(0.0, 0.5, size=(blocks, part)))
            out[at + "ri.b"] = _round(rng.normal(0.0, 0.5, size=(blocks, part)))
            # softplus(lam) from about 0.01 (a channel that forgets over hundreds of tokens) to about 1
            out[at + "lam"] = _round(rng.uniform(-4.5, 0.5, size=(channels,)))
            matrix(at + "o", width, channels)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        vector(base + "norm2", width, 0.0, 0.2)
        name = base + "mlp."
        if mlp["kind"] == "dense":
            gated(name, mlp["ff"])
            continue
        experts = mlp["router"]["experts"]
        matrix(name + "router", experts, width, gain=3.0)
        vector(name + "router.b", experts, 0.0, 0.5)
        for e in range(experts):
            gated(f"{name}e{e}.", mlp["expert"]["ff"])
        if mlp.get("shared") is not None:
            gated(name + "shared.", mlp["shared"]["ff"])
    vector("final.norm", width, 0.0, 0.2)
    matrix("head", vocab, width)
    return out


def write_model(folder: str, raw: dict, seed: int, sharpen: float = 1.0,
                tensors: Optional[Dict[str, torch.Tensor]] = None):
    """Writes ``folder`` and returns (config, {name: bfloat16 tensor})."""
    from safetensors.torch import save_file
    tensors = tensors if tensors is not None else make_tensors(raw, seed, sharpen)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(raw, handle, indent=1)
    save_file({name: value.contiguous() for name, value in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return raw, tensors
