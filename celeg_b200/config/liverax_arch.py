"""The Liverax design as an arrangement of parts.

A block is pre-norm (``prenorm_residual``): x <- x + Mixer(Norm(x)), x <- x + FeedForward(Norm(x)), the norm a layer
norm with a weight and no bias (``layernorm``). Three mixers, all softmax attention over the paged cache:

* ``attention``: ``prepared_attention`` with a rotation of pairs (i, i + half) whose frequencies may be divided by a
  constant (``rope_split_half`` with ``linear_factor``) and a window;
* ``attention_2``: ``prepared_attention`` with biases on q, k and v, RMS norms over the whole q and the whole k
  projection, a query factor that grows with the logarithm of the position, a learned bias per head and distance
  bucket, every earlier position visible, and a sigmoid gate per element on the heads' results;
* ``latent_attention``: the latent mixer with queries through a normed latent of their own, pairs (i, i + half) in the
  rotated part, a window, a sink per head and a gate per element.

Layers marked for it blend their values with those the first marked layer made of the same token (``value_mix``).
Feed-forward: ``swiglu`` with the tanh form of GELU on the gate. Output: the same kind of norm, an untied head, logits
capped smoothly.

Tensor names: ``embed``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``; a bias is its matrix's name plus ``.b``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping

from .errors import ConfigError
from .liverax import ATTENTION, DISTANCE_ATTENTION, LATENT_ATTENTION, LiveraxConfig, LiveraxLayer
from .registry import Architecture, register_architecture
from .spec import ExecutionEntry, LayerSpec, ModelSpec, PartSpec, TensorRef


def _norm(name: str, width: int, eps: float) -> PartSpec:
    return PartSpec(kind="layernorm", params={"width": width, "eps": eps}, tensors={"weight": TensorRef(name, (width,))})


def _rotation(layer: LiveraxLayer, head_dim: int) -> PartSpec:
    rotation = layer.rotation
    return PartSpec(kind="rope_split_half", category="position",
                    params={"theta": rotation.base, "head_dim": head_dim, "rotary_dim": rotation.dims,
                            "linear_factor": rotation.divide_by})


def _mixer(config: LiveraxConfig, index: int, first_mixed: int, width: int) -> PartSpec:
    layer = config.layers[index]
    mix = f"l{index}.mix."
    eps = config.norm_eps
    if layer.type == LATENT_ATTENTION:
        q_width, rot = layer.heads * (layer.dim + layer.rot_dim), layer.rot_dim
        return PartSpec(
            kind="latent_attention",
            params={"hidden_size": width, "heads": layer.heads, "dim": layer.dim, "rot_dim": rot, "vdim": layer.vdim,
                    "kv_rank": layer.kv_rank, "scale": layer.scale, "eps": eps, "window": layer.window,
                    "gate_per_element": True},
            tensors={"q_down": TensorRef(mix + "dq", (layer.q_rank, width)),
                     "q_down_norm": TensorRef(mix + "dq.norm", (layer.q_rank,)),
                     "q": TensorRef(mix + "uq", (q_width, layer.q_rank)),
                     "down": TensorRef(mix + "dkv", (layer.kv_rank + rot, width)),
                     "down_norm": TensorRef(mix + "dkv.norm", (layer.kv_rank,)),
                     "up_keys": TensorRef(mix + "uk", (layer.heads * layer.dim, layer.kv_rank)),
                     "up_values": TensorRef(mix + "uv", (layer.heads * layer.vdim, layer.kv_rank)),
                     "sinks": TensorRef(mix + "sink", (layer.heads,)),
                     "gate": TensorRef(mix + "g", (layer.heads * layer.vdim, width)),
                     "out": TensorRef(mix + "o", (width, layer.heads * layer.vdim))},
            parts={"position": _rotation(layer, rot)})
    q_width, k_width, v_width = layer.heads * layer.dim, layer.kv_heads * layer.dim, layer.kv_heads * layer.vdim
    params = {"hidden_size": width, "heads": layer.heads, "kv_heads": layer.kv_heads, "dim": layer.dim,
              "vdim": layer.vdim, "scale": layer.scale, "window": layer.window}
    tensors = {"q": TensorRef(mix + "q", (q_width, width)), "k": TensorRef(mix + "k", (k_width, width)),
               "v": TensorRef(mix + "v", (v_width, width)), "out": TensorRef(mix + "o", (width, layer.heads * layer.vdim))}
    if layer.value_mix:
        params["value_mix"] = "first" if index == first_mixed else "blend"
        # (the first marked layer stores the number too and never reads it)
        tensors["value_mix"] = TensorRef(mix + "vmix", ())
    parts = {}
    if layer.type == ATTENTION:
        if layer.rotation is not None:
            parts["position"] = _rotation(layer, layer.dim)
        return PartSpec(kind="prepared_attention", params=params, tensors=tensors, parts=parts)
    assert layer.type == DISTANCE_ATTENTION
    buckets = config.buckets_of(index)
    if buckets < 2:
        raise ConfigError(f"layers[{index}]: the distance table's rows are unknown (the checkpoint gives them as the shape "
                          f"of {mix}rel; a configuration without one names them under 'distance_buckets')")
    params.update(whole_qk_norm=True, eps=eps, distance_far=layer.distance_far, output_gate=True)
    if layer.temperature is not None:
        params["temperature"] = {"coef": layer.temperature[0], "every": layer.temperature[1]}
    tensors.update({"q_bias": TensorRef(mix + "q.b", (q_width,)), "k_bias": TensorRef(mix + "k.b", (k_width,)),
                    "v_bias": TensorRef(mix + "v.b", (v_width,)), "q_norm": TensorRef(mix + "q.norm", (q_width,)),
                    "k_norm": TensorRef(mix + "k.norm", (k_width,)),
                    "distance_table": TensorRef(mix + "rel", (buckets, layer.heads)),
                    "gate": TensorRef(mix + "g", (layer.heads * layer.vdim, width))})
    return PartSpec(kind="prepared_attention", params=params, tensors=tensors)


def _feed_forward(base: str, width: int, inner: int) -> PartSpec:
    name = base + ".mlp."
    return PartSpec(kind="swiglu", params={"hidden_size": width, "intermediate_size": inner, "activation": "gelu_tanh"},
                    tensors={"gate": TensorRef(name + "gate", (inner, width)), "up": TensorRef(name + "up", (inner, width)),
                             "down": TensorRef(name + "down", (width, inner))})


def build_liverax_spec(config: LiveraxConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    mixed = [index for index, layer in enumerate(config.layers) if layer.value_mix]
    first_mixed = mixed[0] if mixed else -1
    layers = []
    for index, layer in enumerate(config.layers):
        base = f"l{index}"
        has_ff = layer.ff is not None
        layers.append(LayerSpec(name=base, arrangement="prenorm_residual",
                                mixer_norm=_norm(base + ".norm1", width, eps),
                                mixer=_mixer(config, index, first_mixed, width),
                                feed_forward_norm=_norm(base + ".norm2", width, eps) if has_ff else None,
                                feed_forward=_feed_forward(base, width, layer.ff) if has_ff else None))
    spec = ModelSpec(
        architecture=config.model_type, vocab_size=config.vocab, hidden_size=width, max_context=config.max_context,
        embedding=TensorRef("embed", (config.vocab, width)), layers=tuple(layers),
        order=tuple(ExecutionEntry(layer=index) for index in range(len(layers))),
        final_norm=_norm("final.norm", width, eps), lm_head=TensorRef("head", (config.vocab, width)),
        eos_token_ids=tuple(config.eos_token_ids), bos_token_id=config.bos_token_id,
        logit_softcap=config.logit_softcap)
    spec.validate()
    return spec


def liverax_random_init(config: LiveraxConfig, name: str, shape: tuple) -> str:
    """Distribution of a tensor in random-weights mode: matrices N(0, 1/fan-in), norm weights around 1, biases, sinks,
    distance tables and the blending numbers small."""
    leaf = name.rsplit(".", 1)[-1]
    if leaf in ("norm", "norm1", "norm2"):
        return "norm"
    if leaf in ("rel", "sink", "vmix"):
        return "small"
    if leaf == "b" or len(shape) == 1:
        return "tiny"
    return "fan_in"


def _parse(raw: Mapping[str, Any]) -> LiveraxConfig:
    return LiveraxConfig.from_dict(raw)


def _resolve(config: LiveraxConfig, tensor_shapes: Mapping[str, Any]) -> LiveraxConfig:
    """The number of distance buckets of every ``attention_2`` layer is the row count of its stored table."""
    buckets = []
    for index, layer in enumerate(config.layers):
        shape = tensor_shapes.get(f"l{index}.mix.rel")
        if layer.type == DISTANCE_ATTENTION and shape is not None:
            if len(shape) != 2:
                raise ConfigError(f"l{index}.mix.rel has shape {tuple(shape)}, expected (buckets, {layer.heads})")
            buckets.append(int(shape[0]))
        else:
            buckets.append(config.buckets_of(index))
    return dataclasses.replace(config, distance_buckets=tuple(buckets))


LIVERAX = Architecture(name="Liverax", parse_config=_parse, resolve_config=_resolve,
                       build_spec=build_liverax_spec, random_init=liverax_random_init)
register_architecture(LIVERAX, replace=True)
