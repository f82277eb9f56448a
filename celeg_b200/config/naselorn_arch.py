"""The Naselorn design as an arrangement of parts.

Token rows are embedding rows times a constant plus a sinusoidal vector of the position (``embedding`` input with
``sinusoid_base``). A block is pre-norm (``prenorm_residual``): x <- x + Mixer(Norm(x)), x <- x + FeedForward(Norm(x)),
the norm an RMSNorm whose stored weight lies around zero (``rmsnorm`` with ``weight_offset`` 1). Mixers:
``lightning_attention`` (a matrix state per head with a fixed decay, SiLU on q, k and v, one RMS norm over all heads, a
sigmoid gate) and ``side_by_side`` of two mixers that read the same rows, their results added with two constants:
``chunked_attention`` (softmax attention without rotation, biases on all four projections, values of another size
than keys, queries limited to the keys of their own chunk of positions) and ``gated_linear_recurrence`` (a gated
linear recurrent unit over channels behind a short causal convolution, block-diagonal gates). Feed-forward: ``swiglu``
with ReLU as the gate's activation, or ``moe`` with SiLU-gated experts, a router with a bias whose largest logits
choose and whose softmax over the chosen logits weighs, and a shared expert. Output: the same kind of norm, an
untied head.

Tensor names: ``embed``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``; a bias is its matrix's name plus ``.b``.
"""
from __future__ import annotations

from typing import Any, Mapping

from .naselorn import DENSE, LIGHTNING, PARALLEL, NaselornConfig, NaselornFeedForward, NaselornLayer
from .registry import Architecture, register_architecture
from .spec import ExecutionEntry, LayerSpec, ModelSpec, PartSpec, TensorRef

SINUSOID_BASE = 10000.0     # the position vector's frequencies are SINUSOID_BASE^(-2i / width)
RECURRENCE_GATE_FACTOR = 8.0    # log a = -RECURRENCE_GATE_FACTOR * r * softplus(lam)


def _offset_norm(name: str, width: int, eps: float) -> PartSpec:
    return PartSpec(kind="rmsnorm", params={"width": width, "eps": eps, "weight_offset": 1.0},
                    tensors={"weight": TensorRef(name, (width,))})


def _mixer(layer: NaselornLayer, base: str, width: int, eps: float) -> PartSpec:
    mix = base + ".mix."
    if layer.type == LIGHTNING:
        qk_width, v_width = layer.heads * layer.dim, layer.heads * layer.vdim
        return PartSpec(
            kind="lightning_attention",
            params={"hidden_size": width, "heads": layer.heads, "dim": layer.dim, "vdim": layer.vdim,
                    "decay": tuple(layer.decay), "eps": eps},
            tensors={"q": TensorRef(mix + "q", (qk_width, width)), "k": TensorRef(mix + "k", (qk_width, width)),
                     "v": TensorRef(mix + "v", (v_width, width)), "gate": TensorRef(mix + "g", (v_width, width)),
                     "norm": TensorRef(mix + "norm", (v_width,)), "out": TensorRef(mix + "o", (width, v_width))})
    if layer.type == PARALLEL:
        left, right = layer.left, layer.right
        at = mix + "left."
        q_width, k_width, v_width = left.heads * left.dim, left.kv_heads * left.dim, left.kv_heads * left.vdim
        attention = PartSpec(
            kind="chunked_attention", category="mixer",
            params={"hidden_size": width, "heads": left.heads, "kv_heads": left.kv_heads, "dim": left.dim,
                    "vdim": left.vdim, "scale": left.scale, "chunk": left.chunk},
            tensors={"q": TensorRef(at + "q", (q_width, width)), "q_bias": TensorRef(at + "q.b", (q_width,)),
                     "k": TensorRef(at + "k", (k_width, width)), "k_bias": TensorRef(at + "k.b", (k_width,)),
                     "v": TensorRef(at + "v", (v_width, width)), "v_bias": TensorRef(at + "v.b", (v_width,)),
                     "out": TensorRef(at + "o", (width, left.heads * left.vdim)),
                     "out_bias": TensorRef(at + "o.b", (width,))})
        at = mix + "right."
        part = right.width // right.blocks
        recurrence = PartSpec(
            kind="gated_linear_recurrence", category="mixer",
            params={"hidden_size": width, "width": right.width, "blocks": right.blocks, "taps": right.taps,
                    "gate_factor": RECURRENCE_GATE_FACTOR},
            tensors={"y": TensorRef(at + "y", (right.width, width)), "y_bias": TensorRef(at + "y.b", (right.width,)),
                     "x": TensorRef(at + "x", (right.width, width)), "x_bias": TensorRef(at + "x.b", (right.width,)),
                     "conv": TensorRef(at + "conv", (right.width, right.taps)),
                     "conv_bias": TensorRef(at + "conv.b", (right.width,)),
                     "recurrence_gate": TensorRef(at + "ra", (right.blocks, part, part)),
                     "recurrence_gate_bias": TensorRef(at + "ra.b", (right.blocks, part)),
                     "input_gate": TensorRef(at + "ri", (right.blocks, part, part)),
                     "input_gate_bias": TensorRef(at + "ri.b", (right.blocks, part)),
                     "lam": TensorRef(at + "lam", (right.width,)),
                     "out": TensorRef(at + "o", (width, right.width))})
        return PartSpec(kind="side_by_side", params={"hidden_size": width, "left_scale": layer.left_scale,
                                                     "right_scale": layer.right_scale},
                        parts={"left": attention, "right": recurrence})
    raise AssertionError(layer.type)


def _gated(name: str, width: int, inner: int, activation: str) -> PartSpec:
    return PartSpec(kind="swiglu", category="feed_forward",
                    params={"hidden_size": width, "intermediate_size": inner, "activation": activation},
                    tensors={"gate": TensorRef(name + "gate", (inner, width)), "up": TensorRef(name + "up", (inner, width)),
                             "down": TensorRef(name + "down", (width, inner))})


def _feed_forward(mlp: NaselornFeedForward, base: str, width: int) -> PartSpec:
    name = base + ".mlp."
    if mlp.kind == DENSE:
        return _gated(name, width, mlp.ff, "relu")
    tensors = {"router": TensorRef(name + "router", (mlp.experts, width)),
               "router_bias": TensorRef(name + "router.b", (mlp.experts,))}
    for expert in range(mlp.experts):
        tensors[f"e{expert}.gate"] = TensorRef(f"{name}e{expert}.gate", (mlp.ff, width))
        tensors[f"e{expert}.up"] = TensorRef(f"{name}e{expert}.up", (mlp.ff, width))
        tensors[f"e{expert}.down"] = TensorRef(f"{name}e{expert}.down", (width, mlp.ff))
    parts = {}
    if mlp.shared_ff is not None:
        parts["shared"] = _gated(name + "shared.", width, mlp.shared_ff, "silu")
    return PartSpec(kind="moe", params={"hidden_size": width, "intermediate_size": mlp.ff, "experts": mlp.experts,
                                        "top": mlp.top, "activation": "silu", "gated_experts": True},
                    tensors=tensors, parts=parts)


def build_naselorn_spec(config: NaselornConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    layers = []
    for index, layer in enumerate(config.layers):
        base = f"l{index}"
        has_ff = layer.mlp is not None
        layers.append(LayerSpec(name=base, arrangement="prenorm_residual",
                                mixer_norm=_offset_norm(base + ".norm1", width, eps),
                                mixer=_mixer(layer, base, width, eps),
                                feed_forward_norm=_offset_norm(base + ".norm2", width, eps) if has_ff else None,
                                feed_forward=_feed_forward(layer.mlp, base, width) if has_ff else None))
    table = TensorRef("embed", (config.vocab, width))
    spec = ModelSpec(
        architecture=config.model_type, vocab_size=config.vocab, hidden_size=width, max_context=config.max_context,
        embedding=table, layers=tuple(layers),
        order=tuple(ExecutionEntry(layer=index) for index in range(len(layers))),
        final_norm=_offset_norm("final.norm", width, eps), lm_head=TensorRef("head", (config.vocab, width)),
        eos_token_ids=tuple(config.eos_token_ids), bos_token_id=config.bos_token_id,
        input=PartSpec("embedding", params={"multiplier": config.embedding_scale, "sinusoid_base": SINUSOID_BASE},
                       tensors={"table": table}, category="input"))
    spec.validate()
    return spec


def naselorn_random_init(config: NaselornConfig, name: str, shape: tuple) -> str:
    """Distribution of a tensor in random-weights mode: matrices N(0, 1/fan-in), the norms' stored weights and every
    bias small around zero, the plain norm weight of the lightning mixer around 1, convolution taps N(0, 0.5), the
    recurrence's ``lam`` N(0, 0.3)."""
    leaf = name.rsplit(".", 1)[-1]
    if leaf == "conv":
        return "taps"
    if leaf == "lam":
        return "small"
    if leaf == "norm" and ".mix." in name:
        return "norm"
    if leaf == "b" or len(shape) == 1:
        return "tiny"
    return "fan_in"


def _parse(raw: Mapping[str, Any]) -> NaselornConfig:
    return NaselornConfig.from_dict(raw)


def _resolve(config: NaselornConfig, tensor_shapes: Mapping[str, Any]) -> NaselornConfig:
    return config


NASELORN = Architecture(name="Naselorn", parse_config=_parse, resolve_config=_resolve,
                        build_spec=build_naselorn_spec, random_init=naselorn_random_init)
register_architecture(NASELORN, replace=True)
