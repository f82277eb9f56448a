"""Typed configuration of the Liverax design, read from config.json (``"architecture": "Liverax"``).

Keys: ``vocab``, ``width``, ``norm.eps``, ``logit_softcap`` (absent: logits are not capped), ``layers`` (a list; each
entry has ``type`` = attention | attention_2 | latent_attention, the mixer's sizes and constants under ``mixer``, and
``mlp`` = {kind: dense, ff} | null).
attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` = {base, dims, scaling: {factor} or absent},
``mask`` = {size} or absent, ``v_mix``. attention_2: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``bias_max``, ``q_temp`` = {coef, every} or absent, ``v_mix``. latent_attention: ``heads``, ``dim``, ``rot_dim``,
``vdim``, ``kv_rank``, ``q_rank``, ``scale``, ``rot`` = {base, ...}, ``mask`` = {size} or absent. Every size and every
constant that can differ between two models of the design comes from here, or from a tensor's shape where
config.json is silent (the number of distance buckets).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .ramosun import DEFAULT_MAX_CONTEXT, _need


def _positive_int(mapping: Mapping[str, Any], key: str, where: str) -> int:
    """A count; a JSON writer may have left a whole number as 64.0."""
    value = _need(mapping, key, where)
    if isinstance(value, float) and value.is_integer():
        value = int(value)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"{where}: '{key}' must be a positive integer, got {value!r}")
    return value

ATTENTION, DISTANCE_ATTENTION, LATENT_ATTENTION = "attention", "attention_2", "latent_attention"
LAYER_TYPES = (ATTENTION, DISTANCE_ATTENTION, LATENT_ATTENTION)


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    divide_by: float = 1.0          # every frequency is divided by this ("linear" scaling of positions)

    @staticmethod
    def from_dict(raw: Mapping[str, Any], where: str, dims: Optional[int] = None) -> "RotationConfig":
        base = float(_need(raw, "base", where))
        if base <= 1.0:
            raise ConfigError(f"{where}: a rotation base of {base}")
        found = _positive_int(raw, "dims", where) if raw.get("dims") is not None else dims
        if found is None or found % 2:
            raise ConfigError(f"{where}: 'dims' must be an even number, got {found!r}")
        if dims is not None and found != dims:
            raise ConfigError(f"{where}: {found} rotated dimensions where the mixer has {dims}")
        scaling = raw.get("scaling")
        divide_by = float(_need(scaling, "factor", where + ".scaling")) if scaling else 1.0
        if divide_by <= 0:
            raise ConfigError(f"{where}.scaling: a factor of {divide_by}")
        return RotationConfig(base=base, dims=found, divide_by=divide_by)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.divide_by != 1.0:
            out["scaling"] = {"factor": self.divide_by}
        return out


def _window(mixer: Mapping[str, Any], where: str) -> Optional[int]:
    mask = mixer.get("mask")
    return None if mask is None else _positive_int(mask, "size", where + ".mask")


@dataclass(frozen=True)
class LiveraxLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    scale: float
    ff: Optional[int] = None                      # None: the layer has no feed-forward
    kv_heads: int = 0                             # attention, attention_2
    value_mix: bool = False
    rotation: Optional[RotationConfig] = None     # attention, latent_attention
    window: Optional[int] = None
    distance_far: int = 0                         # attention_2
    temperature: Optional[Tuple[float, int]] = None
    rot_dim: int = 0                              # latent_attention
    kv_rank: int = 0
    q_rank: int = 0

    @staticmethod
    def from_dict(raw: Mapping[str, Any], index: int) -> "LiveraxLayer":
        where = f"layers[{index}]"
        kind = _need(raw, "type", where)
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {', '.join(LAYER_TYPES)}")
        mixer = _need(raw, "mixer", where)
        at = where + ".mixer"
        mlp = raw.get("mlp")
        ff = None
        if mlp is not None:
            if mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"{where}.mlp: unknown kind {mlp.get('kind')!r}; known: dense")
            ff = _positive_int(mlp, "ff", where + ".mlp")
        heads = _positive_int(mixer, "heads", at)
        dim = _positive_int(mixer, "dim", at)
        vdim = _positive_int(mixer, "vdim", at) if mixer.get("vdim") is not None else dim
        # (a configuration that leaves the scale out gets one over the root of a key's size)
        key_size = dim + (_positive_int(mixer, "rot_dim", at) if kind == LATENT_ATTENTION else 0)
        scale = float(mixer["scale"]) if mixer.get("scale") is not None else key_size ** -0.5
        common = dict(type=kind, heads=heads, dim=dim, vdim=vdim, scale=scale, ff=ff)
        if kind == LATENT_ATTENTION:
            rot_dim = _positive_int(mixer, "rot_dim", at)
            return LiveraxLayer(**common, rot_dim=rot_dim, kv_rank=_positive_int(mixer, "kv_rank", at),
                                q_rank=_positive_int(mixer, "q_rank", at),
                                rotation=RotationConfig.from_dict(_need(mixer, "rot", at), at + ".rot", dims=rot_dim),
                                window=_window(mixer, at))
        kv_heads = _positive_int(mixer, "kv_heads", at) if mixer.get("kv_heads") is not None else heads
        if heads % kv_heads:
            raise ConfigError(f"{at}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        common.update(kv_heads=kv_heads, value_mix=bool(mixer.get("v_mix", False)))
        if kind == ATTENTION:
            rotation = mixer.get("rot")
            rotation = None if rotation is None else RotationConfig.from_dict(rotation, at + ".rot")
            if rotation is not None and rotation.dims > dim:
                raise ConfigError(f"{at}.rot: {rotation.dims} rotated dimensions of a head of {dim}")
            return LiveraxLayer(**common, rotation=rotation, window=_window(mixer, at))
        temperature = mixer.get("q_temp")
        if temperature is not None:
            temperature = (float(_need(temperature, "coef", at + ".q_temp")), _positive_int(temperature, "every", at + ".q_temp"))
        return LiveraxLayer(**common, distance_far=_positive_int(mixer, "bias_max", at), temperature=temperature,
                            window=_window(mixer, at))

    def to_dict(self) -> Dict[str, Any]:
        mixer: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            mixer["mask"] = {"size": self.window}
        if self.type == LATENT_ATTENTION:
            mixer.update(rot_dim=self.rot_dim, kv_rank=self.kv_rank, q_rank=self.q_rank, rot=self.rotation.to_dict())
        else:
            mixer.update(kv_heads=self.kv_heads, v_mix=self.value_mix)
            if self.type == ATTENTION and self.rotation is not None:
                mixer["rot"] = self.rotation.to_dict()
            if self.type == DISTANCE_ATTENTION:
                mixer["bias_max"] = self.distance_far
                if self.temperature is not None:
                    mixer["q_temp"] = {"coef": self.temperature[0], "every": self.temperature[1]}
        return {"type": self.type, "mixer": mixer, "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class LiveraxConfig:
    vocab: int
    width: int
    layers: Tuple[LiveraxLayer, ...]
    norm_eps: float
    logit_softcap: Optional[float] = None
    distance_buckets: Tuple[int, ...] = ()         # per layer, 0 where the layer has no table; from tensor shapes
    max_context: int = DEFAULT_MAX_CONTEXT
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    model_type: str = "Liverax"

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "LiveraxConfig":
        layers_raw = _need(raw, "layers", "config.json")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        eos = raw.get("eos_token_id")
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (() if eos is None else (int(eos),))
        context = raw.get("max_context")
        eps = float(_need(_need(raw, "norm", "config.json"), "eps", "norm"))
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        cap = raw.get("logit_softcap")
        if cap is not None and float(cap) <= 0:
            raise ConfigError(f"logit_softcap must be positive, got {cap}")
        layers = tuple(LiveraxLayer.from_dict(layer, index) for index, layer in enumerate(layers_raw))
        mixed = [layer for layer in layers if layer.value_mix]
        for layer in mixed[1:]:
            if (layer.kv_heads, layer.vdim) != (mixed[0].kv_heads, mixed[0].vdim):
                raise ConfigError(f"layers that blend their values need values of one shape: {layer.kv_heads} x "
                                  f"{layer.vdim} beside {mixed[0].kv_heads} x {mixed[0].vdim}")
        buckets = raw.get("distance_buckets")
        return LiveraxConfig(
            vocab=_positive_int(raw, "vocab", "config.json"), width=_positive_int(raw, "width", "config.json"),
            layers=layers, norm_eps=eps, logit_softcap=None if cap is None else float(cap),
            distance_buckets=tuple(int(b) for b in buckets) if buckets else (),
            max_context=DEFAULT_MAX_CONTEXT if context is None else int(context), eos_token_ids=eos_ids,
            bos_token_id=None if raw.get("bos_token_id") is None else int(raw["bos_token_id"]))

    def buckets_of(self, index: int) -> int:
        """Rows of layer ``index``'s distance table (known once the checkpoint's shapes were read, or from the
        configuration of a model that is yet to be written)."""
        return self.distance_buckets[index] if index < len(self.distance_buckets) else 0

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.model_type, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers], "max_context": self.max_context}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if any(self.distance_buckets):
            out["distance_buckets"] = list(self.distance_buckets)
        return out


__all__ = ["ATTENTION", "DISTANCE_ATTENTION", "LATENT_ATTENTION", "RotationConfig", "LiveraxLayer", "LiveraxConfig"]
