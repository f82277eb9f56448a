"""Typed configuration of the Naselorn design, read from config.json (``"architecture": "Naselorn"``).

Keys: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``layers`` (a list; each entry has ``type`` =
lightning | parallel, the mixer's sizes and constants under ``mixer``, and ``mlp`` = {kind: dense, ff} |
{kind: moe, router: {experts, top}, expert: {ff}, shared: {ff} or absent} | null).
Lightning: ``heads``, ``dim``, ``vdim``, ``decay`` (one number a head). Parallel: ``left`` = {heads, kv_heads, dim,
vdim, scale, mask: {size} or absent}, ``right`` = {width, blocks, conv}, ``left_scale``, ``right_scale``. Every size and
every constant that can differ between two models of the design comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .kedesun import DENSE, MOE, KedesunFeedForward
from .ramosun import DEFAULT_MAX_CONTEXT, _need, _positive_int

LIGHTNING, PARALLEL = "lightning", "parallel"

# the feed-forward's description has the same keys as the Kedesun design's (kind, ff, router, expert, shared)
NaselornFeedForward = KedesunFeedForward


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int] = None                # None: every earlier position is visible

    @staticmethod
    def from_dict(raw: Mapping[str, Any], where: str) -> "ChunkedAttentionConfig":
        heads = _positive_int(raw, "heads", where)
        kv_heads = _positive_int(raw, "kv_heads", where) if raw.get("kv_heads") is not None else heads
        if heads % kv_heads:
            raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        dim = _positive_int(raw, "dim", where)
        mask = raw.get("mask")
        chunk = None if mask is None else _positive_int(mask, "size", where + ".mask")
        scale = float(raw["scale"]) if raw.get("scale") is not None else dim ** -0.5
        vdim = _positive_int(raw, "vdim", where) if raw.get("vdim") is not None else dim
        return ChunkedAttentionConfig(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, chunk=chunk)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        return out


@dataclass(frozen=True)
class RecurrentUnitConfig:
    width: int
    blocks: int
    taps: int

    @staticmethod
    def from_dict(raw: Mapping[str, Any], where: str) -> "RecurrentUnitConfig":
        width = _positive_int(raw, "width", where)
        blocks = _positive_int(raw, "blocks", where)
        if width % blocks:
            raise ConfigError(f"{where}: a width of {width} is not a multiple of {blocks} blocks")
        taps = _positive_int(raw, "conv", where)
        if taps > 16:
            raise ConfigError(f"{where}: {taps} taps exceed 16")
        return RecurrentUnitConfig(width=width, blocks=blocks, taps=taps)

    def to_dict(self) -> Dict[str, Any]:
        return {"width": self.width, "blocks": self.blocks, "conv": self.taps}


@dataclass(frozen=True)
class NaselornLayer:
    type: str
    mlp: Optional[NaselornFeedForward] = None
    heads: int = 0                                 # lightning
    dim: int = 0
    vdim: int = 0
    decay: Tuple[float, ...] = ()
    left: Optional[ChunkedAttentionConfig] = None  # parallel
    right: Optional[RecurrentUnitConfig] = None
    left_scale: float = 1.0
    right_scale: float = 1.0

    @staticmethod
    def from_dict(raw: Mapping[str, Any], index: int) -> "NaselornLayer":
        where = f"layers[{index}]"
        kind = _need(raw, "type", where)
        if kind not in (LIGHTNING, PARALLEL):
            raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {LIGHTNING}, {PARALLEL}")
        mixer = _need(raw, "mixer", where)
        where_mixer = where + ".mixer"
        mlp = raw.get("mlp")
        mlp = None if mlp is None else NaselornFeedForward.from_dict(mlp, where + ".mlp")
        if kind == LIGHTNING:
            heads = _positive_int(mixer, "heads", where_mixer)
            decay = _need(mixer, "decay", where_mixer)
            if not isinstance(decay, (list, tuple)) or len(decay) != heads:
                raise ConfigError(f"{where_mixer}: 'decay' must list one number for each of the {heads} heads")
            return NaselornLayer(type=kind, mlp=mlp, heads=heads, dim=_positive_int(mixer, "dim", where_mixer),
                                 vdim=_positive_int(mixer, "vdim", where_mixer), decay=tuple(float(d) for d in decay))
        return NaselornLayer(
            type=kind, mlp=mlp,
            left=ChunkedAttentionConfig.from_dict(_need(mixer, "left", where_mixer), where_mixer + ".left"),
            right=RecurrentUnitConfig.from_dict(_need(mixer, "right", where_mixer), where_mixer + ".right"),
            left_scale=float(mixer.get("left_scale", 1.0)), right_scale=float(mixer.get("right_scale", 1.0)))

    def to_dict(self) -> Dict[str, Any]:
        if self.type == LIGHTNING:
            mixer: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        else:
            mixer = {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                     "right_scale": self.right_scale}
        return {"type": self.type, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class NaselornConfig:
    vocab: int
    width: int
    layers: Tuple[NaselornLayer, ...]
    norm_eps: float
    embedding_scale: float = 1.0
    max_context: int = DEFAULT_MAX_CONTEXT
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    model_type: str = "Naselorn"

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "NaselornConfig":
        layers_raw = _need(raw, "layers", "config.json")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        eos = raw.get("eos_token_id")
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (() if eos is None else (int(eos),))
        context = raw.get("max_context")
        eps = float(_need(_need(raw, "norm", "config.json"), "eps", "norm"))
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        embedding = raw.get("embedding") or {}
        return NaselornConfig(
            vocab=_positive_int(raw, "vocab", "config.json"), width=_positive_int(raw, "width", "config.json"),
            layers=tuple(NaselornLayer.from_dict(layer, index) for index, layer in enumerate(layers_raw)),
            norm_eps=eps, embedding_scale=float(embedding.get("scale", 1.0)),
            max_context=DEFAULT_MAX_CONTEXT if context is None else int(context), eos_token_ids=eos_ids,
            bos_token_id=None if raw.get("bos_token_id") is None else int(raw["bos_token_id"]))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.model_type, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": [layer.to_dict() for layer in self.layers], "max_context": self.max_context}


__all__ = ["DENSE", "MOE", "LIGHTNING", "PARALLEL", "ChunkedAttentionConfig", "RecurrentUnitConfig",
           "NaselornFeedForward", "NaselornLayer", "NaselornConfig"]
