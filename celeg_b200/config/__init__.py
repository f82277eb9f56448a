"""Typed configuration, the model description data, and the architecture registry."""
from .errors import ConfigError, UnknownArchitectureError
from .spec import ExecutionEntry, LayerSpec, ModelSpec, PartSpec, TensorRef
from .registry import (Architecture, architecture_named, architecture_of, known_architectures,
                       read_config_json, register_architecture)
from .lfm2 import CONV, FULL_ATTENTION, Lfm2Config
from . import lfm2_arch as _lfm2_arch  # registers "lfm2"
from .lfm2_arch import build_lfm2_spec
from .ramosun import RamosunConfig
from . import ramosun_arch as _ramosun_arch  # registers "Ramosun"
from .ramosun_arch import build_ramosun_spec
from .kedesun import KedesunConfig
from . import kedesun_arch as _kedesun_arch  # registers "Kedesun"
from .kedesun_arch import build_kedesun_spec
from .naselorn import NaselornConfig
from . import naselorn_arch as _naselorn_arch  # registers "Naselorn"
from .naselorn_arch import build_naselorn_spec
from .liverax import LiveraxConfig
from . import liverax_arch as _liverax_arch  # registers "Liverax"
from .liverax_arch import build_liverax_spec

__all__ = [
    "Architecture", "ConfigError", "UnknownArchitectureError", "ExecutionEntry", "LayerSpec",
    "ModelSpec", "PartSpec", "TensorRef", "architecture_named", "architecture_of",
    "known_architectures", "read_config_json", "register_architecture", "CONV",
    "FULL_ATTENTION", "Lfm2Config", "build_lfm2_spec", "RamosunConfig", "build_ramosun_spec",
    "KedesunConfig", "build_kedesun_spec", "NaselornConfig", "build_naselorn_spec",
    "LiveraxConfig", "build_liverax_spec",
]
