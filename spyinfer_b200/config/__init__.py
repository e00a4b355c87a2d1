"""Typed configuration: the architecture registry, the model description and the engine's options."""
from .engine_config import EngineConfig
from .model_config import (ArchitectureConfig, ConfigError, config_from_json, known_architectures, load_model_config,
                           register_architecture)
from .spec import CompositeCacheNeed, LayerSpec, ModelSpec, PagedCacheNeed, PartSpec, RunEntry, SharedCacheNeed, StateCacheNeed, StreamAdd
from . import qwen3 as _qwen3  # registers "Qwen3ForCausalLM"
from . import nezolorn as _nezolorn  # registers "Nezolorn"
from . import daronex as _daronex  # registers "Daronex"
from . import naforax as _naforax  # registers "Naforax"
from . import dogilorn as _dogilorn  # registers "Dogilorn"
from .daronex import DaronexConfig
from .dogilorn import DogilornConfig
from .naforax import NaforaxConfig
from .nezolorn import NezolornConfig
from .qwen3 import Qwen3Config

__all__ = ["EngineConfig", "ArchitectureConfig", "ConfigError", "config_from_json", "known_architectures",
           "load_model_config", "register_architecture", "LayerSpec", "ModelSpec", "PagedCacheNeed", "PartSpec",
           "RunEntry", "StateCacheNeed", "CompositeCacheNeed", "Qwen3Config", "NezolornConfig", "DaronexConfig", "NaforaxConfig", "DogilornConfig", "StreamAdd"]
