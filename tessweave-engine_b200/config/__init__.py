"""Typed configuration of model and engine, and the architecture registry."""
from .model_config import ConfigError, Qwen2Config
from .linurax_config import LinuraxConfig
from .sapatar_config import SapatarConfig
from .nufatar_config import NufatarConfig
from .dugudra_config import DugudraConfig
from .engine_config import EngineConfig
from .registry import architecture_of, architectures, register_architecture, resolve, resolve_folder

__all__ = ["ConfigError", "Qwen2Config", "LinuraxConfig", "SapatarConfig", "NufatarConfig", "EngineConfig", "architecture_of", "architectures",
           "register_architecture", "resolve", "resolve_folder"]
