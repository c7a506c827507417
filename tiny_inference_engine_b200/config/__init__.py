"""Typed configurations, the model description they turn into, and the architecture registry."""
from .registry import (Architecture, architectures, load_config, read_config_json, register_architecture,
                       resolve_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .qwen3 import Qwen3Config, parse_qwen3_config, qwen3_spec
from .dugazen import DugazenConfig, dugazen_spec, parse_dugazen_config
from .misudra import MisudraConfig, misudra_spec, parse_misudra_config
from .lufatar import LufatarConfig, lufatar_spec, parse_lufatar_config
from .subivik import SubivikConfig, parse_subivik_config, subivik_spec

__all__ = ["Architecture", "architectures", "load_config", "read_config_json", "register_architecture",
           "resolve_architecture", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config",
           "parse_qwen3_config", "qwen3_spec", "DugazenConfig", "dugazen_spec", "parse_dugazen_config", "MisudraConfig",
           "misudra_spec", "parse_misudra_config", "LufatarConfig", "lufatar_spec", "parse_lufatar_config",
           "SubivikConfig", "parse_subivik_config", "subivik_spec"]
