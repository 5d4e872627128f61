from .registry import (Architecture, ConfigError, load_config, read_config_json, register_architecture,
                       registered_architectures, resolve_architecture)
from .specs import LayerSpec, ModelSpec, PartSpec, Run
from .llama import LlamaConfig, RopeScaling, build_llama_spec
from .debonex import DebonexConfig, build_debonex_spec
from .dilalix import DilalixConfig, build_dilalix_spec
from .nazerax import NazeraxConfig, build_nazerax_spec
from .fomodra import FomodraConfig, build_fomodra_spec

__all__ = ["Architecture", "ConfigError", "load_config", "read_config_json", "register_architecture",
           "registered_architectures", "resolve_architecture", "LayerSpec", "ModelSpec", "PartSpec", "Run",
           "LlamaConfig", "RopeScaling", "build_llama_spec", "DebonexConfig", "build_debonex_spec",
           "DilalixConfig", "build_dilalix_spec", "NazeraxConfig", "build_nazerax_spec", "FomodraConfig", "build_fomodra_spec"]
