"""Typed configurations and the registry of architectures."""
from .dense import ConfigError, DenseDecoderConfig, RopeScaling, read_config_json
from .karitar import KaritarConfig, karitar_spec
from .registry import (Architecture, architecture_name, architecture_of, dense_decoder_spec, known_architectures,
                       register_architecture)

__all__ = ["ConfigError", "DenseDecoderConfig", "RopeScaling", "read_config_json", "Architecture", "KaritarConfig",
           "karitar_spec", "architecture_name", "architecture_of", "dense_decoder_spec", "known_architectures", "register_architecture"]
