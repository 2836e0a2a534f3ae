from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec
from .registry import (architecture_name, config_from_dict, known_architectures, load_config,
                       register_architecture)
from .gpt2 import GPT2Config
from .vekedra import VekedraConfig
from .figotar import FigotarConfig
from .vatevik import VatevikConfig
from .divitar import DivitarConfig

for _name in ("GPT2LMHeadModel", "TinyGPT", "gpt2"):
    register_architecture(_name, GPT2Config)
register_architecture("Vekedra", VekedraConfig)
register_architecture("Figotar", FigotarConfig)
register_architecture("Vatevik", VatevikConfig)
register_architecture("Divitar", DivitarConfig)

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "GPT2Config", "VekedraConfig", "FigotarConfig", "VatevikConfig", "DivitarConfig", "architecture_name",
           "config_from_dict", "known_architectures", "load_config", "register_architecture"]
