"""Typed configurations and the architecture registry."""

from .llama import LlamaConfig
from .nilevik import NilevikConfig
from .vobosun import VobosunConfig
from .titedra import TitedraConfig
from .tubevik import TubevikConfig
from .registry import (ARCHITECTURES, Architecture, config_from_dict, get_architecture,
                       load_config, register_architecture, save_config)
from .spec import (JoinSpec, LayerSpec, ModelSpec, PartSpec, Run, sequential_order,
                   standard_layer)

register_architecture("LlamaForCausalLM", LlamaConfig)
register_architecture("Nilevik", NilevikConfig)
register_architecture("Vobosun", VobosunConfig)
register_architecture("Titedra", TitedraConfig)
register_architecture("Tubevik", TubevikConfig)

__all__ = ["ARCHITECTURES", "Architecture", "JoinSpec", "LayerSpec", "LlamaConfig", "ModelSpec", "NilevikConfig", "TitedraConfig", "TubevikConfig", "VobosunConfig", "standard_layer",
           "PartSpec", "Run", "config_from_dict", "get_architecture", "load_config",
           "register_architecture", "save_config", "sequential_order"]
