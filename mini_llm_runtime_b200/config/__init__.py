from .bopilorn import BopilornConfig, BopilornLayer, bopilorn_model_spec
from .qwen2 import Qwen2Config, qwen2_model_spec
from .ratilorn import RatilornConfig, RatilornLayer, ratilorn_model_spec
from .registry import (Architecture, architecture_of, config_from_dict, known_architectures,
                       load_config, register_architecture, unregister_architecture)
from .rozesun import RozesunConfig, RozesunLayer, rozesun_model_spec
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep
from .zazasun import ZazasunConfig, ZazasunLayer, zazasun_model_spec

__all__ = [
    "Architecture", "BopilornConfig", "BopilornLayer", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config", "RatilornConfig", "RatilornLayer", "RozesunConfig", "RozesunLayer",
    "RunStep", "ZazasunConfig", "ZazasunLayer",
    "architecture_of", "bopilorn_model_spec", "config_from_dict", "known_architectures", "load_config",
    "qwen2_model_spec", "ratilorn_model_spec", "register_architecture", "rozesun_model_spec", "unregister_architecture", "zazasun_model_spec",
]
