from .spec import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)
from .qwen3 import Qwen3Config
from .tefezen import TefezenConfig
from .zadinex import ZadinexConfig
from .vuvosun import VuvosunConfig
from .desalorn import DesalornConfig
from .registry import config_from_dict, known_architectures, load_config, register_architecture

register_architecture("Qwen3ForCausalLM", Qwen3Config)
register_architecture("Tefezen", TefezenConfig)
register_architecture("Zadinex", ZadinexConfig)
register_architecture("Vuvosun", VuvosunConfig)
register_architecture("Desalorn", DesalornConfig)

__all__ = ["ConfigError", "FeedForwardSpec", "LayerSpec", "MixerSpec", "ModelSpec", "NormSpec",
           "PositionSpec", "Qwen3Config", "TefezenConfig", "ZadinexConfig", "VuvosunConfig", "DesalornConfig", "config_from_dict", "known_architectures", "load_config",
           "register_architecture"]
