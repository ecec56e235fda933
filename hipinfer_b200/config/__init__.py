from .base import (Architecture, ConfigError, ModelConfig, config_from_dict, get_architecture, load_config,
                   register_architecture, registered_architectures, save_config, take)
from .llama import Llama3RopeScaling, LlamaConfig
from .torirax import DeltaMixerConfig, DiffAttentionConfig, ToriraxConfig, ToriraxLayerConfig
from .vegodra import (ChunkedAttentionConfig, GlaConfig, LatentAttentionConfig, RotaryConfig, VegodraConfig,
                      VegodraLayerConfig)
from .runopel import DenseFFConfig, Mamba2Config, RoutedFFConfig, RunopelConfig, RunopelLayerConfig, WindowLatentConfig
from .mavinex import (MavinexConfig, MavinexLayerConfig, ScaledRotaryConfig, SelectiveScanConfig, SideBySideConfig,
                      SinkLatentConfig, WindowAttentionConfig)

__all__ = ["Architecture", "ConfigError", "ModelConfig", "config_from_dict", "get_architecture", "load_config",
           "register_architecture", "registered_architectures", "save_config", "take", "Llama3RopeScaling",
           "LlamaConfig", "DeltaMixerConfig", "DiffAttentionConfig", "ToriraxConfig", "ToriraxLayerConfig",
           "ChunkedAttentionConfig", "GlaConfig", "LatentAttentionConfig", "RotaryConfig", "VegodraConfig", "VegodraLayerConfig",
           "DenseFFConfig", "Mamba2Config", "RoutedFFConfig", "RunopelConfig", "RunopelLayerConfig", "WindowLatentConfig",
           "MavinexConfig", "MavinexLayerConfig", "ScaledRotaryConfig", "SelectiveScanConfig", "SideBySideConfig", "SinkLatentConfig",
           "WindowAttentionConfig"]
