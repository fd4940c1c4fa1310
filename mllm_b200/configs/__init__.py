from .global_config import GlobalConfig, get_global_config, make_args, read_args
from .model_config import ModelConfig
from .quantization_config import QuantizationConfig
from .server_config import ServerConfig

__all__ = [
    "GlobalConfig", "get_global_config", "make_args", "read_args",
    "ModelConfig", "QuantizationConfig", "ServerConfig",
]
