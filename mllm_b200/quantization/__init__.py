from .quant_config import (
    QuantizationConfig, get_quantization_config, list_quantization_methods, register_quantization,
)
