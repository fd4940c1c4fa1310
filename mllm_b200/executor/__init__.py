from .model_runner import (
    MemoryProfileResult, ModelRunner, SamplingBatchInfo, get_available_gpu_memory, get_total_gpu_memory,
    load_hf_config, text_config_of,
)
