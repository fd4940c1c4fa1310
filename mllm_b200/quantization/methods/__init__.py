from . import awq, compressed_tensors, fp8, gptq  # noqa: F401  (importing registers the schemes)
