from . import awq, compressed_tensors, gptq  # noqa: F401  (importing registers the schemes)
