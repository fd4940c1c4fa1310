from . import awq, compressed_tensors  # noqa: F401  (importing registers the schemes)
