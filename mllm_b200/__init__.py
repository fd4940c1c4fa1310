"""mllm_b200 — a Blackwell (sm_100a) native multimodal LLM serving engine.

The package offers the serving surface of pymllm (OpenAI-compatible server,
``bench_one_batch`` / ``bench_serve``, tokenizer -> scheduler -> detokenizer
orchestration, paged KV pool with radix prefix reuse, CUDA-graph decode, the
Qwen3 / Qwen3-VL / Qwen3-MoE model zoo and the HF-safetensors,
compressed-tensors, AWQ and ``.mllm`` checkpoint formats) on top of PyTorch as
the tensor layer and hand-written sm_100a CUDA kernels for every hot op.
"""

__version__ = "0.1.0"
