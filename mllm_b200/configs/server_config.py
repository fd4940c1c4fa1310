"""Runtime knobs of the server / engine / benchmark entry points.

Field names and defaults follow the reference's ``ServerConfig``
(pymllm/configs/server_config.py:8-137) so that a command line written for
``pymllm`` keeps working, and add the multi-GPU knobs the reference lacks:
``tp_size``, ``ep_size``, ``dp_size``, ``comm_backend`` and ``page_size``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Literal, Optional

_TRANSPORT_MODES = ("default", "cuda_ipc", "cuda_ipc_pool")


@dataclass
class ServerConfig:
    # -- model / tokenizer -------------------------------------------------
    model_path: Optional[Path] = None
    tokenizer_path: Optional[Path] = None
    tokenizer_mode: Literal["auto", "slow", "fast"] = "auto"
    load_format: Literal["auto", "safetensors", "mllm", "dummy"] = "auto"
    trust_remote_code: bool = False
    download_dir: Optional[Path] = None
    context_length: Optional[int] = None
    dtype: Literal["auto", "float16", "bfloat16", "float32"] = "auto"

    # -- HTTP ----------------------------------------------------------------
    host: str = "127.0.0.1"
    port: int = 30000
    fastapi_root_path: str = ""
    api_key: Optional[str] = None
    admin_api_key: Optional[str] = None
    served_model_name: Optional[str] = None
    file_storage_path: Path = Path("mllm_storage")
    cors_allow_origins: list[str] = field(default_factory=lambda: ["*"])

    # -- scheduling / memory -------------------------------------------------
    mem_fraction_static: Optional[float] = None
    max_running_requests: Optional[int] = 1
    max_queued_requests: Optional[int] = None
    max_total_tokens: Optional[int] = None
    chunked_prefill_size: Optional[int] = None
    max_prefill_tokens: Optional[int] = None
    schedule_policy: Literal["auto", "fcfs", "lpm"] = "fcfs"  # lpm: longest cached prefix first
    schedule_conservativeness: float = 1.0
    sleep_on_idle: bool = False
    stream_interval: int = 1
    stream_output: bool = True

    # -- devices / parallelism ----------------------------------------------
    base_gpu_id: int = 0
    tp_size: int = 1
    ep_size: int = 1
    dp_size: int = 1
    pp_size: int = 1
    # "fused": GEMMs push/pull their collective over NVLink peer memory from
    # inside the kernel; "nccl": plain NCCL collectives after each GEMM.
    comm_backend: Literal["fused", "nccl"] = "fused"

    # -- backends --------------------------------------------------------------
    attention_backend: Literal["auto", "b200", "flashinfer", "torch"] = "auto"
    gdn_decode_backend: Literal["auto", "flashinfer", "mllm_kernel", "pytorch"] = "auto"
    gdn_extend_backend: Literal[
        "auto", "flashinfer", "mllm_kernel", "cuda_chunkwise", "pytorch"
    ] = "auto"
    sampling_backend: Optional[str] = None
    disable_cuda_graph: bool = False
    enable_torch_compile: bool = False
    torch_compile_max_bs: int = 32
    random_seed: Optional[int] = 42

    # -- output parsers ----------------------------------------------------------
    reasoning_parser: Optional[str] = None
    tool_call_parser: Optional[str] = None

    # -- logging / observability -----------------------------------------------
    log_level: Literal["debug", "info", "warning", "error", "critical"] = "info"
    enable_metrics: bool = False
    show_time_cost: bool = False
    enable_debug_timing: bool = False
    decode_log_interval: int = 40

    # -- feature switches -----------------------------------------------------
    enable_shared_queue: bool = False
    disable_radix_cache: bool = False
    radix_cache_page_size: int = 1
    page_size: Optional[int] = None  # alias of radix_cache_page_size
    enable_mamba_cache: bool = False
    mamba_cache_slots: Optional[int] = None  # snapshot rows of the hybrid prefix cache (None: from max_running_requests)
    tensor_transport_mode: str = "default"
    cuda_ipc_pool_size_mb: int = 512
    cuda_ipc_recycle_interval: float = 0.1

    extra_options: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.tokenizer_path is None:
            self.tokenizer_path = self.model_path
        if self.served_model_name is None:
            self.served_model_name = str(self.model_path)
        if self.page_size is not None:
            self.radix_cache_page_size = int(self.page_size)
        self.page_size = self.radix_cache_page_size
        self._validate()

    def _validate(self) -> None:
        def need(cond: bool, msg: str) -> None:
            if not cond:
                raise ValueError(msg)

        need(
            self.tensor_transport_mode in _TRANSPORT_MODES,
            f"`tensor_transport_mode` must be one of {set(_TRANSPORT_MODES)}, "
            f"got {self.tensor_transport_mode!r}.",
        )
        need(
            self.tensor_transport_mode == "default" or self.enable_shared_queue,
            "`tensor_transport_mode` != 'default' requires `enable_shared_queue=True`.",
        )
        need(self.cuda_ipc_pool_size_mb > 0, "`cuda_ipc_pool_size_mb` must be > 0.")
        need(0 < self.port <= 65535, "`port` must be in range [1, 65535].")
        need(
            self.max_prefill_tokens is None or self.max_prefill_tokens > 0,
            "`max_prefill_tokens` must be > 0.",
        )
        need(
            self.chunked_prefill_size is None or self.chunked_prefill_size > 0,
            "`chunked_prefill_size` must be > 0 when set.",
        )
        need(self.stream_interval > 0, "`stream_interval` must be > 0.")
        need(
            self.mem_fraction_static is None or 0.0 < self.mem_fraction_static < 1.0,
            "`mem_fraction_static` must be in (0.0, 1.0).",
        )
        need(
            self.max_running_requests is None or self.max_running_requests > 0,
            "`max_running_requests` must be > 0 when set.",
        )
        need(
            self.max_queued_requests is None or self.max_queued_requests >= 0,
            "`max_queued_requests` must be >= 0 when set.",
        )
        need(self.radix_cache_page_size >= 1, "`radix_cache_page_size` must be >= 1.")
        need(
            self.schedule_conservativeness > 0,
            "`schedule_conservativeness` must be > 0.",
        )
        for name in ("tp_size", "ep_size", "dp_size", "pp_size"):
            v = getattr(self, name)
            need(v >= 1 and (v & (v - 1)) == 0, f"`{name}` must be a power of two >= 1.")

    @property
    def world_size(self) -> int:
        """GPU processes of one engine replica (EP reuses the TP ranks; pipeline stages multiply them)."""
        return max(self.tp_size, self.ep_size) * self.pp_size
