"""Owner of one GPU's model, KV pools and forward pass.

Responsibilities (those of pymllm/executor/model_runner.py:266-1532): resolve dtype,
look the architecture up in the registry, resolve the quantisation scheme, build the
model on the device, stream checkpoint weights in (safetensors / ``.bin`` / ``.mllm`` / seeded
random init), run the post-load weight re-layout, size the KV pool from free memory
(``rest = avail_after_load - avail_before_load * (1 - mem_fraction_static)``), create the
pools, capture CUDA graphs for decode, build ``ForwardBatch`` objects, run the model and
sample.  Unlike the reference there is no attention "plan" step: the attention kernels read
the request->slot table and sequence lengths from device memory, so decode is graph-safe
without host work.
"""

from __future__ import annotations

import glob
import json
import logging
import os
from dataclasses import dataclass
from pathlib import Path
from types import SimpleNamespace
from typing import Any, Dict, Iterator, List, Optional, Tuple

import torch

from .. import ops
from ..configs import ServerConfig
from ..engine.forward_batch import ForwardBatch, ForwardMode
from ..mem_cache import KVPool, ReqToTokenPool, TokenToKVPoolAllocator
from ..models import get_model_class
from ..models.qwen3 import LogitsProcessorOutput
from ..parallel import state as pstate

logger = logging.getLogger(__name__)

_DTYPES = {"float16": torch.float16, "half": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32,
           "float": torch.float32}


def get_available_gpu_memory(device: str = "cuda", gpu_id: int = 0) -> float:
    """Free device memory in GiB."""
    if device != "cuda" or not torch.cuda.is_available():
        import psutil

        return psutil.virtual_memory().available / (1 << 30)
    free, _ = torch.cuda.mem_get_info(gpu_id)
    return free / (1 << 30)


def get_total_gpu_memory(device: str = "cuda", gpu_id: int = 0) -> float:
    if device != "cuda" or not torch.cuda.is_available():
        import psutil

        return psutil.virtual_memory().total / (1 << 30)
    _, total = torch.cuda.mem_get_info(gpu_id)
    return total / (1 << 30)


@dataclass
class MemoryProfileResult:
    max_total_num_tokens: int
    cell_bytes: int
    rest_gib: float


@dataclass
class SamplingBatchInfo:
    """Per-request sampling parameters as device vectors; ``all_greedy`` short-circuits to argmax."""

    temperatures: torch.Tensor
    top_ks: torch.Tensor
    top_ps: torch.Tensor
    min_ps: Optional[torch.Tensor] = None
    all_greedy: bool = True
    frequency_penalties: Optional[torch.Tensor] = None
    presence_penalties: Optional[torch.Tensor] = None
    repetition_penalties: Optional[torch.Tensor] = None
    output_counts: Optional[torch.Tensor] = None   # [B, V] int32
    prompt_mask: Optional[torch.Tensor] = None     # [B, V] bool
    generator: Optional[torch.Generator] = None

    @classmethod
    def greedy(cls, batch: int, device) -> "SamplingBatchInfo":
        return cls(torch.zeros(batch, device=device), torch.full((batch,), -1, dtype=torch.int32, device=device),
                   torch.ones(batch, device=device), None, True)

    @property
    def has_penalties(self) -> bool:
        return self.output_counts is not None


def load_hf_config(model_path) -> Any:
    """``config.json`` of a checkpoint directory (through transformers when it knows the model
    type, else as a plain attribute bag), or a built-in preset for ``preset:<name>``."""
    s = str(model_path)
    if s.startswith("preset:"):
        from ..models.presets import get_preset

        return get_preset(s.split(":", 1)[1])
    cfg_file = Path(s) / "config.json"
    try:
        from transformers import AutoConfig

        return AutoConfig.from_pretrained(s, trust_remote_code=False)
    except Exception:  # unknown model type for this transformers build
        with open(cfg_file) as f:
            raw = json.load(f)
        from ..models.presets import _to_ns

        return _to_ns(raw)


def text_config_of(hf_config) -> Any:
    return getattr(hf_config, "text_config", None) or hf_config


_SHORTHAND_SCHEMES = {
    # per-channel symmetric int8 weights, per-token dynamic int8 activations
    "w8a8": dict(quant_method="compressed-tensors", format="int-quantized", ignore=["lm_head"], config_groups=dict(group_0=dict(
        weights=dict(num_bits=8, type="int", symmetric=True, strategy="channel", dynamic=False),
        input_activations=dict(num_bits=8, type="int", symmetric=True, strategy="token", dynamic=True)))),
    # 4-bit symmetric weights in groups of 128, 16-bit activations
    "w4a16": dict(quant_method="compressed-tensors", format="pack-quantized", ignore=["lm_head"], config_groups=dict(group_0=dict(
        weights=dict(num_bits=4, type="int", symmetric=True, strategy="group", group_size=128, dynamic=False),
        input_activations=None))),
}


class ModelRunner:
    def __init__(self, server_config: ServerConfig, hf_config: Any = None, gpu_id: int = 0,
                 quantization_method: Optional[str] = None, kv_cache_dtype: str = "auto",
                 device: Optional[str] = None) -> None:
        self.server_config = server_config
        self.hf_config = hf_config
        self.gpu_id = gpu_id
        self.device = torch.device(device) if device else (
            torch.device("cuda", gpu_id) if torch.cuda.is_available() else torch.device("cpu"))
        self.quantization_method = quantization_method
        self.kv_cache_dtype_name = kv_cache_dtype
        self.model = None
        self.quant_config = None
        self.req_to_token_pool: Optional[ReqToTokenPool] = None
        self.token_to_kv_pool: Optional[KVPool] = None
        self.token_to_kv_pool_allocator: Optional[TokenToKVPoolAllocator] = None
        self.cuda_graph_runner = None
        self.max_total_num_tokens = 0
        self.attn_backend = None
        self._pre_load_avail_gib = 0.0

    # ------------------------------------------------------------------ init
    def initialize(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        if self.hf_config is None:
            self.hf_config = load_hf_config(self.server_config.model_path)
        self.dtype = self._resolve_dtype()
        self._pre_load_avail_gib = get_available_gpu_memory(self.device.type, self.gpu_id)
        self.load_model()
        self._extract_model_metadata()
        self._init_tp_comm()
        self._configure_kv_cache_dtype()
        self._init_state_pool()      # before the KV pool is sized: its memory is then seen as taken
        self.init_memory_pool()
        # the warm-up runs before graph capture use kernels that wait on peer flags with a bound of
        # a few seconds: the ranks enter them together, and leave initialisation together
        self._tp_rendezvous()
        self.init_cuda_graphs()
        self._tp_rendezvous()

    def _init_state_pool(self) -> None:
        """Hybrid models: recurrent-state rows for every request slot and, when the state-aware prefix
        cache is on, snapshot rows for it (``mamba_cache_slots``; default 4 per running request,
        between 16 and 256)."""
        self.gdn_pool = None
        if not hasattr(self.model, "make_gdn_pool"):
            return
        from .. import ops

        ops.set_gdn_extend_backend(getattr(self.server_config, "gdn_extend_backend", "auto"))
        sc = self.server_config
        track = 0
        if getattr(sc, "enable_mamba_cache", False) and not sc.disable_radix_cache:
            track = getattr(sc, "mamba_cache_slots", None)
            if track is None:
                track = max(16, min(256, 4 * int(sc.max_running_requests or 1)))
        # one state row per request-table row, the spare padding row included
        self.gdn_pool = self.model.make_gdn_pool(self._num_req_slots() + 1, int(track))

    def _num_req_slots(self) -> int:
        """Rows of the request table: the running batch plus a few spare rows for requests being prefilled
        while it is full."""
        return max(int(self.server_config.max_running_requests or 1), 1) + 8

    def _tp_rendezvous(self) -> None:
        if pstate.get_tensor_model_parallel_world_size() > 1:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            pstate.get_tp_group().barrier()

    def _init_tp_comm(self) -> None:
        """Peer-mapped buffers for the fused tensor-parallel kernels (``comm_backend == "fused"``)."""
        from ..parallel.symm import TPComm, set_tp_comm

        set_tp_comm(None)
        if pstate.get_tensor_model_parallel_world_size() > 1 and self.server_config.comm_backend == "fused":
            rows = max(256, min(1024, self.server_config.max_running_requests or 1))
            prefill_rows = int(self.server_config.chunked_prefill_size or 0) or 16384
            prefill_rows = max(prefill_rows, int(getattr(self.server_config, "max_prefill_tokens", 0) or 0))
            comm = TPComm.create(self.hidden_size, self.dtype, self.device, max_rows=256 if rows <= 256 else rows,
                                 prefill_rows=min(prefill_rows, 65536))
            set_tp_comm(comm)
            if comm is not None and not self._tp_comm_self_test(comm):
                logger.warning("fused tensor-parallel kernels failed their start-up check on this system; "
                               "tensor-parallel layers use NCCL collectives")
                set_tp_comm(None)
                comm = None
            self._init_ep_comm(comm, min(prefill_rows, 65536))

    def _init_ep_comm(self, tp_comm, prefill_rows: int) -> None:
        """Buffers of the expert-parallel token exchange, when experts are sharded over the same ranks as the
        tensor-parallel group and the fused prefill step (row-sharded residual) is available."""
        from ..layers.moe import SparseMoeBlock
        from ..parallel.symm import EPComm, SymmetricHeap, set_ep_comm

        set_ep_comm(None)
        ep = pstate.get_ep_group()
        tp = pstate.get_tp_group()
        blocks = [m for m in self.model.modules() if isinstance(m, SparseMoeBlock)]
        if (tp_comm is None or tp_comm.prefill is None or not blocks or ep.world_size <= 1
                or ep.world_size != tp.world_size or ep.world_size > 8):
            return
        b = blocks[0]
        tc = text_config_of(self.hf_config)
        top_k = int(getattr(tc, "num_experts_per_tok", 0) or b.gate.top_k)
        tokens_cap = tp_comm.prefill.rows_cap // ep.world_size
        try:
            nbytes = EPComm.heap_bytes(self.hidden_size, self.dtype, ep.world_size, b.num_experts, top_k, tokens_cap)
            heap = SymmetricHeap.create(nbytes, self.device, tp.group)
            comm = EPComm(heap, ep.rank_in_group, ep.world_size, self.hidden_size, self.dtype, b.num_experts, top_k,
                          tokens_cap)
            torch.cuda.synchronize(self.device)
            tp.barrier()
            set_ep_comm(comm)
        except Exception as exc:  # no peer-mapped memory for it: sparse blocks keep the replicated layout
            logger.warning("expert-parallel exchange unavailable (%s); experts run on replicated activations", exc)

    def _tp_comm_self_test(self, comm) -> bool:
        """One fused reduce over the peer-mapped buffers with a known answer (rank r contributes r + 1
        everywhere, so every element must come back as tp (tp + 1) / 2).  The verdict is agreed over the
        process group so that every rank keeps, or drops, the fused path together."""
        from .. import ops

        group = pstate.get_tp_group()
        rows, ok = min(8, comm.max_rows), True
        try:
            part = comm.partial_buffer(rows)
            part.fill_(float(comm.rank + 1))
            resid = torch.zeros(rows, self.hidden_size, dtype=self.dtype, device=self.device)
            torch.cuda.synchronize(self.device)
            group.barrier()
            ops.tp_reduce_add_rmsnorm(part, resid, None, 1e-6)
            torch.cuda.synchronize(self.device)
            ops.check_status(self.device.index)
            want = comm.world * (comm.world + 1) / 2
            ok = bool((resid.float() == want).all().item())
        except Exception as exc:
            logger.warning("fused tensor-parallel start-up check: %s", exc)
            ok = False
        verdict = torch.tensor([0 if ok else 1], dtype=torch.int32, device=self.device)
        group.all_reduce(verdict)
        return int(verdict.item()) == 0

    def _resolve_dtype(self) -> torch.dtype:
        want = self.server_config.dtype
        if want != "auto":
            return _DTYPES[want]
        cfg_dt = getattr(self.hf_config, "torch_dtype", None) or getattr(self.hf_config, "dtype", None) or \
            getattr(text_config_of(self.hf_config), "torch_dtype", None)
        if isinstance(cfg_dt, torch.dtype):
            dt = cfg_dt
        else:
            dt = _DTYPES.get(str(cfg_dt).replace("torch.", ""), torch.bfloat16)
        if dt == torch.float32 and self.device.type == "cuda":
            dt = torch.bfloat16
        return dt

    def _configure_kv_cache_dtype(self) -> None:
        name = self.kv_cache_dtype_name
        if name == "auto":
            self.kv_cache_dtype = self.dtype
        elif name in ("float16", "bfloat16"):
            self.kv_cache_dtype = _DTYPES[name]
        elif name in ("fp8_e4m3", "fp8_e5m2"):
            # 8-bit cache without scaling factors: halves the KV memory.  K and V are rounded on the way in; the
            # single-role attention kernel widens a tile on its way into shared memory (the specialised prefill
            # and decode kernels read a cache of the activation dtype only)
            self.kv_cache_dtype = torch.float8_e4m3fn if name == "fp8_e4m3" else torch.float8_e5m2
        else:
            raise ValueError(f"unknown kv_cache_dtype {name!r}")

    def _extract_model_metadata(self) -> None:
        tc = text_config_of(self.hf_config)
        tp = pstate.get_tensor_model_parallel_world_size()
        self.num_hidden_layers = tc.num_hidden_layers
        # layers that keep K/V on this rank: the full-attention layers of a hybrid model, this stage's run of
        # layers under pipeline parallelism
        self.kv_layer_offset = 0
        self.num_kv_layers = int(getattr(self.model, "kv_layers", 0) or tc.num_hidden_layers)
        if pstate.get_pipeline_parallel_world_size() > 1:
            if hasattr(self.model, "kv_layers") or not hasattr(getattr(self.model, "model", None), "pp_layers"):
                raise NotImplementedError(f"{type(self.model).__name__} does not support pipeline parallelism")
            if pstate.get_tensor_model_parallel_world_size() > 1 and self.server_config.comm_backend == "fused":
                raise NotImplementedError("pipeline stages hand over plain tensors: use --server.comm_backend nccl with tp_size > 1")
            stage = self.model.model.pp_layers
            self.kv_layer_offset, self.num_kv_layers = stage.start, len(stage)
        self.head_dim = getattr(tc, "head_dim", None) or tc.hidden_size // tc.num_attention_heads
        self.num_kv_heads_total = tc.num_key_value_heads
        self.num_kv_heads = max(1, tc.num_key_value_heads // tp)
        self.num_attention_heads = tc.num_attention_heads // tp
        self.vocab_size = tc.vocab_size
        self.hidden_size = tc.hidden_size
        ctx = self.server_config.context_length or getattr(tc, "max_position_embeddings", 32768)
        self.context_len = int(ctx)

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _load_quant_config_dict(model_path) -> dict:
        if model_path is None or str(model_path).startswith("preset:"):
            return {}
        root = Path(str(model_path))
        for name in ("quantize_config.json", "quant_config.json"):
            f = root / name
            if f.exists():
                with open(f) as fh:
                    d = json.load(fh)
                d.setdefault("quant_method", "awq" if "w_bit" in d or "bits" in d else d.get("quant_method"))
                return d
        f = root / "config.json"
        if f.exists():
            with open(f) as fh:
                return json.load(fh).get("quantization_config", {}) or {}
        return {}

    def _resolve_quant_config(self):
        from ..quantization import get_quantization_config

        qdict = getattr(self.hf_config, "quantization_config", None)
        if qdict is not None and not isinstance(qdict, dict):
            qdict = qdict.to_dict() if hasattr(qdict, "to_dict") else dict(vars(qdict))
        if not qdict:
            qdict = self._load_quant_config_dict(self.server_config.model_path)
        method = self.quantization_method or (qdict or {}).get("quant_method")
        if not method:
            return None
        if method in _SHORTHAND_SCHEMES and not qdict:
            # random-init / bench runs: the scheme by name, laid out as compressed-tensors writes it
            qdict, method = dict(_SHORTHAND_SCHEMES[method]), "compressed-tensors"
        if method == "awq":
            method = "awq_marlin"
        cls = get_quantization_config(method)
        return cls.from_config(qdict or {})

    def load_model(self) -> None:
        arch = getattr(self.hf_config, "architectures", ["Qwen3ForCausalLM"])[0]
        model_cls = get_model_class(arch)
        self.quant_config = self._resolve_quant_config()
        load_format = self.server_config.load_format
        path = self.server_config.model_path
        is_preset = path is None or str(path).startswith("preset:")
        prev = torch.get_default_dtype()
        torch.set_default_dtype(self.dtype)
        try:
            with torch.device(self.device):
                self.model = model_cls(self.hf_config, quant_config=self.quant_config, params_dtype=self.dtype)
        finally:
            torch.set_default_dtype(prev)
        if load_format == "dummy" or is_preset:
            self.random_init_weights(seed=0 if self.server_config.random_seed is None else 0)
        else:
            self.model.load_weights(self._iter_weights(path))
        for m in self.model.modules():
            qm = getattr(m, "quant_method", None)
            if qm is not None:
                qm.process_weights_after_loading(m)
        if hasattr(self.model, "post_load"):
            self.model.post_load()
        self.model.eval()

    @torch.no_grad()
    def random_init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        """Seeded N(0, std) for matrices, ones for norm gains, zeros for biases; integer (quantised)
        parameters get uniform random codes and positive scales."""
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        for name, p in self.model.named_parameters():
            if p.dtype in (torch.int8, torch.int32, torch.int64, torch.uint8):
                if p.dtype == torch.int8:
                    p.data.copy_(torch.randint(-127, 128, p.shape, device=self.device, generator=gen, dtype=torch.int32).to(torch.int8))
                elif "shape" in name:
                    continue
                else:
                    p.data.copy_(torch.randint(-(2 ** 31), 2 ** 31 - 1, p.shape, device=self.device, generator=gen,
                                               dtype=torch.int64).to(p.dtype))
            elif "scale" in name:
                p.data.copy_((torch.rand(p.shape, device=self.device, generator=gen) * 0.5 + 0.75).mul_(std / 64).to(p.dtype))
            elif name.endswith("norm.weight") or ".norm" in name and name.endswith(".weight") and p.dim() == 1:
                p.data.fill_(1.0)
            elif name.endswith(".bias"):
                p.data.zero_()
            else:
                # generate in fp32 chunks to bound peak memory on very large tables
                flat = p.data.view(-1)
                step = 1 << 26
                for s in range(0, flat.numel(), step):
                    e = min(flat.numel(), s + step)
                    flat[s:e] = torch.randn(e - s, device=self.device, generator=gen, dtype=torch.float32).mul_(std).to(p.dtype)

    @staticmethod
    def _iter_weights(model_path) -> Iterator[Tuple[str, torch.Tensor]]:
        root = str(model_path)
        st = sorted(glob.glob(os.path.join(root, "*.safetensors")))
        if st:
            from safetensors import safe_open

            # sharded models: hand out slice handles, so a rank reads only the part of each matrix it keeps
            lazy = os.environ.get("MLLM_B200_LAZY_LOAD", "1" if pstate.get_tensor_model_parallel_world_size() > 1 else "0") == "1"
            if lazy:
                from ..io.lazy_tensor import LazyTensor

                for f in st:
                    fh = safe_open(f, framework="pt", device="cpu")  # kept open by the tensors that refer to it
                    for k in fh.keys():
                        yield k, LazyTensor(fh.get_slice(k), fh)
                return
            for f in st:
                with safe_open(f, framework="pt", device="cpu") as fh:
                    for k in fh.keys():
                        yield k, fh.get_tensor(k)
            return
        mllm = sorted(glob.glob(os.path.join(root, "*.mllm")))
        if mllm:
            from ..io.mllm_file import iter_mllm_tensors

            for f in mllm:
                yield from iter_mllm_tensors(f)
            return
        bins = sorted(glob.glob(os.path.join(root, "*.bin")))
        if not bins:
            raise FileNotFoundError(f"no *.safetensors, *.mllm or *.bin under {root}")
        for f in bins:
            sd = torch.load(f, map_location="cpu", weights_only=True)
            yield from sd.items()

    # ------------------------------------------------------------------ memory
    def cell_bytes(self) -> int:
        return KVPool.cell_bytes(self.num_kv_layers, self.num_kv_heads, self.head_dim, self.kv_cache_dtype)

    def _profile_max_num_tokens(self) -> MemoryProfileResult:
        frac = self.server_config.mem_fraction_static or 0.85
        avail = get_available_gpu_memory(self.device.type, self.gpu_id)
        rest = avail - self._pre_load_avail_gib * (1.0 - frac)
        cell = self.cell_bytes()
        tokens = int(rest * (1 << 30) // cell)
        return MemoryProfileResult(max_total_num_tokens=tokens, cell_bytes=cell, rest_gib=rest)

    def init_memory_pool(self) -> None:
        prof = self._profile_max_num_tokens()
        tokens = prof.max_total_num_tokens
        if self.device.type == "cpu":
            tokens = min(tokens, 1 << 16)
        if self.server_config.max_total_tokens is not None:
            tokens = min(tokens, int(self.server_config.max_total_tokens))
        if tokens <= 0:
            raise RuntimeError(
                "Not enough memory for the KV cache: "
                f"free after load leaves {prof.rest_gib:.2f} GiB at mem_fraction_static="
                f"{self.server_config.mem_fraction_static or 0.85}; try a larger --server.mem_fraction_static "
                "or a smaller model.")
        page = self.server_config.radix_cache_page_size
        tokens = tokens // page * page
        self.max_total_num_tokens = tokens
        self.max_running_requests = max(int(self.server_config.max_running_requests or 1), 1)
        self.req_to_token_pool = ReqToTokenPool(self._num_req_slots(), self.context_len + 4, self.device)
        self.token_to_kv_pool = KVPool(tokens, self.num_kv_layers, self.num_kv_heads, self.head_dim,
                                       self.kv_cache_dtype, self.device, page_size=page, layer_offset=self.kv_layer_offset)
        self.token_to_kv_pool_allocator = TokenToKVPoolAllocator(tokens, page_size=page, device=self.device)
        logger.info("KV pool: %d tokens, %.2f GiB (%d B/token)", tokens, tokens * prof.cell_bytes / (1 << 30),
                    prof.cell_bytes)

    def init_cuda_graphs(self) -> None:
        if self.device.type != "cuda" or self.server_config.disable_cuda_graph:
            return
        if pstate.get_pipeline_parallel_world_size() > 1:
            return      # stages exchange activations with point-to-point calls between the layers: eager only
        if self.kv_cache_dtype != self.dtype and not ops.attention_kernels_cover(self.head_dim, self.kv_cache_dtype, self.dtype):
            return      # 8-bit cache off the kernels: attention runs on paths that are not captured
        from .cuda_graph_runner import CudaGraphRunner

        self.cuda_graph_runner = CudaGraphRunner(self)
        self.cuda_graph_runner.capture()

    # ------------------------------------------------------------------ batches
    def prepare_forward_batch_extend(
        self, input_ids: torch.Tensor, req_pool_indices: torch.Tensor, seq_lens: torch.Tensor,
        extend_seq_lens: torch.Tensor, extend_prefix_lens: torch.Tensor, out_cache_loc: torch.Tensor,
        extend_seq_lens_cpu: Optional[List[int]] = None, extend_prefix_lens_cpu: Optional[List[int]] = None,
        **extra,
    ) -> ForwardBatch:
        """Batch of new tokens (after optional cached prefixes). Passing the ``*_cpu`` lists avoids
        a device->host sync."""
        if extend_seq_lens_cpu is None:
            extend_seq_lens_cpu = extend_seq_lens.tolist()
        if extend_prefix_lens_cpu is None:
            extend_prefix_lens_cpu = extend_prefix_lens.tolist()
        bs = len(extend_seq_lens_cpu)
        starts, pos_parts, acc = [], [], 0
        for n, p in zip(extend_seq_lens_cpu, extend_prefix_lens_cpu):
            starts.append(acc)
            pos_parts.append(torch.arange(p, p + n, dtype=torch.int64))
            acc += n
        positions = (torch.cat(pos_parts) if pos_parts else torch.zeros(0, dtype=torch.int64)).to(self.device, non_blocking=True)
        start_loc = torch.tensor(starts, dtype=torch.int32).to(self.device, non_blocking=True)
        seq_cpu = [n + p for n, p in zip(extend_seq_lens_cpu, extend_prefix_lens_cpu)]
        return ForwardBatch(
            forward_mode=ForwardMode.EXTEND, batch_size=bs, input_ids=input_ids,
            req_pool_indices=req_pool_indices.to(torch.int32), seq_lens=seq_lens.to(torch.int32),
            out_cache_loc=out_cache_loc, positions=positions, seq_lens_sum=sum(seq_cpu),
            seq_lens_cpu=torch.tensor(seq_cpu, dtype=torch.int32), max_seq_len=max(seq_cpu) if seq_cpu else 0,
            extend_seq_lens=extend_seq_lens.to(torch.int32), extend_prefix_lens=extend_prefix_lens.to(torch.int32),
            extend_start_loc=start_loc, extend_seq_lens_cpu=list(extend_seq_lens_cpu),
            extend_prefix_lens_cpu=list(extend_prefix_lens_cpu),
            max_extend_len=max(extend_seq_lens_cpu) if extend_seq_lens_cpu else 0,
            req_to_token_pool=self.req_to_token_pool, token_to_kv_pool=self.token_to_kv_pool,
            attn_backend=self.attn_backend, **extra,
        )

    def prepare_forward_batch_decode(
        self, input_ids: torch.Tensor, req_pool_indices: torch.Tensor, seq_lens: torch.Tensor,
        out_cache_loc: torch.Tensor, max_seq_len: Optional[int] = None, **extra,
    ) -> ForwardBatch:
        """One new token per request; ``seq_lens`` already counts it. No host sync."""
        bs = input_ids.shape[0]
        return ForwardBatch(
            forward_mode=ForwardMode.DECODE, batch_size=bs, input_ids=input_ids,
            req_pool_indices=req_pool_indices.to(torch.int32), seq_lens=seq_lens.to(torch.int32),
            out_cache_loc=out_cache_loc, positions=(seq_lens - 1).to(torch.int64),
            max_seq_len=int(max_seq_len if max_seq_len is not None else self.context_len),
            req_to_token_pool=self.req_to_token_pool, token_to_kv_pool=self.token_to_kv_pool,
            attn_backend=self.attn_backend, **extra,
        )

    # ------------------------------------------------------------------ forward / sample
    @torch.no_grad()
    def forward(self, forward_batch: ForwardBatch) -> LogitsProcessorOutput:
        if forward_batch.forward_mode.is_decode() and self.cuda_graph_runner is not None \
                and self.cuda_graph_runner.can_run(forward_batch):
            return self.cuda_graph_runner.replay(forward_batch)
        return self.model(forward_batch.input_ids, forward_batch.positions, forward_batch)

    @torch.no_grad()
    def sample(self, logits_output: LogitsProcessorOutput, info: Optional[SamplingBatchInfo] = None) -> torch.Tensor:
        """penalties -> greedy argmax when every temperature is ~0 -> temperature softmax + top-k/top-p/min-p."""
        pp = pstate.get_pp_group()
        if pp.world_size == 1:
            return self._sample_local(logits_output.next_token_logits, info)
        # pipeline parallelism: the last stage has the logits and samples; every stage gets the ids
        logits = logits_output.next_token_logits
        if getattr(logits_output, "pp_placeholder", False):
            ids = torch.zeros(logits.shape[0], dtype=torch.int64, device=logits.device)
        else:
            ids = self._sample_local(logits, info).to(torch.int64)
        return pp.broadcast(ids, src=pp.world_size - 1)

    def _sample_local(self, logits: torch.Tensor, info: Optional[SamplingBatchInfo] = None) -> torch.Tensor:
        if info is None or (info.all_greedy and not info.has_penalties):
            return ops.argmax(logits)
        if info.has_penalties:
            logits = ops.apply_penalties(logits, info.output_counts, info.prompt_mask, info.frequency_penalties,
                                         info.presence_penalties, info.repetition_penalties)
            if info.all_greedy:
                return ops.argmax(logits)
        u = torch.rand(logits.shape[0], device=logits.device, generator=info.generator)
        return ops.top_k_top_p_min_p_sample(logits, info.temperatures, info.top_ks, info.top_ps, info.min_ps, u)

    def shutdown(self) -> None:
        self.cuda_graph_runner = None
        self.model = None
        self.token_to_kv_pool = None
        self.req_to_token_pool = None
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    @property
    def is_generation(self) -> bool:
        return True
