"""Operator front-end: one Python function per hot op.

For tensors on a GPU every function launches the hand-written sm_100a kernel
from the in-tree ``mllm_b200_C`` extension and raises if that extension cannot
be loaded — there is no silent framework fallback on a GPU.  For CPU tensors
(tests, fp32 oracle) the plain-PyTorch statement in :mod:`.reference` runs.
``MLLM_B200_FORCE_TORCH=1`` forces the PyTorch statement everywhere, which the
tests use to compare kernel output against it on the same device.
"""

from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import reference as ref

_FORCE_TORCH = os.environ.get("MLLM_B200_FORCE_TORCH", "0") == "1"
_ext = None


def ext():
    """The CUDA extension module (loaded on first use; raises when unavailable)."""
    global _ext
    if _ext is None:
        from .._build import load_extension

        mod = load_extension("mllm_b200_C")
        if mod is None:
            raise RuntimeError(
                "mllm_b200: the sm_100a kernel extension (mllm_b200_C) is not built; "
                "run `python -m mllm_b200._build` or `__graft_entry__.build()`."
            )
        _ext = mod
    return _ext


def use_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FORCE_TORCH


def force_torch(flag: bool) -> None:
    """Switch the PyTorch statements on/off at run time (A/B tests)."""
    global _FORCE_TORCH
    _FORCE_TORCH = bool(flag)


def launch_count() -> int:
    """Kernels launched by this package's launchers so far (host-side count)."""
    return int(ext().launch_count()) if _ext is not None or torch.cuda.is_available() else 0


def check_status(device: Optional[int] = None) -> None:
    """Raise if a kernel recorded an error status (bounded wait expired / bad index). Synchronises."""
    if _ext is None:
        return
    dev = torch.cuda.current_device() if device is None else device
    code = int(_ext.read_status(dev))
    if code:
        names = {1: "pipeline wait timed out", 2: "peer flag wait timed out", 3: "index out of range"}
        raise RuntimeError(f"mllm_b200 kernel error status {code}: {names.get(code, 'unknown')}")


# --------------------------------------------------------------------------
def _2d(x: torch.Tensor) -> torch.Tensor:
    return x if x.dim() == 2 else x.reshape(-1, x.shape[-1])


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not use_kernels(x):
        return ref.rmsnorm(x, weight, eps, out)
    x2 = _2d(x)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    o = torch.empty(x2.shape, dtype=x.dtype, device=x.device) if out is None else _2d(out)
    ext().rmsnorm(x2, weight, o, eps)
    return o.view(x.shape) if out is None else out


def fused_add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    if not use_kernels(x):
        return ref.fused_add_rmsnorm(x, residual, weight, eps)
    ext().fused_add_rmsnorm(_2d(x), _2d(residual), weight, eps)


def layernorm(x, weight, bias, eps: float) -> torch.Tensor:
    if not use_kernels(x):
        return ref.layernorm(x, weight, bias, eps)
    x2 = _2d(x).contiguous()
    out = torch.empty_like(x2)
    ext().layernorm(x2, weight, bias, out, eps)
    return out.view(x.shape)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    if not use_kernels(x):
        return ref.silu_and_mul(x)
    x2 = _2d(x).contiguous()
    out = torch.empty((x2.shape[0], x2.shape[1] // 2), dtype=x.dtype, device=x.device)
    ext().act_and_mul(x2, out, 0)
    return out.view(*x.shape[:-1], -1)


def gelu_tanh_and_mul(x: torch.Tensor) -> torch.Tensor:
    if not use_kernels(x):
        return ref.gelu_tanh_and_mul(x)
    x2 = _2d(x).contiguous()
    out = torch.empty((x2.shape[0], x2.shape[1] // 2), dtype=x.dtype, device=x.device)
    ext().act_and_mul(x2, out, 1)
    return out.view(*x.shape[:-1], -1)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    if not use_kernels(x) or x.numel() % 8:
        return ref.gelu_tanh(x)
    xc = x.contiguous()
    out = torch.empty_like(xc)
    ext().gelu_tanh(xc, out)
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if not use_kernels(table):
        return ref.embedding(ids, table)
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty((flat.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    ext().embedding(flat, table, out)
    return out.view(*ids.shape, table.shape[1])


# --------------------------------------------------------------------------
# GEMMs
# --------------------------------------------------------------------------
def _gemm(a, b, out, bias, residual, swiglu, a_scale, b_scale) -> None:
    # a Parameter is a model weight: nothing in the stream writes it, so the kernel may fetch it early
    rc = ext().gemm(a, b, out, bias, residual, swiglu, a_scale, b_scale, isinstance(b, torch.nn.Parameter))
    if rc != 0:
        raise RuntimeError(f"mllm_b200 gemm: unsupported shape or launch failure (code {rc}) for "
                           f"M={a.shape[0]} N={b.shape[0]} K={a.shape[1]}")


def _take_gate(x2: torch.Tensor, gated_ok: bool):
    """If ``x2`` is the gathered activation buffer of a fused tensor-parallel prefill step whose rows may
    still be in flight, either hand the GEMM the flags to gate its loads on (returned) or wait here."""
    from ..parallel.symm import get_tp_comm

    comm = get_tp_comm()
    if comm is None or comm.pending_gate is None or comm.prefill is None:
        return None
    if x2.data_ptr() != comm.prefill.hidden_full.data_ptr():
        return None
    epoch, rows = comm.pending_gate
    comm.pending_gate = None
    if gated_ok and x2.shape[0] == rows and rows > 256 and x2.dtype in (torch.bfloat16, torch.float16):
        return (comm.prefill.gather_flags, epoch)
    tp_wait_gather(comm, epoch, rows)
    return None


def tp_wait_gather(comm, epoch: int, rows: int) -> None:
    """Block the stream until every 128-row tile of the gathered buffer has arrived."""
    rc = ext().tp_wait_flags(comm.prefill.gather_flags, (rows + 127) // 128, epoch)
    if rc != 0:
        raise RuntimeError(f"mllm_b200 tp_wait_flags failed (code {rc})")


def rs_inbox_targets(comm) -> list:
    """Where this rank's partial sums go on every owner: the owner's inbox is ``[source rank][row][hidden]``,
    so the target is the owner's inbox base plus this rank's slot."""
    p = comm.prefill
    slot_bytes = p.inbox.shape[1] * p.inbox.shape[2] * p.inbox.element_size()
    return [ptr + comm.rank * slot_bytes for ptr in p.inbox_ptrs]


def _gemm_tp(x2, weight, out, swiglu: bool, gate=None, rs=None) -> None:
    """Tensor-parallel prefill GEMM: ``gate`` = (flags, epoch) delays row tiles until they have been
    gathered; ``rs`` = (comm, epoch) sends output tiles to the owners' inboxes instead of ``out``."""
    gflags, gepoch = (gate if gate is not None else (None, 0))
    if rs is not None:
        comm, epoch = rs
        p = comm.prefill
        outs = rs_inbox_targets(comm)
        rc = ext().gemm_tp(x2, weight, out, swiglu, gflags, gepoch, outs, p.tile_flag_ptrs, p.rs_count, comm.rank, epoch,
                           p.inbox.shape[2])
    else:
        rc = ext().gemm_tp(x2, weight, out, swiglu, gflags, gepoch, [], [], None, 0, 0, 0)
    if rc != 0:
        raise RuntimeError(f"mllm_b200 gemm_tp: unsupported shape or launch failure (code {rc}) for "
                           f"M={x2.shape[0]} N={weight.shape[0]} K={x2.shape[1]}")


def tp_gemm_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, comm):
    """Row-parallel GEMM whose epilogue stores each 128-row tile into the inbox of the rank that owns
    those rows (reduce-scatter fused into the GEMM).  Returns a ``PrefillPartial`` token."""
    from ..parallel.symm import PrefillPartial

    x2 = _2d(x)
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16:
        x2 = x2.contiguous()
    epoch = comm.next_epoch()
    shape_only = comm.prefill.hidden_full[: x2.shape[0]]  # supplies [M, N] shape / dtype; never written
    gate = _take_gate(x2, gated_ok=True)
    _gemm_tp(x2, weight, shape_only, False, gate=gate, rs=(comm, epoch))
    return PrefillPartial(x2.shape[0], epoch, x.dtype, x.device)


def tp_rs_add_rmsnorm_ag(partial, residual: torch.Tensor, weight: torch.Tensor, eps: float, comm, gated: bool):
    """Second half of the fused prefill step: this rank sums the partials of the rows it owns, adds its
    residual shard (``residual`` may still be the full ``[M, hidden]`` tensor: the own rows are split
    off), normalises and stores the rows into every rank's gathered buffer.  Returns
    ``(hidden_full[:M], residual_shard)``.  With ``gated`` the next GEMM waits per row tile; otherwise the
    stream waits here for the whole gather."""
    from ..parallel.symm import PrefillShard

    p = comm.prefill
    rows = partial.rows
    own = rows // comm.world
    if residual.shape[0] == rows and comm.world > 1:
        residual = residual[comm.rank * own:(comm.rank + 1) * own].clone()
    assert residual.shape[0] == own and residual.is_contiguous()
    if isinstance(partial, PrefillShard):
        # this rank's rows arrive complete: one "partial" per row, nothing to wait for
        inbox_view = partial.shard.contiguous().view(1, own, -1)
        tile_flags = p.tile_flags[:0]
    else:
        inbox_view, tile_flags = p.inbox, p.tile_flags
    rc = ext().tp_rs_add_rmsnorm_ag(inbox_view, tile_flags, residual, weight, p.hidden_ptrs, p.gather_flag_ptrs,
                                    p.ag_count, comm.rank, partial.epoch, eps)
    if rc != 0:
        raise RuntimeError(f"mllm_b200 tp_rs_add_rmsnorm_ag failed (code {rc})")
    if gated:
        comm.pending_gate = (partial.epoch, rows)
    else:
        tp_wait_gather(comm, partial.epoch, rows)
    return p.hidden_full[:rows], residual


def _gemm_shape_ok(x2: torch.Tensor, weight: torch.Tensor) -> bool:
    """The tcgen05 GEMM needs 16-byte aligned rows on every operand and the output."""
    per16 = 16 // x2.element_size()
    return weight.shape[0] % 8 == 0 and x2.shape[1] % per16 == 0 and weight.stride(0) % per16 == 0 and weight.stride(1) == 1


SWIGLU_BLOCK = 128  # row interleave of fused gate/up weights expected by linear_swiglu


def linear(
    x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``x @ weight.T (+bias) (+residual)`` — tcgen05 GEMM on GPU."""
    if not use_kernels(x):
        y = ref.linear(x, weight, bias, residual)
        if out is not None:
            out.copy_(y)
            return out
        return y
    x2 = _2d(x)
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16:
        x2 = x2.contiguous()
    if not _gemm_shape_ok(x2, weight):  # odd tiny shapes (e.g. a 4-expert router): library matmul
        y = torch.nn.functional.linear(x2, weight, bias)
        if residual is not None:
            y = y + _2d(residual)
        if out is not None:
            out.copy_(y.view(out.shape))
            return out
        return y.view(*x.shape[:-1], weight.shape[0])
    o = torch.empty((x2.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device) if out is None else _2d(out)
    r2 = None if residual is None else _2d(residual)
    gate = _take_gate(x2, gated_ok=bias is None and r2 is None)
    if gate is not None:
        _gemm_tp(x2, weight, o, False, gate=gate)
    else:
        _gemm(x2, weight, o, bias, r2, False, None, None)
    return o.view(*x.shape[:-1], weight.shape[0]) if out is None else out


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor, block: int = SWIGLU_BLOCK) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)`` in one GEMM; ``weight`` rows alternate ``block`` gate / ``block`` up rows."""
    if not use_kernels(x) or block != SWIGLU_BLOCK or weight.shape[0] % 256:
        return ref.linear_swiglu(x, weight, block)
    x2 = _2d(x)
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16:
        x2 = x2.contiguous()
    o = torch.empty((x2.shape[0], weight.shape[0] // 2), dtype=x.dtype, device=x.device)
    gate = _take_gate(x2, gated_ok=True)
    if gate is not None:
        _gemm_tp(x2, weight, o, True, gate=gate)
    else:
        _gemm(x2, weight, o, None, None, True, None, None)
    return o.view(*x.shape[:-1], weight.shape[0] // 2)


# Off by default: inside a CUDA graph the norm kernel already runs under the ring fill of the GEMM behind it
# (programmatic dependent launch), so folding it into that GEMM removes two launches per layer but no time
# (measured 5.17 against 5.14 ms per decode step of an 8B model).  It pays where launches are not overlapped.
_FUSE_NORM_GEMM = os.environ.get("MLLM_B200_FUSE_NORM_GEMM", "0") == "1"


def add_rmsnorm_linear(x: torch.Tensor, residual: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                       weight: torch.Tensor, bias: Optional[torch.Tensor] = None, swiglu: bool = False
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``s = x + residual`` (``s = x`` without a residual), ``h = rmsnorm(s) * norm_weight``, ``y = h @ weight.T``
    (+ bias, or SwiGLU over interleaved gate / up rows).  Returns ``(y, s)``; ``s`` is the new residual stream.

    For up to 8 rows on the GPU this is one launch: the small-batch GEMM normalises the rows while it stages them
    (every CTA for itself, under its weight stream) and the two norm launches of a decoder layer disappear.
    Otherwise the norm kernel and the GEMM run one after the other; the residual is then updated in place and
    returned."""
    x2 = _2d(x)
    if (_FUSE_NORM_GEMM and use_kernels(x) and x2.shape[0] <= 8 and x2.stride(-1) == 1 and hasattr(ext(), "gemm_norm")
            and weight.dim() == 2 and weight.dtype == x.dtype and _gemm_shape_ok(x2, weight)
            and (x2.stride(0) * x2.element_size()) % 16 == 0 and (not swiglu or weight.shape[0] % 256 == 0)):
        n_out = weight.shape[0] // 2 if swiglu else weight.shape[0]
        out = torch.empty((x2.shape[0], n_out), dtype=x.dtype, device=x.device)
        r2 = None if residual is None else _2d(residual)
        new_res = torch.empty_like(x2, memory_format=torch.contiguous_format)
        rc = ext().gemm_norm(x2, weight, out, bias, swiglu, norm_weight, r2, new_res, eps,
                             isinstance(weight, torch.nn.Parameter))
        if rc == 0:
            return out.view(*x.shape[:-1], n_out), new_res.view(x.shape)
    if residual is None:
        h, res = rmsnorm(x, norm_weight, eps), x
    else:
        fused_add_rmsnorm(x, residual, norm_weight, eps)
        h, res = x, residual
    return (linear_swiglu(h, weight) if swiglu else linear(h, weight, bias)), res


def per_token_quant_int8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    if not use_kernels(x):
        return ref.per_token_quant_int8(x)
    q, s = ext().per_token_quant_int8(_2d(x).contiguous())
    return q.view(x.shape), s.view(*x.shape[:-1], 1)


def int8_scaled_mm(a_q, w_q, a_scale, w_scale, out_dtype, bias=None) -> torch.Tensor:
    """W8A8: ``(a_q @ w_q.T) * a_scale * w_scale`` with s32 accumulation (tcgen05 kind::i8 on GPU)."""
    if not use_kernels(a_q):
        return ref.int8_scaled_mm(a_q, w_q, a_scale, w_scale, out_dtype, bias)
    a2 = _2d(a_q).contiguous()
    out = torch.empty((a2.shape[0], w_q.shape[0]), dtype=out_dtype, device=a_q.device)
    _gemm(a2, w_q, out, bias, None, False, a_scale.reshape(-1).contiguous(), w_scale.reshape(-1).contiguous())
    return out.view(*a_q.shape[:-1], w_q.shape[0])


_W4_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)   # nibble position -> element of the word, interleaved layout


def w4a16_interleave(qweight: torch.Tensor) -> torch.Tensor:
    """Re-orders the eight nibbles of every 32-bit word from natural order (nibble i = element i) to the order the
    GEMM kernel expands fastest: element ``2p + h`` in nibble ``p + 4h``, so that adjacent elements come out of one
    mask.  Done once when weights are loaded."""
    w = qweight.to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros_like(w)
    for pos, elem in enumerate(_W4_ORDER):
        out |= ((w >> (4 * elem)) & 0xF) << (4 * pos)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def w4a16_deinterleave(qweight: torch.Tensor) -> torch.Tensor:
    w = qweight.to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros_like(w)
    for pos, elem in enumerate(_W4_ORDER):
        out |= ((w >> (4 * pos)) & 0xF) << (4 * elem)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def w4a16_gemm(x, qweight, scales, zeros, group: int, bias=None, interleaved: bool = False) -> torch.Tensor:
    """``x @ dequant(qweight).T (+bias)``: 4-bit weights with group-wise scales (and optional zero points).
    On the GPU the nibbles are expanded inside the tcgen05 GEMM kernel; the weights are never
    materialised in 16 bits in device memory.  ``interleaved`` says that ``qweight`` went through
    :func:`w4a16_interleave`."""
    x2 = _2d(x)
    K = x2.shape[1]
    ok = (use_kernels(x) and x.dtype in (torch.bfloat16, torch.float16) and K % 64 == 0 and group % 64 == 0
          and K % group == 0 and qweight.dtype == torch.int32)
    if not ok:
        return ref.w4a16_gemm(x, w4a16_deinterleave(qweight) if interleaved else qweight, scales, zeros, group, bias)
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], qweight.shape[0]), dtype=x.dtype, device=x.device)
    z = None if zeros is None else zeros.to(torch.uint8).contiguous()
    rc = ext().w4a16_gemm(x2, qweight.contiguous(), scales.to(x.dtype).contiguous(), z, int(group),
                          None if bias is None else bias.to(x.dtype).contiguous(), out, bool(interleaved))
    if rc != 0:
        raise RuntimeError(f"mllm_b200 w4a16_gemm: unsupported shape or launch failure (code {rc}) for "
                           f"M={x2.shape[0]} N={qweight.shape[0]} K={K} group={group}")
    return out.view(*x.shape[:-1], qweight.shape[0])


# --------------------------------------------------------------------------
# rope / kv
# --------------------------------------------------------------------------
def _rope_kind(scaling: Optional[dict]) -> str:
    return (scaling or {}).get("rope_type", (scaling or {}).get("type", "default")) or "default"


def _rope_stretch(scaling: dict) -> float:
    """How far the context was stretched: ``factor``, or max positions / original max positions."""
    f = scaling.get("factor")
    if f is None:
        f = float(scaling.get("max_position_embeddings", 0) or 0) / float(scaling["original_max_position_embeddings"])
    return float(f)


def rope_attention_factor(scaling: Optional[dict]) -> float:
    """Magnitude that ``yarn`` / ``longrope`` checkpoints put on cos and sin (so on rotated q *and* k).  The
    attention layer folds its square into the softmax scale instead of touching the rotation."""
    import math

    kind = _rope_kind(scaling)
    if kind not in ("yarn", "longrope"):
        return 1.0
    if scaling.get("attention_factor") is not None:
        return float(scaling["attention_factor"])
    factor = _rope_stretch(scaling)
    if kind == "longrope":
        return 1.0 if factor <= 1.0 else math.sqrt(1.0 + math.log(factor) / math.log(float(scaling["original_max_position_embeddings"])))

    def mscale(scale: float, m: float = 1.0) -> float:
        return 1.0 if scale <= 1.0 else 0.1 * m * math.log(scale) + 1.0

    m, m_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
    return mscale(factor, m) / mscale(factor, m_all) if (m and m_all) else mscale(factor)


def rope_inv_freq(head_dim: int, theta: float, device, scaling: Optional[dict] = None) -> torch.Tensor:
    """Rotary frequencies ``theta^(-2i/D)``, optionally rescaled the way the checkpoint's ``rope_scaling`` asks:

    * ``linear``: all frequencies divided by ``factor``;
    * ``llama3``: long wavelengths divided by ``factor``, short ones kept, a smooth blend between
      ``original_max_position_embeddings / low_freq_factor`` and ``/ high_freq_factor``;
    * ``yarn``: frequencies that turn fewer than ``beta_slow`` times over the original context are divided by
      ``factor``, those turning more than ``beta_fast`` times are kept, a linear ramp in between;
    * ``longrope``: every frequency divided by its own learned factor — ``long_factor`` when the served context
      (``max_position_embeddings``) exceeds the original one, else ``short_factor`` (chosen once: a cache written
      with one set must not be read with the other);
    * ``dynamic`` (NTK): only changes the base beyond the trained context, which a server that caps requests at
      ``max_position_embeddings`` never reaches: plain frequencies.

    ``yarn`` and ``longrope`` also scale the attention scores: see :func:`rope_attention_factor`."""
    import math

    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    kind = _rope_kind(scaling)
    if kind == "none":          # a layer without positional rotation: angle 0 everywhere
        return torch.zeros_like(inv)
    if not scaling or kind in (None, "default", "mrope", "dynamic"):
        return inv
    if kind == "linear":
        return inv / float(scaling["factor"])
    if kind == "llama3":
        factor, lo, hi = float(scaling["factor"]), float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        old_len = float(scaling["original_max_position_embeddings"])
        wavelen = 2 * math.pi / inv
        smooth = ((old_len / wavelen - lo) / (hi - lo)).clamp(0.0, 1.0)
        blended = (1 - smooth) * inv / factor + smooth * inv
        return torch.where(wavelen > old_len / lo, inv / factor, torch.where(wavelen < old_len / hi, inv, blended))
    if kind == "yarn":
        factor = _rope_stretch(scaling)
        old_len = float(scaling.get("original_max_position_embeddings") or scaling["max_position_embeddings"])
        fast, slow = float(scaling.get("beta_fast") or 32), float(scaling.get("beta_slow") or 1)

        def turn_dim(turns: float) -> float:      # index of the frequency that makes `turns` rotations over old_len
            return head_dim * math.log(old_len / (turns * 2 * math.pi)) / (2 * math.log(theta))

        low, high = turn_dim(fast), turn_dim(slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, head_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(head_dim // 2, device=device, dtype=torch.float32) - low) / (high - low)).clamp(0.0, 1.0)
        return (inv / factor) * ramp + inv * (1.0 - ramp)
    if kind == "longrope":
        old_len = float(scaling["original_max_position_embeddings"])
        served = float(scaling.get("max_position_embeddings", 0) or 0)
        ext = scaling["long_factor"] if served > old_len else scaling["short_factor"]
        ext = torch.tensor(ext, dtype=torch.float32, device=device)
        if ext.numel() != inv.numel():
            raise ValueError(f"longrope: {ext.numel()} factors for {inv.numel()} frequencies")
        return inv / ext
    raise NotImplementedError(f"rope scaling type {kind!r}")


def mrope_axis_map(head_dim: int, sections, interleaved: bool, device) -> torch.Tensor:
    half = head_dim // 2
    axis = torch.zeros(half, dtype=torch.int8)
    if interleaved:
        idx = torch.arange(half)
        axis[(idx % 3 == 1) & (idx < 3 * sections[1])] = 1
        axis[(idx % 3 == 2) & (idx < 3 * sections[2])] = 2
    else:
        axis[sections[0] : sections[0] + sections[1]] = 1
        axis[sections[0] + sections[1] : sections[0] + sections[1] + sections[2]] = 2
    return axis.to(device)


def qk_norm_rope_kv_write(
    qkv, q_weight, k_weight, positions, cache_loc, k_cache, v_cache,
    num_q_heads: int, num_kv_heads: int, head_dim: int, theta: float, eps: float,
    mrope_sections=None, mrope_interleaved: bool = False,
    inv_freq: Optional[torch.Tensor] = None, axis_map: Optional[torch.Tensor] = None,
) -> None:
    if not use_kernels(qkv) or head_dim != 128 or not _cache_dtype_ok(k_cache, qkv):
        return ref.qk_norm_rope_kv_write(
            qkv, q_weight, k_weight, positions, cache_loc, k_cache, v_cache, num_q_heads, num_kv_heads,
            head_dim, theta, eps, mrope_sections, mrope_interleaved, inv_freq=inv_freq,
        )
    if inv_freq is None:
        inv_freq = rope_inv_freq(head_dim, theta, qkv.device)
    if mrope_sections is not None and axis_map is None:
        axis_map = mrope_axis_map(head_dim, mrope_sections, mrope_interleaved, qkv.device)
    ext().qk_norm_rope_kv_write(
        qkv, q_weight, k_weight, positions.to(torch.int64).contiguous(), axis_map, inv_freq,
        cache_loc.to(torch.int64).contiguous(), k_cache, v_cache, num_q_heads, num_kv_heads, head_dim, eps,
    )


def create_kv_indices(req_to_token, req_pool_indices, seq_lens, kv_start=None, max_len=None):
    """``(kv_indptr, kv_indices)`` of a batch for callers that want a flat index list (device-side, no loop)."""
    return ref.create_kv_indices(req_to_token, req_pool_indices, seq_lens, kv_start, max_len)


def kv_write(k, v, loc, k_cache, v_cache) -> None:
    if not use_kernels(k) or not _cache_dtype_ok(k_cache, k):
        return ref.kv_write(k, v, loc, k_cache, v_cache)
    ext().kv_write(k, v, loc.to(torch.int64).contiguous(), k_cache, v_cache)


# --------------------------------------------------------------------------
# tensor-parallel reduction fused with residual add + RMSNorm
# --------------------------------------------------------------------------
def tp_reduce_add_rmsnorm(partial: torch.Tensor, residual: Optional[torch.Tensor], weight: Optional[torch.Tensor],
                          eps: float) -> torch.Tensor:
    """``residual += sum over TP ranks of partial`` (in place when given); returns
    ``rmsnorm(residual) * weight`` (or the plain sum when ``weight`` is None).

    On GPUs with peer-mapped buffers this is one kernel that pulls every rank's partial sums over
    NVLink; otherwise it is the process group's all-reduce followed by the local add + norm."""
    from ..parallel import state as pstate
    from ..parallel.symm import get_tp_comm

    comm = get_tp_comm()
    slot = comm.slot_of(partial) if (comm is not None and use_kernels(partial)) else None
    if slot is not None:
        p2 = _2d(partial)
        out = torch.empty((p2.shape[0], p2.shape[1]), dtype=partial.dtype, device=partial.device)
        ext().tp_reduce_add_rmsnorm(slot.data_ptrs, slot.flag_ptrs, slot.seq,
                                    None if residual is None else _2d(residual), weight, out, comm.rank,
                                    slot.data.stride(0), eps)
        return out.view(partial.shape)
    total = pstate.tensor_model_parallel_all_reduce(partial.contiguous() if slot is None else partial.clone())
    if residual is None:
        return total if weight is None else rmsnorm(total, weight, eps)
    if weight is None:
        residual.add_(total)
        return residual
    fused_add_rmsnorm(total, residual, weight, eps)
    return total


# --------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------
# Head sizes the tcgen05 attention kernels take: 128 through the specialised prefill and decode kernels, 64 and 256
# through the single-role kernel.  MLLM_B200_ATTN_HEAD_SIZES=128 sends the other two back to the library / PyTorch
# paths (and the vision towers back to zero-padding their 64-wide heads to 128).
_ATTN_HEAD_SIZES = tuple(int(v) for v in os.environ.get("MLLM_B200_ATTN_HEAD_SIZES", "64,128,256").split(",") if v.strip())
# An 8-bit KV cache (unscaled e4m3 / e5m2) is written by the fused q/k prologue and the cache-write kernel and read
# by the single-role attention kernel, which widens a tile on its way into shared memory.  MLLM_B200_KV8_KERNELS=0
# sends such a cache back to the library / PyTorch paths.
_KV8_KERNELS = os.environ.get("MLLM_B200_KV8_KERNELS", "1") != "0"
_KV8_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)


def _cache_dtype_ok(cache: torch.Tensor, act: torch.Tensor) -> bool:
    return cache.dtype == act.dtype or (_KV8_KERNELS and cache.dtype in _KV8_DTYPES)


def attention_kernels_cover(head_dim: int, cache_dtype, act_dtype) -> bool:
    """Whether attention of this head size over a cache of this dtype runs on the package's kernels."""
    return head_dim in _ATTN_HEAD_SIZES and (cache_dtype == act_dtype or (_KV8_KERNELS and cache_dtype in _KV8_DTYPES))


def _attention_kernel_ok(q: torch.Tensor, k_cache: torch.Tensor, window, logit_cap) -> bool:
    """The tcgen05 attention kernels cover head sizes 64, 128 and 256 (causal, optionally with a sliding window and a
    soft cap on the scores) and a cache of the activation dtype or of an unscaled 8-bit float."""
    return use_kernels(q) and q.shape[-1] in _ATTN_HEAD_SIZES and _cache_dtype_ok(k_cache, q)


def attention_prefill(q, k_cache, v_cache, req_to_token, req_pool_indices, seq_lens, prefix_lens,
                      q_start_loc, scale: float, out=None, max_q_len: int = 0, window: Optional[int] = None,
                      logit_cap: float = 0.0, seq_lens_cpu=None, prefix_lens_cpu=None) -> torch.Tensor:
    """Causal attention of new tokens over cached prefix + themselves.  ``window``: sliding-window attention
    (each query sees its last ``window`` keys); ``logit_cap``: soft-capping of the scores; both are mask /
    score options of the tcgen05 kernels.  Head sizes other than 64 / 128 / 256 and caches that hold neither the
    activation dtype nor an 8-bit float take library / PyTorch fallbacks."""
    if _attention_kernel_ok(q, k_cache, window, logit_cap) and hasattr(ext(), "attention_prefill"):
        if out is None:
            out = torch.empty((q.shape[0], q.shape[1], q.shape[2]), dtype=q.dtype, device=q.device)
        ext().attention_prefill(q, k_cache, v_cache, req_to_token, req_pool_indices, seq_lens, prefix_lens,
                                q_start_loc, scale, out, max_q_len, True, int(window or 0), float(logit_cap or 0.0))
        return out
    if q.is_cuda and not logit_cap:
        o = ref.attention_prefill_sdpa(q, k_cache, v_cache, req_to_token, req_pool_indices, seq_lens, prefix_lens,
                                       q_start_loc, scale, seq_lens_cpu, prefix_lens_cpu, window)
        if out is None:
            return o
        out.copy_(o)
        return out
    return ref.attention_prefill(q, k_cache, v_cache, req_to_token, req_pool_indices, seq_lens, prefix_lens,
                                 q_start_loc, scale, out, window=window, logit_cap=logit_cap)


def attention_decode(q, k_cache, v_cache, req_to_token, req_pool_indices, seq_lens, scale: float,
                     out=None, max_seq_len: int = 0, window: Optional[int] = None, logit_cap: float = 0.0) -> torch.Tensor:
    if _attention_kernel_ok(q, k_cache, window, logit_cap) and hasattr(ext(), "attention_decode"):
        if out is None:
            out = torch.empty((q.shape[0], q.shape[1], q.shape[2]), dtype=q.dtype, device=q.device)
        ext().attention_decode(q, k_cache, v_cache, req_to_token, req_pool_indices, seq_lens, scale, out, max_seq_len,
                               int(window or 0), float(logit_cap or 0.0))
        return out
    if q.is_cuda and max_seq_len:
        return ref.attention_decode_batched(q, k_cache, v_cache, req_to_token, req_pool_indices, seq_lens, scale,
                                            max_seq_len, out, window, logit_cap)
    return ref.attention_decode(q, k_cache, v_cache, req_to_token, req_pool_indices, seq_lens, scale, out,
                                window=window, logit_cap=logit_cap)


def attention_varlen_bidirectional(q, k, v, cu_seqlens, scale: float) -> torch.Tensor:
    """Bidirectional attention inside each segment; q, k, v [T, H, D].  On the GPU the tcgen05 prefill kernel runs
    without its causal mask, every segment being one "request" whose keys sit at rows ``cu[i]..cu[i+1]`` of k / v;
    a head size the kernel has no instantiation for is zero-padded to 128."""
    if not use_kernels(q) or (q.shape[-1] > 128 and q.shape[-1] not in _ATTN_HEAD_SIZES):
        return ref.attention_varlen_bidirectional(q, k, v, cu_seqlens.cu_host if isinstance(cu_seqlens, VarlenPlan) else cu_seqlens,
                                                  scale)
    D = q.shape[-1]
    if D not in _ATTN_HEAD_SIZES:
        pad = (0, 128 - D)
        q, k, v = (torch.nn.functional.pad(t, pad) for t in (q, k, v))
    return _varlen_bidirectional_padded(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens, scale)[..., :D]


class VarlenPlan:
    """Everything the bidirectional variable-length attention needs besides q, k, v, built once for a set of
    segment boundaries and reused by every block of a vision tower (and captured with it in a CUDA graph): the
    device copies of the boundaries and lengths, the row table that lets the prefill kernel see every segment as
    one request, and the host-side maximum length."""

    def __init__(self, cu_seqlens: torch.Tensor, total_rows: int, device) -> None:
        self.cu_host = cu_seqlens.cpu()
        lens_host = (self.cu_host[1:] - self.cu_host[:-1]).tolist()
        self.max_len = int(max(lens_host)) if lens_host else 0
        self.n = len(lens_host)
        dev = torch.device(device)
        if dev.type != "cuda":
            return
        cu = self.cu_host.to(device=dev, dtype=torch.int32)
        self.lens = (cu[1:] - cu[:-1]).contiguous()
        self.starts = cu[:-1].contiguous()
        rtt = self.starts.unsqueeze(1) + torch.arange(self.max_len, device=dev, dtype=torch.int32).unsqueeze(0)
        self.rtt = rtt.clamp_(max=max(0, total_rows - 1)).contiguous()
        self.req = torch.arange(self.n, device=dev, dtype=torch.int32)
        self.zeros = torch.zeros(self.n, device=dev, dtype=torch.int32)


def _varlen_bidirectional_padded(q, k, v, cu_seqlens, scale: float) -> torch.Tensor:
    plan = cu_seqlens if isinstance(cu_seqlens, VarlenPlan) else VarlenPlan(cu_seqlens, q.shape[0], q.device)
    out = torch.empty_like(q)
    ext().attention_prefill(q, k, v, plan.rtt, plan.req, plan.lens, plan.zeros, plan.starts, scale, out, plan.max_len,
                            False, 0, 0.0)
    return out


def vision_attention(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, cu_seqlens: torch.Tensor, num_heads: int,
                     scale: float) -> torch.Tensor:
    """ViT attention block core: qkv [T, 3 * H * D] -> 2-D rotary on q, k -> bidirectional attention per
    image -> [T, H * D]."""
    T = qkv.shape[0]
    D = qkv.shape[1] // (3 * num_heads)
    q4 = qkv.view(T, 3, num_heads, D)
    if use_kernels(qkv) and D <= 128 and D % 2 == 0:
        width = D if D in _ATTN_HEAD_SIZES else 128              # 64-wide heads run unpadded
        q = torch.empty((T, num_heads, width), dtype=qkv.dtype, device=qkv.device)
        k, v = torch.empty_like(q), torch.empty_like(q)
        cos32 = cos if (cos.dtype == torch.float32 and cos.is_contiguous()) else cos.float().contiguous()
        sin32 = sin if (sin.dtype == torch.float32 and sin.is_contiguous()) else sin.float().contiguous()
        ext().vision_rope_split_pad(q4.contiguous(), cos32, sin32, q, k, v)
        o = _varlen_bidirectional_padded(q, k, v, cu_seqlens, scale)
        return o[..., :D].reshape(T, num_heads * D)
    if isinstance(cu_seqlens, VarlenPlan):
        cu_seqlens = cu_seqlens.cu_host
    q, k, v = q4.unbind(1)
    q, k = ref.vision_rope(q, cos, sin), ref.vision_rope(k, cos, sin)
    return ref.attention_varlen_bidirectional(q, k, v, cu_seqlens, scale).reshape(T, num_heads * D)


def vision_pos_embed_add(x: torch.Tensor, table: torch.Tensor, idx: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    if not use_kernels(x):
        return ref.vision_pos_embed_add(x, table, idx, w)
    x = x.contiguous()
    ext().vision_pos_embed_add(x, table, idx.contiguous(), w.float().contiguous())
    return x


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    if not use_kernels(x):
        return ref.gelu_erf(x)
    xc = x.contiguous()
    out = torch.empty_like(xc)
    ext().gelu_erf(xc, out)
    return out


# --------------------------------------------------------------------------
# gated delta net (linear attention of the hybrid models)
# --------------------------------------------------------------------------
def rmsnorm_gated(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if use_kernels(x) and hasattr(ext(), "rmsnorm_gated") and x.shape[-1] % 8 == 0:
        x2, g2 = _2d(x).contiguous(), _2d(gate).contiguous()
        out = torch.empty_like(x2)
        ext().rmsnorm_gated(x2, g2, weight, out, eps)
        return out.view(x.shape)
    return ref.rmsnorm_gated(x, gate, weight, eps)


def causal_conv1d_silu(x, weight, conv_state, state_indices, seq_lens, has_state, q_start=None) -> torch.Tensor:
    """Depth-wise causal conv (kernel K) + SiLU over the new tokens of every request, reading / updating
    the per-request history rows of ``conv_state``.  ``seq_lens`` / ``has_state`` may be host lists (CPU
    path) or device int32 tensors (GPU path, no host sync; ``q_start`` = first row of each request)."""
    if use_kernels(x) and hasattr(ext(), "gdn_conv1d_silu"):
        dev = x.device
        lens = seq_lens if isinstance(seq_lens, torch.Tensor) else torch.tensor(list(seq_lens), dtype=torch.int32, device=dev)
        has = has_state if isinstance(has_state, torch.Tensor) else torch.tensor([int(h) for h in has_state], dtype=torch.int32, device=dev)
        if q_start is None:
            q_start = torch.cumsum(lens, 0, dtype=torch.int32) - lens
        out = torch.empty_like(x)
        ext().gdn_conv1d_silu(x.contiguous(), weight.contiguous(), conv_state, state_indices.to(torch.int32), lens.to(torch.int32),
                              has.to(torch.int32), q_start.to(torch.int32), out)
        return out
    lens = seq_lens.tolist() if isinstance(seq_lens, torch.Tensor) else seq_lens
    has = has_state.tolist() if isinstance(has_state, torch.Tensor) else has_state
    return ref.causal_conv1d_silu(x, weight, conv_state, state_indices, lens, has)


_GDN_EXTEND_BACKEND = "auto"


def set_gdn_extend_backend(name: str) -> None:
    """How the gated delta rule runs on new tokens (``--server.gdn_extend_backend``).  ``pytorch``: the chunk-parallel
    PyTorch form on every device; ``cuda_chunkwise``: the chunk-parallel CUDA kernel for every batch; ``mllm_kernel``:
    the token-sequential CUDA kernel for every batch; anything else: the chunk-parallel kernel for batches that
    average 32 new tokens per request or more (prefill), the sequential one otherwise (decode, short extends)."""
    global _GDN_EXTEND_BACKEND
    _GDN_EXTEND_BACKEND = str(name)


def gated_delta_rule(q, k, v, g, beta, state, state_indices, seq_lens, has_state, q_start=None) -> torch.Tensor:
    """Gated delta rule over ragged sequences with per-request recurrent state (read when ``has_state``,
    always written back).  q, k [T, H, Dk], v [T, H, Dv], g / beta [T, H] fp32."""
    if (use_kernels(q) and hasattr(ext(), "gdn_recurrent") and q.shape[-1] == 128 and v.shape[-1] == 128
            and _GDN_EXTEND_BACKEND != "pytorch"):
        dev = q.device
        lens = seq_lens if isinstance(seq_lens, torch.Tensor) else torch.tensor(list(seq_lens), dtype=torch.int32, device=dev)
        has = has_state if isinstance(has_state, torch.Tensor) else torch.tensor([int(h) for h in has_state], dtype=torch.int32, device=dev)
        if q_start is None:
            q_start = torch.cumsum(lens, 0, dtype=torch.int32) - lens
        out = torch.empty_like(v)
        chunked = _GDN_EXTEND_BACKEND == "cuda_chunkwise" or (
            _GDN_EXTEND_BACKEND != "mllm_kernel" and q.shape[0] >= 32 * max(1, lens.numel()))
        rule = ext().gdn_chunk if chunked and hasattr(ext(), "gdn_chunk") else ext().gdn_recurrent
        rule(q.contiguous(), k.contiguous(), v.contiguous(), g.float().contiguous(), beta.float().contiguous(),
             state, state_indices.to(torch.int32), lens.to(torch.int32), has.to(torch.int32), q_start.to(torch.int32), out)
        return out
    lens = seq_lens.tolist() if isinstance(seq_lens, torch.Tensor) else seq_lens
    has = has_state.tolist() if isinstance(has_state, torch.Tensor) else has_state
    if max(lens, default=0) > 16:  # prefill: the chunk-parallel form (matrix products) instead of a token loop
        return ref.gated_delta_rule_chunked(q, k, v, g, beta, state, state_indices, lens, has)
    return ref.gated_delta_rule(q, k, v, g, beta, state, state_indices, lens, has)


# --------------------------------------------------------------------------
# mixture of experts
# --------------------------------------------------------------------------
def moe_router_topk(hidden: torch.Tensor, gate_weight: torch.Tensor, top_k: int, renormalize: bool = True):
    """Router: fp32 softmax over experts -> sorted top-k -> optional renormalisation."""
    if use_kernels(hidden) and hasattr(ext(), "moe_router_topk") and gate_weight.shape[0] <= 256 and top_k <= 8:
        logits = linear(hidden, gate_weight)  # [T, E] on the tensor cores; the kernel does the rest in fp32
        T = hidden.shape[0]
        w = torch.empty((T, top_k), dtype=torch.float32, device=hidden.device)
        ids = torch.empty((T, top_k), dtype=torch.int32, device=hidden.device)
        ext().moe_router_topk(logits, w, ids, renormalize)
        return w, ids
    return ref.moe_router_topk(hidden, gate_weight, top_k, renormalize)


def moe_chunk_rows(tokens: int, top_k: int, num_experts_global: int) -> int:
    """MMA N (rows of one expert handled per work item) for the grouped GEMM: about twice the mean
    number of rows per expert, within the instruction's 16..128 range."""
    avg = max(1, (tokens * top_k + num_experts_global - 1) // num_experts_global)
    for bn in (16, 32, 64):
        if 2 * avg <= bn + bn // 2:
            return bn
    return 128


def _moe_gemm(x, w, out, offsets, work, n_work, bn, swiglu) -> None:
    rc = ext().moe_grouped_gemm(x, w, out, offsets, work, n_work, bn, swiglu)
    if rc != 0:
        raise RuntimeError(f"mllm_b200 moe_grouped_gemm: unsupported shape or launch failure (code {rc}) for "
                           f"x={tuple(x.shape)} w={tuple(w.shape)}")


def moe_experts(x, w13, w2, topk_w, topk_ids, expert_offset: int = 0, swiglu_block: int = 0,
                num_experts_global: Optional[int] = None) -> torch.Tensor:
    """Grouped expert MLPs.  On the GPU everything stays on the device (no host read of the routing,
    so the step can be captured in a CUDA graph): pairs are counting-sorted by expert, activations
    gathered into expert order, both expert GEMMs run as one grouped tcgen05 launch each (SwiGLU fused
    into the first when ``w13`` is stored in 128-row gate/up blocks), and the k results per token are
    summed with the router weights."""
    if not use_kernels(x):
        return ref.moe_experts(x, w13, w2, topk_w, topk_ids, expert_offset, swiglu_block)
    if swiglu_block not in (0, SWIGLU_BLOCK):
        raise ValueError(f"w13 interleave block must be 0 or {SWIGLU_BLOCK}")
    T, H = x.shape
    E, N13, _ = w13.shape
    inter = N13 // 2
    k = topk_ids.shape[1]
    P = T * k
    dev = x.device
    bn = moe_chunk_rows(T, k, num_experts_global or E)
    max_work = E + (P + bn - 1) // bn
    i32 = dict(dtype=torch.int32, device=dev)
    sorted_pos = torch.empty(P, **i32)
    src_token = torch.empty(P, **i32)
    offsets = torch.empty(E + 1, **i32)
    work = torch.empty((max_work, 2), **i32)
    n_work = torch.empty(1, **i32)
    e = ext()
    ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
    e.moe_align(ids.contiguous(), int(expert_offset), E, bn, sorted_pos, src_token, offsets, work, n_work)
    xs = torch.empty((P, H), dtype=x.dtype, device=dev)
    e.moe_gather(x, src_token, offsets, xs)
    h = torch.empty((P, inter), dtype=x.dtype, device=dev)
    if swiglu_block:
        _moe_gemm(xs, w13, h, offsets, work, n_work, bn, True)
    else:
        gu = torch.empty((P, N13), dtype=x.dtype, device=dev)
        _moe_gemm(xs, w13, gu, offsets, work, n_work, bn, False)
        e.act_and_mul(gu, h, 0)
    ys = torch.empty((P, H), dtype=x.dtype, device=dev)
    _moe_gemm(h, w2, ys, offsets, work, n_work, bn, False)
    out = torch.empty((T, H), dtype=x.dtype, device=dev)
    e.moe_combine(ys, sorted_pos, topk_w.contiguous(), out)
    return out


def ep_moe_exchange(x_own, w13, w2, topk_w, topk_ids, swiglu_block: int, comm) -> torch.Tensor:
    """Expert-parallel MoE for the token rows this rank owns (``x_own [T/ep, H]``, routed here: ``topk_ids`` are
    global expert ids): the rows travel to the ranks that own their experts, run through the grouped expert GEMMs
    there, come back and are summed with the router weights.  Everything stays on the device; the flags that
    order the exchange are epochs in peer-mapped memory, waited for with a bound."""
    if swiglu_block != SWIGLU_BLOCK:
        raise ValueError("the expert-parallel exchange needs w13 in 128-row gate / up blocks")
    T, H = x_own.shape
    k = topk_ids.shape[1]
    E_local, N13, _ = w13.shape
    inter = N13 // 2
    e = ext()
    epoch = comm.next_epoch()
    bn = moe_chunk_rows(T * comm.world, k, comm.experts)
    ids = (topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)).contiguous()
    x2 = x_own if x_own.stride(-1) == 1 and (x_own.stride(0) * x_own.element_size()) % 16 == 0 else x_own.contiguous()

    def check(rc, what):
        if rc != 0:
            raise RuntimeError(f"mllm_b200 {what} failed (code {rc})")

    check(e.ep_plan(ids, comm.ptrs, comm.rank, comm.experts, H, comm.cap_rows, epoch, bn, comm.pair_dst_rank,
                    comm.pair_dst_row, comm.expert_offsets, comm.work, comm.n_work, comm.recv_rows), "ep_plan")
    check(e.ep_dispatch(x2, k, comm.pair_dst_rank, comm.pair_dst_row, comm.ptrs, comm.rank, comm.experts, comm.cap_rows,
                        epoch, comm.done[0:1]), "ep_dispatch")
    check(e.tp_wait_flags(comm.disp_flags, comm.world, epoch), "ep dispatch wait")
    h = torch.empty((comm.cap_rows, inter), dtype=x_own.dtype, device=x_own.device)
    _moe_gemm(comm.recv_x, w13, h, comm.expert_offsets, comm.work, comm.n_work, bn, True)
    ys = torch.empty((comm.cap_rows, H), dtype=x_own.dtype, device=x_own.device)
    _moe_gemm(h, w2, ys, comm.expert_offsets, comm.work, comm.n_work, bn, False)
    check(e.ep_return(ys, comm.recv_rows, comm.ptrs, comm.rank, comm.experts, epoch, comm.done[1:2]), "ep_return")
    check(e.tp_wait_flags(comm.ret_flags, comm.world, epoch), "ep return wait")
    out = torch.empty((T, H), dtype=x_own.dtype, device=x_own.device)
    e.moe_combine(comm.ret_y[: T * k], comm.pair_index[: T * k], topk_w.contiguous(), out)
    return out


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not use_kernels(logits):
        r = ref.argmax(logits)
        if out is not None:
            out.copy_(r)
            return out
        return r
    l2 = _2d(logits)
    if l2.stride(-1) != 1:
        l2 = l2.contiguous()
    o = torch.empty((l2.shape[0],), dtype=torch.int64, device=logits.device) if out is None else out
    ext().argmax(l2, o)
    return o


def apply_penalties(logits, output_counts, prompt_mask, frequency_penalty, presence_penalty, repetition_penalty):
    """Frequency / presence / repetition penalties; returns fp32 logits."""
    if not use_kernels(logits):
        return ref.apply_penalties(logits, output_counts, prompt_mask, frequency_penalty, presence_penalty,
                                   repetition_penalty)
    lf = logits.float().contiguous()
    if lf.data_ptr() == logits.data_ptr():
        lf = lf.clone()
    pm = None if prompt_mask is None else prompt_mask.to(torch.uint8).contiguous()
    ext().apply_penalties(lf, output_counts.to(torch.int32).contiguous(), pm, frequency_penalty.float().contiguous(),
                          presence_penalty.float().contiguous(), repetition_penalty.float().contiguous())
    return lf


def top_k_top_p_min_p_sample(logits, temperature, top_k, top_p, min_p, uniform) -> torch.Tensor:
    """One token per row: temperature, top-k, top-p, min-p, inverse-CDF draw (one kernel, no sort)."""
    if not use_kernels(logits):
        return ref.top_k_top_p_min_p_sample(logits, temperature, top_k, top_p, min_p, uniform)
    l2 = _2d(logits)
    if l2.stride(-1) != 1:
        l2 = l2.contiguous()
    out = torch.empty((l2.shape[0],), dtype=torch.int64, device=logits.device)
    ext().sample(l2, temperature.float().contiguous(), top_k.to(torch.int32).contiguous(), top_p.float().contiguous(),
                 None if min_p is None else min_p.float().contiguous(), uniform.float().contiguous(), out)
    return out
