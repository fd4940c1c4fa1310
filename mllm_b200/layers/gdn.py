"""Gated DeltaNet token mixer of the Qwen3.5 hybrid models (roles of pymllm/layers/gated_delta_net.py,
layers/attention/gdn_backend.py and rms_norm_gated.py; math of HF ``Qwen3_5GatedDeltaNet``):

    qkv = conv1d_silu(in_proj_qkv(x))      depth-wise causal conv over the last 4 inputs, SiLU
    beta = sigmoid(in_proj_b(x)),  g = -exp(A_log) * softplus(in_proj_a(x) + dt_bias)
    S <- S * exp(g);  S <- S + k (x) ((v - S^T k) * beta);  o = S^T q      (q, k l2-normalised, q / sqrt(Dk))
    y = out_proj( rmsnorm(o) * w * silu(in_proj_z(x)) )

State (recurrent matrix and conv history) lives in a :class:`GDNPool` row per request, so prefill of a
continuation (chunked prefill) and decode both resume from it.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..parallel import state as pstate


class GatedDeltaNet(nn.Module):
    def __init__(self, config, layer_id: int, gdn_index: int, params_dtype=None, prefix: str = "") -> None:
        super().__init__()
        dt = params_dtype or torch.get_default_dtype()
        H = config.hidden_size
        self.layer_id, self.gdn_index = layer_id, gdn_index
        # tensor parallelism: every rank owns num_heads / tp value heads with their key heads (the
        # recurrent state, the convolution channels and the gates are per head, so nothing is exchanged
        # until the row-parallel output projection, whose partial sums are all-reduced)
        self.tp, self.tp_rank = pstate.get_tensor_model_parallel_world_size(), pstate.get_tensor_model_parallel_rank()
        hv, hk = config.linear_num_value_heads, config.linear_num_key_heads
        if hv % self.tp or hk % self.tp:
            raise ValueError(f"gated delta net: {hk} key / {hv} value heads do not divide over {self.tp} ranks")
        self.total_k_heads, self.total_v_heads = hk, hv
        self.num_v_heads, self.num_k_heads = hv // self.tp, hk // self.tp
        self.head_k_dim, self.head_v_dim = config.linear_key_head_dim, config.linear_value_head_dim
        self.key_dim, self.value_dim = self.head_k_dim * self.num_k_heads, self.head_v_dim * self.num_v_heads
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.conv_kernel = config.linear_conv_kernel_dim
        self.eps = getattr(config, "rms_norm_eps", 1e-6)

        def w(*shape, loader=None, dtype=dt, init=None):
            t = torch.empty(*shape, dtype=dtype) if init is None else torch.full(shape, init, dtype=dtype)
            p = nn.Parameter(t, requires_grad=False)
            if loader is not None:
                p.weight_loader = loader
            return p

        self.in_proj_qkv = nn.Module()
        self.in_proj_qkv.weight = w(self.conv_dim, H, loader=self._load_qkv_rows)
        self.in_proj_z = nn.Module()
        self.in_proj_z.weight = w(self.value_dim, H, loader=self._load_v_rows)
        self.in_proj_b = nn.Module()
        self.in_proj_b.weight = w(self.num_v_heads, H, loader=self._load_v_rows)
        self.in_proj_a = nn.Module()
        self.in_proj_a.weight = w(self.num_v_heads, H, loader=self._load_v_rows)
        self.conv1d = nn.Module()
        self.conv1d.weight = w(self.conv_dim, self.conv_kernel, loader=self._load_qkv_rows)
        self.dt_bias = w(self.num_v_heads, loader=self._load_v_rows, dtype=torch.float32, init=1.0)
        self.A_log = w(self.num_v_heads, loader=self._load_v_rows, dtype=torch.float32, init=0.0)
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(self.head_v_dim, dtype=dt), requires_grad=False)
        self.out_proj = nn.Module()
        self.out_proj.weight = w(H, self.value_dim, loader=self._load_v_cols)

    # ---- loading: slices of the full (unsharded) checkpoint tensors ----
    def _load_qkv_rows(self, param, full, shard_id=None) -> None:
        """Rows are [q heads | k heads | v heads]; take this rank's heads of each block (also the layout
        of the convolution channels, whose checkpoint shape is [C, 1, K])."""
        full = full.reshape(full.shape[0], -1)
        kd, vd = self.head_k_dim * self.total_k_heads, self.head_v_dim * self.total_v_heads
        q, k, v = full[:kd], full[kd:2 * kd], full[2 * kd:2 * kd + vd]
        r = self.tp_rank
        param.data.copy_(torch.cat([q[r * self.key_dim:(r + 1) * self.key_dim], k[r * self.key_dim:(r + 1) * self.key_dim],
                                    v[r * self.value_dim:(r + 1) * self.value_dim]], 0).reshape(param.shape))

    def _load_v_rows(self, param, full, shard_id=None) -> None:
        n = param.shape[0]
        param.data.copy_(full[self.tp_rank * n:(self.tp_rank + 1) * n].reshape(param.shape))

    def _load_v_cols(self, param, full, shard_id=None) -> None:
        n = param.shape[1]
        param.data.copy_(full[:, self.tp_rank * n:(self.tp_rank + 1) * n])

    def forward(self, x: torch.Tensor, fb) -> torch.Tensor:
        pool = fb.extra["gdn_pool"]
        recurrent, conv = pool.layer(self.gdn_index)
        T = x.shape[0]
        slots = fb.req_pool_indices
        if fb.forward_mode.is_decode():
            lens = fb.extra.get("gdn_ones")
            if lens is None:
                lens = torch.ones(fb.batch_size, dtype=torch.int32, device=x.device)
                fb.extra["gdn_ones"] = lens
            has, q_start = lens, torch.arange(fb.batch_size, dtype=torch.int32, device=x.device)
        else:
            lens = fb.extend_seq_lens.to(torch.int32)
            has = (fb.extend_prefix_lens > 0).to(torch.int32)
            q_start = fb.extend_start_loc.to(torch.int32) if fb.extend_start_loc is not None else None
        qkv = ops.linear(x, self.in_proj_qkv.weight)
        z = ops.linear(x, self.in_proj_z.weight)
        ba = ops.linear(x, torch.cat([self.in_proj_b.weight, self.in_proj_a.weight], 0)) if not hasattr(self, "_ba") else \
            ops.linear(x, self._ba)
        b, a = ba[:, : self.num_v_heads], ba[:, self.num_v_heads:]
        qkv = ops.causal_conv1d_silu(qkv, self.conv1d.weight, conv, slots, lens, has, q_start)
        q, k, v = torch.split(qkv, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q = q.reshape(T, self.num_k_heads, self.head_k_dim)
        k = k.reshape(T, self.num_k_heads, self.head_k_dim)
        v = v.reshape(T, self.num_v_heads, self.head_v_dim)
        rep = self.num_v_heads // self.num_k_heads
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
        beta = torch.sigmoid(b.float())
        g = -torch.exp(self.A_log.float()) * torch.nn.functional.softplus(a.float() + self.dt_bias.float())
        o = ops.gated_delta_rule(q, k, v, g, beta, recurrent, slots, lens, has, q_start)
        o = ops.rmsnorm_gated(o.reshape(-1, self.head_v_dim), z.reshape(-1, self.head_v_dim), self.norm.weight, self.eps)
        y = ops.linear(o.reshape(T, self.value_dim), self.out_proj.weight)
        return pstate.tensor_model_parallel_all_reduce(y) if self.tp > 1 else y

    def fuse_small_projections(self) -> None:
        """One GEMM for the beta / decay projections (call after loading)."""
        self._ba = torch.cat([self.in_proj_b.weight.data, self.in_proj_a.weight.data], 0).contiguous()
