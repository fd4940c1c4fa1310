"""MiniCPM4 decoder against a plain fp32 restatement of its forward pass (embedding, residual and logit
constants; ``longrope`` rotary factors with their attention factor), prefill in two chunks then decode; tied and
untied output projection."""
import math
import types

import pytest
import torch

from mllm_b200.configs import ServerConfig
from mllm_b200.executor import ModelRunner

V, H, I, L, HQ, HKV, D = 300, 64, 96, 3, 4, 2, 16
ORIG, MAXPOS = 16, 128
SHORT = [1.0, 1.0, 1.05, 1.1, 1.2, 1.3, 1.4, 1.5]
LONG = [1.0, 1.3, 1.9, 2.7, 4.2, 6.5, 7.5, 8.0]


def weights(tied, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g) * 0.08  # noqa: E731
    sd = {"model.embed_tokens.weight": r(V, H), "model.norm.weight": 1 + r(H)}
    if not tied:
        sd["lm_head.weight"] = r(V, H)
    for i in range(L):
        p = f"model.layers.{i}."
        sd.update({p + "self_attn.q_proj.weight": r(HQ * D, H), p + "self_attn.k_proj.weight": r(HKV * D, H),
                   p + "self_attn.v_proj.weight": r(HKV * D, H), p + "self_attn.o_proj.weight": r(H, HQ * D),
                   p + "input_layernorm.weight": 1 + r(H), p + "post_attention_layernorm.weight": 1 + r(H),
                   p + "mlp.gate_proj.weight": r(I, H), p + "mlp.up_proj.weight": r(I, H), p + "mlp.down_proj.weight": r(H, I)})
    return sd


def oracle(sd, ids, cfg):
    """Logits of the last position of ``ids`` [T]."""
    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    T = ids.numel()
    ext = torch.tensor(LONG if MAXPOS > ORIG else SHORT)
    inv = 1.0 / (ext * cfg.rope_theta ** (torch.arange(0, D, 2).float() / D))
    af = math.sqrt(1 + math.log(MAXPOS / ORIG) / math.log(ORIG))
    ang = torch.arange(T).float()[:, None] * inv[None]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1) * af, torch.cat([ang.sin(), ang.sin()], -1) * af

    def rope(x):                                              # [T, heads, D], half rotation
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return x * cos[:, None] + torch.cat([-x2, x1], -1) * sin[:, None]

    s = cfg.scale_depth / math.sqrt(L)
    h = sd["model.embed_tokens.weight"][ids] * cfg.scale_emb
    mask = torch.full((T, T), float("-inf")).triu(1)
    for i in range(L):
        p = f"model.layers.{i}."
        x = norm(h, sd[p + "input_layernorm.weight"])
        q = rope((x @ sd[p + "self_attn.q_proj.weight"].T).view(T, HQ, D))
        k = rope((x @ sd[p + "self_attn.k_proj.weight"].T).view(T, HKV, D)).repeat_interleave(HQ // HKV, 1)
        v = (x @ sd[p + "self_attn.v_proj.weight"].T).view(T, HKV, D).repeat_interleave(HQ // HKV, 1)
        att = torch.softmax(torch.einsum("thd,shd->hts", q, k) / math.sqrt(D) + mask, -1)
        o = torch.einsum("hts,shd->thd", att, v).reshape(T, HQ * D)
        h = h + (o @ sd[p + "self_attn.o_proj.weight"].T) * s
        x = norm(h, sd[p + "post_attention_layernorm.weight"])
        m = torch.nn.functional.silu(x @ sd[p + "mlp.gate_proj.weight"].T) * (x @ sd[p + "mlp.up_proj.weight"].T)
        h = h + (m @ sd[p + "mlp.down_proj.weight"].T) * s
    h = norm(h, sd["model.norm.weight"]) / (H / cfg.dim_model_base)
    return h[-1] @ sd.get("lm_head.weight", sd["model.embed_tokens.weight"]).T


@pytest.mark.parametrize("tied", [False, True])
def test_minicpm4_matches_plain_forward(tied):
    cfg = types.SimpleNamespace(
        architectures=["MiniCPMForCausalLM"], vocab_size=V, hidden_size=H, intermediate_size=I, num_hidden_layers=L,
        num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=D, rms_norm_eps=1e-5, tie_word_embeddings=tied,
        max_position_embeddings=MAXPOS, hidden_act="silu", rope_theta=10000.0, scale_emb=12.0, scale_depth=1.4,
        dim_model_base=16,
        rope_scaling=dict(rope_type="longrope", short_factor=SHORT, long_factor=LONG, original_max_position_embeddings=ORIG))
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=512),
                     hf_config=cfg, device="cpu")
    mr.initialize()
    assert type(mr.model).__name__ == "MiniCPMForCausalLM"
    sd = weights(tied)
    loaded = mr.model.load_weights(sd.items())
    assert not set(dict(mr.model.named_parameters())) - loaded
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    ids = torch.randint(0, V, (30,), generator=torch.Generator().manual_seed(1))
    slots = mr.req_to_token_pool.alloc(1)
    sl = torch.tensor(slots)
    loc = mr.token_to_kv_pool_allocator.alloc(30)
    mr.req_to_token_pool.req_to_token[slots[0], :30] = loc.int()
    mr.forward(mr.prepare_forward_batch_extend(ids[:13], sl, torch.tensor([13]), torch.tensor([13]), torch.tensor([0]), loc[:13]))
    got = mr.forward(mr.prepare_forward_batch_extend(ids[13:], sl, torch.tensor([30]), torch.tensor([17]), torch.tensor([13]),
                                                     loc[13:])).next_token_logits[0]
    torch.testing.assert_close(got, oracle(sd, ids, cfg), atol=5e-4, rtol=5e-4)
    nxt = got.argmax().view(1)
    loc1 = mr.token_to_kv_pool_allocator.alloc(1)
    mr.req_to_token_pool.req_to_token[slots[0], 30] = loc1.int()
    got = mr.forward(mr.prepare_forward_batch_decode(nxt, sl, torch.tensor([31]), loc1)).next_token_logits[0]
    torch.testing.assert_close(got, oracle(sd, torch.cat([ids, nxt]), cfg), atol=5e-4, rtol=5e-4)


def test_residual_constant_goes_into_quantisation_scales_not_integers():
    from mllm_b200.models.minicpm import MiniCPMForCausalLM

    m = MiniCPMForCausalLM.__new__(MiniCPMForCausalLM)
    m.residual_scale, m.logit_divisor = 0.5, 4.0
    items = [("model.layers.0.mlp.down_proj.weight_packed", torch.full((4, 2), 7, dtype=torch.int32)),
             ("model.layers.0.mlp.down_proj.weight_scale", torch.ones(4, 1, dtype=torch.bfloat16)),
             ("model.layers.0.self_attn.o_proj.scales", torch.ones(2, 4, dtype=torch.float16)),
             ("model.layers.0.self_attn.o_proj.qweight", torch.full((1, 4), 3, dtype=torch.int32)),
             ("model.layers.0.self_attn.q_proj.weight", torch.ones(4, 4)),
             ("model.layers.0.mlp.down_proj.weight", torch.ones(4, 4).to(torch.float8_e4m3fn)),
             ("model.norm.weight", torch.full((4,), 2.0))]
    out = dict(m._folded(items))
    assert out["model.layers.0.mlp.down_proj.weight_packed"].eq(7).all()
    assert out["model.layers.0.self_attn.o_proj.qweight"].eq(3).all()
    assert out["model.layers.0.mlp.down_proj.weight_scale"].float().eq(0.5).all()
    assert out["model.layers.0.self_attn.o_proj.scales"].float().eq(0.5).all()
    assert out["model.layers.0.self_attn.q_proj.weight"].eq(1).all()
    assert out["model.layers.0.mlp.down_proj.weight"].dtype == torch.float8_e4m3fn        # untouched: its scale carries it
    assert out["model.norm.weight"].eq(0.5).all()
