"""CPU oracle / timed CPU baseline: a Qwen3-shaped decoder with seeded N(0, 0.02) weights, a uniform
random prompt, greedy decoding — run by the stand-alone C++ implementation (`csrc/host/cpu_oracle.cpp`)
and, optionally, checked against the PyTorch fp32 statement of the model.

    python -m mllm_b200.benchmarks.cpu_oracle --preset qwen3-0.6b --prompt-len 128 --new-tokens 32 [--check]

Weights are written once to a `.mllm` file (fp32) that both implementations read.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time
from typing import Dict, Iterator, List, Tuple

import torch

from ..io.mllm_file import write_mllm
from ..mem_cache.native import host_ext
from ..models.presets import get_preset


def config_dict(cfg) -> Dict[str, object]:
    rp = getattr(cfg, "rope_parameters", None) or {}
    return dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, rms_norm_eps=float(cfg.rms_norm_eps),
                rope_theta=float(getattr(cfg, "rope_theta", None) or rp.get("rope_theta", 1e6)),
                tie_word_embeddings=bool(getattr(cfg, "tie_word_embeddings", False)))


def seeded_weights(cfg, seed: int = 0, std: float = 0.02) -> Iterator[Tuple[str, torch.Tensor]]:
    """HF-named fp32 tensors: N(0, std) matrices, unit norm gains."""
    g = torch.Generator().manual_seed(seed)
    H, D, I, V = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size

    def mat(*shape):
        return torch.randn(*shape, generator=g) * std

    yield "model.embed_tokens.weight", mat(V, H)
    if not getattr(cfg, "tie_word_embeddings", False):
        yield "lm_head.weight", mat(V, H)
    yield "model.norm.weight", torch.ones(H)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        yield p + "self_attn.q_proj.weight", mat(cfg.num_attention_heads * D, H)
        yield p + "self_attn.k_proj.weight", mat(cfg.num_key_value_heads * D, H)
        yield p + "self_attn.v_proj.weight", mat(cfg.num_key_value_heads * D, H)
        yield p + "self_attn.o_proj.weight", mat(H, cfg.num_attention_heads * D)
        yield p + "self_attn.q_norm.weight", torch.ones(D)
        yield p + "self_attn.k_norm.weight", torch.ones(D)
        yield p + "input_layernorm.weight", torch.ones(H)
        yield p + "post_attention_layernorm.weight", torch.ones(H)
        yield p + "mlp.gate_proj.weight", mat(I, H)
        yield p + "mlp.up_proj.weight", mat(I, H)
        yield p + "mlp.down_proj.weight", mat(H, I)


def run_cpp(path: str, cfg, prompt: List[int], new_tokens: int, threads: int = 0) -> Dict[str, object]:
    return host_ext().qwen3_cpu_generate(path, config_dict(cfg), prompt, new_tokens, threads)


def run_torch(path: str, cfg, prompt: List[int], new_tokens: int):
    """The same generation through the engine's model on CPU (PyTorch statements of the ops)."""
    import json as _json

    from ..configs import ServerConfig
    from ..executor import ModelRunner

    d = os.path.dirname(path)
    if not os.path.exists(os.path.join(d, "config.json")):
        cd = config_dict(cfg)
        cd.update(architectures=["Qwen3ForCausalLM"], model_type="qwen3", max_position_embeddings=40960, attention_bias=False)
        with open(os.path.join(d, "config.json"), "w") as f:
            _json.dump(cd, f)
    mr = ModelRunner(ServerConfig(model_path=d, dtype="float32", max_running_requests=1,
                                  max_total_tokens=len(prompt) + new_tokens + 8), device="cpu")
    mr.initialize()
    ids = torch.tensor(prompt)
    L = len(prompt)
    slots = mr.req_to_token_pool.alloc(1)
    sl = torch.tensor(slots)
    loc = mr.token_to_kv_pool_allocator.alloc(L)
    mr.req_to_token_pool.req_to_token[slots[0], :L] = loc.int()
    lens = torch.tensor([L])
    t0 = time.perf_counter()
    logits = mr.forward(mr.prepare_forward_batch_extend(ids, sl, lens, lens, torch.zeros_like(lens), loc)).next_token_logits
    prefill_s = time.perf_counter() - t0
    first = logits[0].clone()
    toks, cur = [], L
    t0 = time.perf_counter()
    for i in range(new_tokens):
        toks.append(int(logits.argmax(-1)))
        if i + 1 == new_tokens:
            break
        loc1 = mr.token_to_kv_pool_allocator.alloc(1)
        mr.req_to_token_pool.req_to_token[slots[0], cur] = loc1.int()
        cur += 1
        logits = mr.forward(mr.prepare_forward_batch_decode(torch.tensor([toks[-1]]), sl, torch.tensor([cur]), loc1)).next_token_logits
    return dict(tokens=toks, prefill_logits=first, last_logits=logits[0], prefill_seconds=prefill_s,
                decode_seconds=time.perf_counter() - t0)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="qwen3-0.6b")
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--new-tokens", type=int, default=32)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--check", action="store_true", help="also run the PyTorch fp32 model and compare logits")
    ap.add_argument("--workdir", default=None)
    a = ap.parse_args(argv)
    cfg = get_preset(a.preset)
    work = a.workdir or tempfile.mkdtemp(prefix="mllm_b200_oracle_")
    os.makedirs(work, exist_ok=True)
    path = os.path.join(work, "model.mllm")
    if not os.path.exists(path):
        write_mllm(path, seeded_weights(cfg, a.seed), model_name=a.preset)
    prompt = torch.randint(0, cfg.vocab_size, (a.prompt_len,), generator=torch.Generator().manual_seed(a.seed)).tolist()
    r = run_cpp(path, cfg, prompt, a.new_tokens, a.threads)
    out = dict(preset=a.preset, prompt_len=a.prompt_len, new_tokens=a.new_tokens, tokens=list(r["tokens"]),
               cpp_prefill_tok_s=a.prompt_len / r["prefill_seconds"], cpp_prefill_s=r["prefill_seconds"],
               cpp_decode_tok_s=(a.new_tokens - 1) / max(r["decode_seconds"], 1e-9), cpp_decode_s=r["decode_seconds"])
    if a.check:
        t = run_torch(path, cfg, prompt, a.new_tokens)
        out.update(torch_tokens_equal=t["tokens"] == list(r["tokens"]),
                   max_abs_logit_diff_prefill=float((t["prefill_logits"] - torch.from_numpy(r["prefill_logits"])).abs().max()),
                   max_abs_logit_diff_last=float((t["last_logits"] - torch.from_numpy(r["last_logits"])).abs().max()),
                   torch_prefill_s=t["prefill_seconds"], torch_decode_s=t["decode_seconds"])
    print(json.dumps(out))


if __name__ == "__main__":
    main()
