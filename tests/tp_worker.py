"""Child process of the tensor-parallel tests: one rank of a gloo (CPU) or NCCL (GPU) job.

Builds the tiny Qwen3 preset from a seeded full state dict (so every TP degree sees the same
weights), runs one prefill and two decode steps and, on rank 0, saves the logits."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def full_state_dict(cfg, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    H, D = cfg.hidden_size, cfg.head_dim
    hq, hkv, I, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size, cfg.vocab_size

    def r(*shape):
        return (torch.randn(*shape, generator=g) * 0.05).to(dtype)

    sd = {"model.embed_tokens.weight": r(V, H), "lm_head.weight": r(V, H),
          "model.norm.weight": torch.ones(H, dtype=dtype) + r(H)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        sd.update({
            p + "self_attn.q_proj.weight": r(hq * D, H), p + "self_attn.k_proj.weight": r(hkv * D, H),
            p + "self_attn.v_proj.weight": r(hkv * D, H), p + "self_attn.o_proj.weight": r(H, hq * D),
            p + "self_attn.q_norm.weight": torch.ones(D, dtype=dtype) + r(D),
            p + "self_attn.k_norm.weight": torch.ones(D, dtype=dtype) + r(D),
            p + "input_layernorm.weight": torch.ones(H, dtype=dtype) + r(H),
            p + "post_attention_layernorm.weight": torch.ones(H, dtype=dtype) + r(H),
            p + "mlp.gate_proj.weight": r(I, H), p + "mlp.up_proj.weight": r(I, H), p + "mlp.down_proj.weight": r(H, I),
        })
    E = getattr(cfg, "num_experts", 0)
    if E:
        Im = cfg.moe_intermediate_size
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}.mlp."
            for k in ("gate_proj.weight", "up_proj.weight", "down_proj.weight"):
                sd.pop(p + k, None)
            sd[p + "gate.weight"] = r(E, H) * 10
            for e in range(E):
                sd[p + f"experts.{e}.gate_proj.weight"] = r(Im, H)
                sd[p + f"experts.{e}.up_proj.weight"] = r(Im, H)
                sd[p + f"experts.{e}.down_proj.weight"] = r(H, Im)
    return sd


def hybrid_state_dict(cfg, seed=0, dtype=torch.float32):
    """Full (unsharded) weights of a Qwen3.5-style hybrid model under their checkpoint names."""
    g = torch.Generator().manual_seed(seed)
    H, D, I, V = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    kd = cfg.linear_key_head_dim * cfg.linear_num_key_heads
    vd = cfg.linear_value_head_dim * cfg.linear_num_value_heads
    hv, K = cfg.linear_num_value_heads, cfg.linear_conv_kernel_dim

    def r(*shape, s=0.05):
        return (torch.randn(*shape, generator=g) * s).to(dtype)

    sd = {"model.embed_tokens.weight": r(V, H), "lm_head.weight": r(V, H), "model.norm.weight": r(H)}
    for i, kind in enumerate(cfg.layer_types):
        p = f"model.layers.{i}."
        sd.update({p + "input_layernorm.weight": r(H), p + "post_attention_layernorm.weight": r(H),
                   p + "mlp.gate_proj.weight": r(I, H), p + "mlp.up_proj.weight": r(I, H), p + "mlp.down_proj.weight": r(H, I)})
        if kind == "linear_attention":
            a = p + "linear_attn."
            sd.update({a + "in_proj_qkv.weight": r(2 * kd + vd, H), a + "in_proj_z.weight": r(vd, H),
                       a + "in_proj_b.weight": r(hv, H), a + "in_proj_a.weight": r(hv, H),
                       a + "conv1d.weight": r(2 * kd + vd, 1, K, s=0.3), a + "dt_bias": r(hv, s=0.5).float(),
                       a + "A_log": r(hv, s=0.5).float(), a + "norm.weight": torch.ones(cfg.linear_value_head_dim, dtype=dtype) + r(cfg.linear_value_head_dim),
                       a + "out_proj.weight": r(H, vd)})
        else:
            a = p + "self_attn."
            sd.update({a + "q_proj.weight": r(hq * D * 2, H), a + "k_proj.weight": r(hkv * D, H), a + "v_proj.weight": r(hkv * D, H),
                       a + "o_proj.weight": r(H, hq * D), a + "q_norm.weight": r(D), a + "k_norm.weight": r(D)})
    return sd


def run(out_path: str, device: str, dtype_name: str) -> None:
    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner
    from mllm_b200.models.presets import get_preset
    from mllm_b200.parallel import state as pstate

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    pstate.init_distributed(backend="gloo" if device == "cpu" else "nccl", timeout_s=120)
    pp = int(os.environ.get("TP_TEST_PP", "1"))
    if world > 1:
        pstate.initialize_model_parallel(tp_size=world // pp, pp_size=pp,
                                         ep_size=world if os.environ.get("TP_TEST_EP") == "1" else 1)
    dev = device if device == "cpu" else f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}"
    preset = os.environ.get("TP_TEST_PRESET", "qwen3-tiny")
    hybrid = preset.startswith("qwen3.5")
    if hybrid:   # enough heads of every kind for two ranks; TP_TEST_KV_HEADS=1 exercises KV-head replication
        cfg = get_preset(preset, num_attention_heads=4, num_key_value_heads=int(os.environ.get("TP_TEST_KV_HEADS", "2")),
                         linear_num_key_heads=2, linear_num_value_heads=4, tie_word_embeddings=False)
    else:
        heads = int(os.environ.get("TP_TEST_HEADS", "4"))
        cfg = get_preset(preset, num_attention_heads=heads, num_key_value_heads=2, tie_word_embeddings=False)
    L = int(os.environ.get("TP_TEST_PREFILL_LEN", "9"))
    sc = ServerConfig(model_path=f"preset:{preset}", dtype=dtype_name, max_running_requests=4,
                      max_total_tokens=max(1024, 4 * L), chunked_prefill_size=max(2048, 2 * L),
                      tp_size=world // pp, pp_size=pp, ep_size=world if os.environ.get("TP_TEST_EP") == "1" else 1, disable_cuda_graph=os.environ.get("TP_TEST_GRAPH", "0") != "1",
                      comm_backend=os.environ.get("TP_TEST_COMM", "fused"))
    mr = ModelRunner(sc, hf_config=cfg, device=dev)
    mr.initialize()
    dtype = mr.dtype
    sd = (hybrid_state_dict if hybrid else full_state_dict)(cfg, dtype=dtype)
    files = os.environ.get("TP_TEST_FROM_FILES")
    if files:   # through the checkpoint reader (slice handles under tensor parallelism) instead of a dict
        from safetensors.torch import save_file

        from mllm_b200.io.lazy_tensor import LazyTensor

        if rank == 0:
            os.makedirs(files, exist_ok=True)
            save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(files, "model.safetensors"))
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        mr.model.load_weights(mr._iter_weights(files))
        with open(os.path.join(files, f"bytes_read_rank{rank}_of{world}.txt"), "w") as fh:
            fh.write(f"{LazyTensor.bytes_read} {sum(v.numel() * v.element_size() for v in sd.values())}")
    else:
        mr.model.load_weights(sd.items())
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
        if hasattr(m, "swiglu_block") and hasattr(m, "w13"):
            m.swiglu_block = 0
    if hasattr(mr.model, "post_load"):
        mr.model.post_load()
    if mr.cuda_graph_runner is not None:  # graphs hold the addresses of the weights they were captured with
        mr.cuda_graph_runner = None
        mr.init_cuda_graphs()

    torch.manual_seed(3)
    B = 2
    ids = torch.randint(0, cfg.vocab_size, (B, L))
    slots = mr.req_to_token_pool.alloc(B)
    loc = mr.token_to_kv_pool_allocator.alloc(B * L)
    sl = torch.tensor(slots, device=dev)
    mr.req_to_token_pool.req_to_token[sl.long(), :L] = loc.view(B, L).int()
    lens = torch.full((B,), L, device=dev)
    fb = mr.prepare_forward_batch_extend(ids.reshape(-1).to(dev), sl, lens, lens, torch.zeros_like(lens), loc,
                                         extend_seq_lens_cpu=[L] * B, extend_prefix_lens_cpu=[0] * B)
    out = mr.forward(fb)
    outs = [out.next_token_logits.float().cpu()]
    # The decode inputs are fixed ids, not the sampled ones: with random weights the two best logits of a row
    # can lie closer than the 16-bit rounding differences between two layouts, and one flipped token would
    # make every later step incomparable.  The sampler still runs (under pipeline parallelism the ids come
    # from the last stage).
    forced = torch.randint(0, cfg.vocab_size, (2, B))
    mr.sample(out)
    cur = L
    for step in range(2):
        nxt = forced[step].to(dev)
        loc1 = mr.token_to_kv_pool_allocator.alloc(B)
        mr.req_to_token_pool.req_to_token[sl.long(), cur] = loc1.int()
        cur += 1
        fb = mr.prepare_forward_batch_decode(nxt, sl, torch.full((B,), cur, device=dev), loc1, max_seq_len=cur)
        out = mr.forward(fb)
        outs.append(out.next_token_logits.float().cpu())
        mr.sample(out)
    if world > 1 and pp == 1 and hasattr(mr.model, "pick_greedy"):
        # greedy decoding without gathering logits: per-rank best candidate + one tiny all-gather must agree with
        # the argmax over the full vocabulary (columns that pad the vocabulary must never win)
        full = out.next_token_logits.float()
        V = full.shape[-1]
        per = -(-(V + 3) // world)                      # pretend the vocabulary needed padding
        padded = torch.full((full.shape[0], per * world), 1e4, device=full.device)
        padded[:, :V] = full
        saved_v = mr.model.config.vocab_size
        mr.model.config.vocab_size = V
        vals, ids_l = mr.model.local_greedy(padded[:, rank * per:(rank + 1) * per])
        picked = mr.model.pick_greedy(vals, ids_l)
        mr.model.config.vocab_size = saved_v
        assert torch.equal(picked.cpu(), full.argmax(-1).cpu()), (picked, full.argmax(-1))
    if device != "cpu":
        from mllm_b200 import ops

        ops.check_status()
    from mllm_b200.parallel.symm import get_tp_comm as _comm

    if _comm() is not None and getattr(_comm(), "heap", None) is not None:
        if device != "cpu":
            torch.cuda.synchronize()
        assert _comm().heap.check_guards() == [], "a kernel wrote outside a symmetric buffer"
    if os.environ.get("TP_TEST_EXPECT_EP_EXCHANGE") == "1":
        from mllm_b200.parallel.symm import get_ep_comm

        assert get_ep_comm() is not None and get_ep_comm().epoch > 0, "the expert-parallel exchange was not used"
        assert get_ep_comm().heap.check_guards() == [], "a kernel wrote outside an exchange buffer"
    if os.environ.get("TP_TEST_EXPECT_FUSED_PREFILL") == "1":
        from mllm_b200.parallel.symm import get_tp_comm

        assert get_tp_comm() is not None and get_tp_comm().epoch > 0, "fused prefill path was not taken"
    if rank == (world - 1 if pp > 1 else 0):      # under pipeline parallelism the last stage holds the logits
        torch.save(torch.stack(outs), out_path)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    run(sys.argv[1], sys.argv[2], sys.argv[3])
