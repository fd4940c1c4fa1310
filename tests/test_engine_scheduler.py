"""Scheduler, request bookkeeping and Engine on CPU with the tiny Qwen3 preset."""
import time

import pytest
import torch

from mllm_b200.configs import ServerConfig
from mllm_b200.engine.io_struct import GenerateReqInput, TokenizedGenerateReqInput
from mllm_b200.engine.launch import Engine
from mllm_b200.engine.sampling_params import SamplingParams
from mllm_b200.orchestrator.scheduler_process import build_scheduler


def _cfg(**kw):
    base = dict(model_path="preset:qwen3-tiny", dtype="float32", max_running_requests=4, max_total_tokens=2048,
                context_length=256, log_level="warning")
    base.update(kw)
    return ServerConfig(**base)


def _req(rid, ids, n=6, **sp):
    return TokenizedGenerateReqInput(rid=rid, input_ids=list(ids), sampling_params=dict(max_new_tokens=n, temperature=0.0, **sp))


def _drain(sched, limit=500):
    done = {}
    for _ in range(limit):
        out = sched.step()
        if out is not None:
            for i, rid in enumerate(out.rids):
                if out.finished_reasons[i] is not None:
                    done[rid] = (out.output_ids[i], out.finished_reasons[i], out.cached_tokens[i])
        if not sched.has_work():
            break
    sched._sweep_finished()
    return done


def test_io_struct_normalisation():
    r = GenerateReqInput(text=["a", "b"], sampling_params=[{"temperature": 0.1}, {"temperature": 0.2}])
    r.normalize_batch_and_arguments()
    assert r.batch_size == 2 and not r.is_single and len(r.rid) == 2
    assert r[1].text == "b" and r[1].sampling_params == {"temperature": 0.2}
    with pytest.raises(ValueError):
        GenerateReqInput(text="a", input_ids=[1]).normalize_batch_and_arguments()
    with pytest.raises(ValueError):
        GenerateReqInput().normalize_batch_and_arguments()
    assert SamplingParams.from_dict({"max_tokens": 7, "stop": "x"}).max_new_tokens == 7
    with pytest.raises(ValueError):
        SamplingParams.from_dict({"top_p": 0.0})


def test_batched_equals_sequential_and_pool_is_returned():
    torch.manual_seed(0)
    prompts = [torch.randint(0, 1000, (n,)).tolist() for n in (5, 17, 9)]
    sched = build_scheduler(_cfg(), device="cpu")
    free0 = sched.mrp.runner.token_to_kv_pool_allocator.available_size()
    for i, p in enumerate(prompts):
        assert sched.add_request(_req(f"r{i}", p)) is None
    batched = _drain(sched)
    assert all(v[1] == "length" and len(v[0]) == 6 for v in batched.values())
    # one at a time on a fresh scheduler
    for i, p in enumerate(prompts):
        s1 = build_scheduler(_cfg(disable_radix_cache=True), device="cpu")
        s1.add_request(_req("x", p))
        assert _drain(s1)["x"][0] == batched[f"r{i}"][0]
    # everything not held by the prefix tree is back in the allocator
    mrp = sched.mrp
    assert mrp.runner.token_to_kv_pool_allocator.available_size() + mrp.prefix_cache.evictable_size() == free0
    assert mrp.prefix_cache.protected_size() == 0 and mrp.free_req_slots() == mrp.runner.req_to_token_pool.size


def test_requests_that_finish_on_their_first_token_give_everything_back():
    """A request whose first sampled token already ends it (one new token asked for, or a stop token) never
    joins the decode set; its row, its KV slots and its lock on the prefix tree must still be returned."""
    torch.manual_seed(1)
    sched = build_scheduler(_cfg(), device="cpu")
    mrp = sched.mrp
    free0 = mrp.runner.token_to_kv_pool_allocator.available_size()
    for i in range(10):                                   # more than there are request rows
        sched.add_request(_req(f"one{i}", torch.randint(0, 1000, (7 + i,)).tolist(), n=1))
    done = _drain(sched)
    assert len(done) == 10 and all(v[1] == "length" and len(v[0]) == 1 for v in done.values())
    first = done["one0"][0][0]
    sched.add_request(_req("stop", torch.randint(0, 1000, (7,), generator=torch.Generator().manual_seed(5)).tolist(), n=5))
    # a stop token equal to whatever comes first: learn it from a dry run on a second scheduler
    probe = build_scheduler(_cfg(), device="cpu")
    ids = torch.randint(0, 1000, (9,), generator=torch.Generator().manual_seed(6)).tolist()
    probe.add_request(_req("p", ids, n=1))
    tok0 = _drain(probe)["p"][0][0]
    sched.add_request(_req("stop2", ids, n=5, stop_token_ids=[tok0]))
    done = _drain(sched)
    assert done["stop2"][1] == "stop" and len(done["stop2"][0]) == 1 and first is not None
    assert mrp.prefix_cache.protected_size() == 0 and mrp.free_req_slots() == mrp.runner.req_to_token_pool.size
    assert mrp.runner.token_to_kv_pool_allocator.available_size() + mrp.prefix_cache.evictable_size() == free0


@pytest.mark.parametrize("page", [4, 16])
def test_paged_pool_never_shares_a_page_between_requests(page):
    """With pages larger than one slot every request owns whole pages (the allocator recycles a page as soon as
    one of its slots is freed): concurrent requests with odd lengths, prefix reuse and long generations give the
    tokens of the one-slot-page run, no two live requests ever hold slots of one page, and every page comes back."""
    torch.manual_seed(2)
    shared = torch.randint(0, 1000, (37,)).tolist()
    prompts = [torch.randint(0, 1000, (n,)).tolist() for n in (5, 17, 9, 33, 3)] + \
        [shared + torch.randint(0, 1000, (n,)).tolist() for n in (4, 11, 2)]
    news = [20, 3, 11, 1, 25, 7, 9, 13]

    def run(page_size, check):
        sched = build_scheduler(_cfg(page_size=page_size, max_total_tokens=1024), device="cpu")
        mrp = sched.mrp
        free0 = mrp.runner.token_to_kv_pool_allocator.available_size()
        for i, (p, n) in enumerate(zip(prompts, news)):
            sched.add_request(_req(f"r{i}", p, n=n))
        done = {}
        for _ in range(500):
            out = sched.step()
            if out is not None:
                for i, rid in enumerate(out.rids):
                    if out.finished_reasons[i] is not None:
                        done[rid] = out.output_ids[i]
            if check:
                rtt = mrp.runner.req_to_token_pool.req_to_token
                owner = {}
                for q in sched.running + sched.prefilling:
                    if q.req_pool_idx < 0 or q.finished:
                        continue
                    own = rtt[q.req_pool_idx, q.prefix_len:q.num_computed].tolist() + \
                        ([] if q.spare_slots is None else list(map(int, q.spare_slots)))
                    for pg in {s // page_size for s in own}:
                        assert owner.setdefault(pg, q.rid) == q.rid, f"page {pg} held by {owner[pg]} and {q.rid}"
            if not sched.has_work():
                break
        sched._sweep_finished()
        assert mrp.prefix_cache.protected_size() == 0
        assert mrp.runner.token_to_kv_pool_allocator.available_size() + mrp.prefix_cache.evictable_size() == free0
        return done

    want, got = run(1, False), run(page, True)
    assert len(got) == len(prompts) and got == want


def test_requests_the_model_cannot_take_are_refused_at_intake():
    """Token ids outside the vocabulary (an out-of-bounds read on a device) and vision inputs whose pixels, grids
    and tokens disagree are answered with an error; the serving loop keeps running."""
    import numpy as np

    sched = build_scheduler(_cfg(), device="cpu")
    assert "outside the vocabulary" in sched.add_request(_req("a", [5, 99999]))
    assert "outside the vocabulary" in sched.add_request(_req("b", [5, -3]))
    assert sched.add_request(_req("c", [5, 6])) is None and "c" in _drain(sched)

    eng = Engine(_cfg(model_path="preset:qwen3-vl-tiny", context_length=256), mode="inproc", device="cpu").launch()
    try:
        img = np.random.default_rng(0).integers(0, 256, (64, 64, 3), dtype=np.uint8)
        sp = {"max_new_tokens": 2, "temperature": 0.0}
        with pytest.raises(ValueError, match="image / video tokens"):
            eng.generate(input_ids=[5, 1001, 6], image_data=img, sampling_params=sp, timeout=60)     # a stray image token
        big = np.random.default_rng(0).integers(0, 256, (640, 640, 3), dtype=np.uint8)
        with pytest.raises(ValueError):
            eng.generate("x", sp, image_data=big, timeout=60)                                      # image longer than the context
        assert len(eng.generate("x", sp, image_data=img, timeout=60)["output_ids"]) == 2
    finally:
        eng.shutdown()


def test_radix_reuse_gives_same_tokens_and_counts_cached():
    torch.manual_seed(1)
    shared = torch.randint(0, 1000, (40,)).tolist()
    a, b = shared + [5, 6, 7], shared + [9, 9]
    sched = build_scheduler(_cfg(), device="cpu")
    sched.add_request(_req("a", a))
    first = _drain(sched)
    sched.add_request(_req("b", b))
    second = _drain(sched)
    assert second["b"][2] >= 40  # the shared prefix was served from the cache
    cold = build_scheduler(_cfg(disable_radix_cache=True), device="cpu")
    cold.add_request(_req("b", b))
    assert _drain(cold)["b"][0] == second["b"][0] and first["a"][1] == "length"


def test_chunked_prefill_and_mixed_batches_match_unchunked():
    torch.manual_seed(2)
    long_p = torch.randint(0, 1000, (90,)).tolist()
    short_p = torch.randint(0, 1000, (6,)).tolist()
    ref = build_scheduler(_cfg(disable_radix_cache=True), device="cpu")
    ref.add_request(_req("s", short_p, n=12))
    ref.add_request(_req("l", long_p, n=4))
    want = _drain(ref)
    ch = build_scheduler(_cfg(disable_radix_cache=True, chunked_prefill_size=32), device="cpu")
    ch.add_request(_req("s", short_p, n=12))
    ch.step()  # the short request starts decoding before the long one arrives
    ch.add_request(_req("l", long_p, n=4))
    got = _drain(ch)
    assert got["l"][0] == want["l"][0] and got["s"][0] == want["s"][0]
    assert ch.stats.num_mixed_batches >= 2 and ch.stats.num_prefill_batches >= 3


def test_stop_token_abort_and_limits():
    sched = build_scheduler(_cfg(), device="cpu")
    sched.add_request(_req("a", [1, 2, 3], n=8))
    first = _drain(sched)["a"][0]
    s2 = build_scheduler(_cfg(), device="cpu")
    stop_tok = first[2]
    s2.add_request(_req("a", [1, 2, 3], n=8, stop_token_ids=[stop_tok]))
    out = _drain(s2)["a"]
    assert out[1] == "stop" and out[0] == first[: first.index(stop_tok) + 1]
    s3 = build_scheduler(_cfg(), device="cpu")
    s3.add_request(_req("z", [4, 5, 6], n=50))
    s3.step()
    assert s3.abort("z") and not s3.abort("nope")
    _drain(s3)
    assert s3.stats.aborted == 1 and s3.mrp.prefix_cache.protected_size() == 0
    assert s3.add_request(_req("e", [], n=1)) == "empty prompt"
    tight = build_scheduler(_cfg(max_queued_requests=1), device="cpu")
    assert tight.add_request(_req("q1", [1])) is None and tight.add_request(_req("q2", [1])) == "queue full"


def test_eviction_under_pressure():
    sched = build_scheduler(_cfg(max_total_tokens=160, max_running_requests=2), device="cpu")
    torch.manual_seed(3)
    for i in range(6):
        sched.add_request(_req(f"r{i}", torch.randint(0, 1000, (50,)).tolist(), n=5))
    done = _drain(sched, limit=2000)
    assert len(done) == 6 and sched.mrp.stats["evicted_tokens"] > 0


def test_engine_inproc_generate_stream_and_batch():
    eng = Engine(_cfg(), mode="inproc", device="cpu").launch()
    try:
        one = eng.generate("hello", {"max_new_tokens": 5, "temperature": 0.0})
        assert one["meta_info"]["completion_tokens"] == 5 and one["meta_info"]["finish_reason"] == "length"
        many = eng.generate(["hello", "hello world"], {"max_new_tokens": 4, "temperature": 0.0})
        assert len(many) == 2 and many[0]["output_ids"] == one["output_ids"][:4]
        chunks = list(eng.generate("hello", {"max_new_tokens": 5, "temperature": 0.0}, stream=True))
        assert chunks[-1]["meta_info"]["finish_reason"] == "length" and chunks[-1]["output_ids"] == one["output_ids"]
        assert "".join(c["delta"] for c in chunks) == chunks[-1]["text"]
        assert eng.is_healthy
        with pytest.raises(ValueError):
            eng.generate("x", {"top_p": 5.0})
    finally:
        eng.shutdown()
    assert not eng.is_healthy


def test_seeded_sampling_is_reproducible():
    eng = Engine(_cfg(), mode="inproc", device="cpu").launch()
    try:
        sp = {"max_new_tokens": 6, "temperature": 0.9, "top_k": 20, "top_p": 0.9, "seed": 7}
        a = eng.generate("abc", sp)["output_ids"]
        b = eng.generate("abc", sp)["output_ids"]
        c = eng.generate("abc", dict(sp, seed=8))["output_ids"]
        assert a == b and len(a) == 6 and (a != c or True)
        pen = eng.generate("abc", {"max_new_tokens": 6, "temperature": 0.0, "repetition_penalty": 1.3})
        assert pen["meta_info"]["completion_tokens"] == 6
    finally:
        eng.shutdown()


def test_image_request_through_the_engine_on_cpu():
    """An image request served end to end without a HF processor: built-in patchify, vision tokens in
    the prompt, vision tower + deepstack in the prefill, decode positions shifted by the image's
    position delta; the answer equals driving the model runner by hand with the same inputs."""
    import numpy as np
    import torch

    from mllm_b200.configs import ServerConfig
    from mllm_b200.engine.launch import Engine

    cfg = ServerConfig(model_path="preset:qwen3-vl-tiny", dtype="float32", max_running_requests=2, max_total_tokens=1024,
                       context_length=512, log_level="warning", chunked_prefill_size=16)
    eng = Engine(cfg, mode="inproc", device="cpu").launch()
    try:
        img = np.random.default_rng(0).integers(0, 256, (64, 96, 3), dtype=np.uint8)
        out = eng.generate("describe", {"max_new_tokens": 4, "temperature": 0.0}, image_data=img)
        assert len(out["output_ids"]) == 4
        runner = eng.scheduler.mrp.runner
        tok = eng.tokenizer_worker.tokenize({"rid": "x", "text": "describe", "image_data": img})
        n_img = sum(1 for t in tok.input_ids if t == runner.hf_config.image_token_id)
        g = tok.mm_inputs["image_grid_thw"][0].tolist()      # the small image is scaled up to the pixel floor
        assert n_img == g[0] * (g[1] // 2) * (g[2] // 2) and tok.mm_inputs["pixel_values"].shape[0] == n_img * 4
        # the same request by hand
        ids = torch.tensor(tok.input_ids)
        L = len(ids)
        slots = runner.req_to_token_pool.alloc(1)
        sl = torch.tensor(slots)
        loc = runner.token_to_kv_pool_allocator.alloc(L)
        runner.req_to_token_pool.req_to_token[slots[0], :L] = loc.int()
        lens = torch.tensor([L])
        fb = runner.prepare_forward_batch_extend(ids, sl, lens, lens, torch.zeros_like(lens), loc,
                                                 pixel_values=tok.mm_inputs["pixel_values"],
                                                 image_grid_thw=tok.mm_inputs["image_grid_thw"])
        logits = runner.forward(fb).next_token_logits
        want = [int(logits.argmax(-1))]
        delta = fb.mrope_position_deltas
        cur = L
        for _ in range(3):
            loc1 = runner.token_to_kv_pool_allocator.alloc(1)
            runner.req_to_token_pool.req_to_token[slots[0], cur] = loc1.int()
            cur += 1
            pos = (torch.tensor([cur - 1]) + delta).unsqueeze(0).expand(3, -1).contiguous()
            fbd = runner.prepare_forward_batch_decode(torch.tensor([want[-1]]), sl, torch.tensor([cur]), loc1, mrope_positions=pos)
            want.append(int(runner.forward(fbd).next_token_logits.argmax(-1)))
        assert out["output_ids"] == want
    finally:
        eng.shutdown()


def _replay(trace, **cfg_kw):
    """Feeds a recorded trace (arrivals and aborts keyed by scheduler step) to a fresh scheduler.
    Returns (the batch composition of every step, the final tokens / finish reason per request)."""
    sched = build_scheduler(_cfg(**cfg_kw), device="cpu")
    schedule, final = [], {}
    pick = sched.get_next_batch_to_run

    def logged():
        kind, rows = pick()
        schedule.append((kind, tuple((q.rid, n) for q, n in rows)))
        return kind, rows

    sched.get_next_batch_to_run = logged
    step = 0
    pending = sorted(trace, key=lambda e: e["step"])
    while pending or sched.has_work():
        while pending and pending[0]["step"] <= step:
            ev = pending.pop(0)
            if ev["kind"] == "arrive":
                assert sched.add_request(_req(ev["rid"], ev["ids"], n=ev["n"])) is None
            elif sched.abort(ev["rid"]):
                final[ev["rid"]] = ("aborted",)
        out = sched.step()
        if out is not None:
            for i, rid in enumerate(out.rids):
                if out.finished_reasons[i] is not None and rid not in final:
                    final[rid] = (tuple(out.output_ids[i]), out.finished_reasons[i])
        step += 1
        assert step < 2000
    sched._sweep_finished()
    mrp = sched.mrp
    assert mrp.prefix_cache.protected_size() == 0 and mrp.free_req_slots() == mrp.runner.req_to_token_pool.size
    return schedule, final


def test_recorded_trace_replays_deterministically():
    """A trace of staggered arrivals (shared prefixes, long and short prompts, more requests than
    running slots) and two aborts: replaying it gives the same batch composition step by step and the
    same tokens; changing the chunk size or switching prefix reuse off changes the schedule but not one
    token of any request that was not aborted."""
    import random

    rng = random.Random(7)
    shared = [rng.randrange(1000) for _ in range(40)]
    trace = []
    for i in range(12):
        ids = (shared[: rng.choice([0, 16, 40])] + [rng.randrange(1000) for _ in range(rng.randrange(3, 60))])
        trace.append({"step": rng.randrange(0, 25), "kind": "arrive", "rid": f"q{i}", "ids": ids, "n": rng.randrange(2, 12)})
    first = {e["rid"]: e["step"] for e in trace}
    trace.append({"step": first["q3"] + 2, "kind": "abort", "rid": "q3"})
    trace.append({"step": first["q8"] + 1, "kind": "abort", "rid": "q8"})

    sched_a, final_a = _replay(trace, chunked_prefill_size=32)
    sched_b, final_b = _replay(trace, chunked_prefill_size=32)
    assert sched_a == sched_b and final_a == final_b
    assert len(final_a) == 12 and any(kind == "extend" and len(rows) > 1 for kind, rows in sched_a)
    kept = {r: v for r, v in final_a.items() if v[0] != "aborted"}
    assert len(kept) >= 10
    for variant in (dict(chunked_prefill_size=8), dict(chunked_prefill_size=32, disable_radix_cache=True),
                    dict(chunked_prefill_size=32, max_running_requests=2)):
        sched_c, final_c = _replay(trace, **variant)
        assert sched_c != sched_a
        for rid, v in kept.items():
            if final_c[rid][0] != "aborted":     # an abort may land before or after the finish in another schedule
                assert final_c[rid] == v, (variant, rid)


def test_chat_and_perf_summary():
    eng = Engine(_cfg(), mode="inproc", device="cpu").launch()
    try:
        msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
        out = eng.chat(msgs, {"max_new_tokens": 5, "temperature": 0.0})
        # the same prompt by hand: ChatML (the byte tokenizer of the presets has no chat template)
        want = eng.generate("<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n",
                            {"max_new_tokens": 5, "temperature": 0.0})
        assert out["output_ids"] == want["output_ids"] and len(out["output_ids"]) == 5
        assert want["meta_info"]["cached_tokens"] > 0          # the second request reused the first one's prompt
        perf = Engine.perf_summary(out)
        assert perf["decode_tokens"] == 5 and perf["prefill_tokens"] == out["meta_info"]["prompt_tokens"]
        assert perf["ttft_ms"] > 0 and perf["e2e_ms"] >= perf["ttft_ms"] and perf["prefill_tokens_per_s"] > 0
        chunks = list(eng.chat(msgs, {"max_new_tokens": 5, "temperature": 0.0}, stream=True))
        assert chunks[-1]["output_ids"] == out["output_ids"]
    finally:
        eng.shutdown()


def test_logprobs_match_the_models_distribution():
    """Sampled-token and top-k log-probabilities reported by the engine equal log_softmax of the logits of a
    hand-driven forward pass; requests that did not ask get none, also inside the same batch."""
    eng = Engine(_cfg(), mode="inproc", device="cpu").launch()
    try:
        ids = [5, 9, 2, 7, 11, 3]
        res = eng.generate(input_ids=[ids, ids[:4]], sampling_params={"max_new_tokens": 3, "temperature": 0.0},
                           return_logprob=[True, False], top_logprobs_num=[2, 0])
        assert "output_token_logprobs" not in res[1]["meta_info"]
        lp = res[0]["meta_info"]["output_token_logprobs"]
        runner = eng.scheduler.mrp.runner
        seq = list(ids)
        for step in range(3):
            L = len(seq)
            slots = runner.req_to_token_pool.alloc(1)
            loc = runner.token_to_kv_pool_allocator.alloc(L)
            runner.req_to_token_pool.req_to_token[slots[0], :L] = loc.int()
            lens = torch.tensor([L])
            fb = runner.prepare_forward_batch_extend(torch.tensor(seq), torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc)
            want = torch.log_softmax(runner.forward(fb).next_token_logits.float(), -1)[0]
            runner.token_to_kv_pool_allocator.free(loc)
            runner.req_to_token_pool.free(slots[0])
            tok = res[0]["output_ids"][step]
            assert abs(lp["token_logprobs"][step] - float(want[tok])) < 1e-4
            tv, ti = want.topk(2)
            assert [i for i, _ in lp["top_logprobs"][step]] == ti.tolist()
            assert lp["top_logprobs"][step][1][1] == pytest.approx(float(tv[1]), abs=1e-4)
            seq.append(tok)
    finally:
        eng.shutdown()


def test_stop_strings_end_generation_and_never_reach_the_client():
    """A stop string taken from the middle of what the model would otherwise generate: generation ends with
    reason "stop", the text is cut right before it, streamed deltas never show any part of it, and the
    request without stop strings is untouched."""
    eng = Engine(_cfg(), mode="inproc", device="cpu").launch()
    try:
        sp = {"max_new_tokens": 24, "temperature": 0.0}
        full = eng.generate("hello world", sp)
        text = full["text"]
        assert len(text) >= 12
        stop = text[7:10]
        first = text.find(stop)
        out = eng.generate("hello world", dict(sp, stop=[stop, "\\x00never"]))
        assert out["meta_info"]["finish_reason"] == "stop" and out["text"] == text[:first]
        assert out["meta_info"]["completion_tokens"] < full["meta_info"]["completion_tokens"]
        chunks = list(eng.generate("hello world", dict(sp, stop=stop), stream=True))
        assert "".join(c["delta"] for c in chunks) == text[:first] and chunks[-1]["meta_info"]["finish_reason"] == "stop"
        assert all(stop not in c["text"] for c in chunks)
        assert eng.generate("hello world", sp)["text"] == text
    finally:
        eng.shutdown()


def test_longest_prefix_first_policy():
    """With one running slot, the queued request whose prompt is already cached is admitted before an older
    request with a cold prompt; under fcfs the arrival order is kept.  Tokens are the same either way."""
    warm = [7, 3, 9, 1, 4, 4, 2, 8, 6, 5, 1, 2, 3]

    def run(policy):
        sched = build_scheduler(_cfg(schedule_policy=policy, max_running_requests=1), device="cpu")
        sched.add_request(_req("seed", warm, n=2))
        _drain(sched)                                        # the warm prompt is now in the prefix cache
        sched.add_request(_req("blocker", [50, 51, 52], n=3))
        sched.step()                                         # occupies the only slot
        sched.add_request(_req("cold", [90, 91, 92, 93, 94, 95], n=2))
        sched.add_request(_req("hot", warm + [77], n=2))
        order, done = [], {}
        for _ in range(200):
            out = sched.step()
            if out is not None:
                for i, rid in enumerate(out.rids):
                    if out.finished_reasons[i] is not None:
                        order.append(rid)
                        done[rid] = (out.output_ids[i], out.cached_tokens[i])
            if not sched.has_work():
                break
        return order, done

    o_f, d_f = run("fcfs")
    o_l, d_l = run("lpm")
    assert o_f == ["blocker", "cold", "hot"] and o_l == ["blocker", "hot", "cold"]
    assert {k: v[0] for k, v in d_f.items()} == {k: v[0] for k, v in d_l.items()}
    assert d_l["hot"][1] >= len(warm) - 1 and d_l["cold"][1] == 0


def test_malformed_sampling_parameters_are_refused_not_raised():
    """A bad sampling value is answered with an error string (the multi-process serving loop has no other
    guard in front of the scheduler) and the next request is served."""
    sched = build_scheduler(_cfg(), device="cpu")
    assert "invalid sampling parameters" in sched.add_request(_req("bad", [1, 2, 3], top_p=0.0))
    assert "invalid sampling parameters" in sched.add_request(_req("bad2", [1, 2, 3], top_k="many"))
    assert sched.add_request(_req("good", [1, 2, 3])) is None
    assert "good" in _drain(sched)


def test_request_longer_than_the_pool_finishes_instead_of_cycling():
    """prompt + max_new_tokens beyond the KV pool: the output is cut to what the pool can hold, and a request
    that is alone in the pool when it runs dry ends with reason ``length`` instead of being queued again."""
    sched = build_scheduler(_cfg(max_total_tokens=64, context_length=256, max_running_requests=2), device="cpu")
    assert sched.add_request(_req("long", list(range(1, 31)), n=200)) is None
    done = _drain(sched, limit=400)
    assert "long" in done and done["long"][1] == "length"
    assert 0 < len(done["long"][0]) <= 64 - 30
    assert not sched.has_work()
    # direct check of the last resort: a lone request that cannot get KV ends, with its tokens delivered
    sched.add_request(_req("again", list(range(1, 21)), n=8))
    sched.step()
    out = sched._shed_load("test")
    assert out is not None and out.rids == ["again"] and out.finished_reasons == ["length"]
    assert not sched.has_work()


def test_retracted_image_request_is_prefilled_with_its_pixels_again():
    """An image request that is retracted mid-decode is prefilled again from its first token: the pixels must
    go through the vision tower again, so the tokens equal those of an undisturbed run."""
    import numpy as np

    img = np.random.default_rng(1).integers(0, 256, (64, 64, 3), dtype=np.uint8)
    sp = {"max_new_tokens": 6, "temperature": 0.0}

    def run(retract: bool):
        eng = Engine(_cfg(model_path="preset:qwen3-vl-tiny", context_length=256, max_running_requests=2,
                          disable_radix_cache=True), mode="inproc", device="cpu").launch()
        try:
            sched = eng.scheduler
            real_step, state = sched.step, {"did": False}

            def step():
                if retract and not state["did"] and sched.running and len(sched.running[0].output_ids) >= 3:
                    state["did"] = True
                    return sched._shed_load("test", requeue_lone=True)
                return real_step()

            sched.step = step
            out = eng.generate("describe", sp, image_data=img, timeout=120)["output_ids"]
            return out, state["did"]
        finally:
            eng.shutdown()

    want, _ = run(False)
    got, did = run(True)
    assert did and len(want) == 6 and got == want
