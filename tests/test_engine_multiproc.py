"""The multi-process engine (tokenizer -> scheduler -> detokenizer over ZMQ) on CPU, including the
liveness path: a worker process that dies turns the engine unhealthy (host-side fault, no GPU)."""
import time

import pytest

from mllm_b200.configs import ServerConfig
from mllm_b200.engine.launch import Engine


def _cfg():
    return ServerConfig(model_path="preset:qwen3-tiny", dtype="float32", max_running_requests=4, max_total_tokens=1024,
                        context_length=128, log_level="warning")


def test_multiproc_generate_matches_inproc_and_detects_dead_worker():
    ref = Engine(_cfg(), mode="inproc", device="cpu").launch()
    want = ref.generate("hello", {"max_new_tokens": 5, "temperature": 0.0})["output_ids"]
    ref.shutdown()
    eng = Engine(_cfg(), mode="multiproc", device="cpu").launch()
    try:
        got = eng.generate("hello", {"max_new_tokens": 5, "temperature": 0.0}, timeout=120)
        assert got["output_ids"] == want and got["meta_info"]["finish_reason"] == "length"
        chunks = list(eng.generate("hello", {"max_new_tokens": 5, "temperature": 0.0}, stream=True))
        assert chunks[-1]["output_ids"] == want
        # host-side failure injection: kill the detokenizer process (the last one spawned)
        eng._procs[-1].terminate()
        eng._procs[-1].join(10)
        eng._health_loop.__func__  # the monitor thread polls every 5 s
        deadline = time.time() + 12
        while eng.is_healthy and time.time() < deadline:
            time.sleep(0.25)
        assert not eng.is_healthy
        with pytest.raises((RuntimeError, TimeoutError)):
            eng.generate("x", {"max_new_tokens": 2}, timeout=5)
    finally:
        eng.shutdown()


def test_two_rank_tensor_parallel_engine_on_cpu():
    """Two scheduler/model-runner ranks (gloo, CPU) run in lock step behind one tokenizer/detokenizer
    pair: requests complete, repeated prompts (prefix-cache hits on both ranks) reproduce their tokens,
    and killing the follower rank turns the engine unhealthy.  (Numerical agreement of tensor-parallel
    and single-rank models is covered by the tensor-parallel tests, which load one set of weights.)"""
    prompts = ["hello", "the quick brown fox", "a"]
    cfg = _cfg()
    cfg.tp_size = 2
    eng = Engine(cfg, mode="multiproc", device="cpu").launch()
    try:
        assert len(eng._procs) == 4      # tokenizer, two scheduler ranks, detokenizer
        first = [eng.generate(p, {"max_new_tokens": 6, "temperature": 0.0}, timeout=180) for p in prompts]
        assert all(len(r["output_ids"]) == 6 and r["meta_info"]["finish_reason"] == "length" for r in first)
        again = [eng.generate(p, {"max_new_tokens": 6, "temperature": 0.0}, timeout=180)["output_ids"] for p in prompts]
        assert again == [r["output_ids"] for r in first]
        eng._procs[2].terminate()        # the follower rank: its peers' next control broadcast fails
        eng._procs[2].join(10)
        deadline = time.time() + 15
        while eng.is_healthy and time.time() < deadline:
            time.sleep(0.25)
        assert not eng.is_healthy
    finally:
        eng.shutdown()


def test_two_data_parallel_replicas_on_cpu():
    """Two complete replicas behind the tokenizer's router: same seeded weights, so every prompt gets
    the tokens the single engine gives, whichever replica serves it; concurrent requests spread over
    both; an abort reaches the replica that holds the request."""
    import threading

    prompts = ["hello", "the quick brown fox", "a", "lorem ipsum dolor", "hello"]
    ref = Engine(_cfg(), mode="inproc", device="cpu").launch()
    want = [ref.generate(p, {"max_new_tokens": 5, "temperature": 0.0})["output_ids"] for p in prompts]
    ref.shutdown()
    cfg = _cfg()
    cfg.dp_size = 2
    with pytest.raises(ValueError):
        Engine(cfg, mode="inproc", device="cpu").launch()
    eng = Engine(cfg, mode="multiproc", device="cpu").launch()
    try:
        assert len(eng._procs) == 4      # tokenizer, two replicas, detokenizer
        got = [None] * len(prompts)

        def one(i):
            got[i] = eng.generate(prompts[i], {"max_new_tokens": 5, "temperature": 0.0}, timeout=180)["output_ids"]

        threads = [threading.Thread(target=one, args=(i,)) for i in range(len(prompts))]
        for t in threads:
            t.start()
        for t in threads:
            t.join(200)
        assert got == want
        chunks = eng.generate("abort me", {"max_new_tokens": 100, "temperature": 0.0}, stream=True)
        first = next(chunks)
        chunks.close()                   # closing the stream aborts the request on its replica
        assert first["output_ids"]
        assert eng.generate("a", {"max_new_tokens": 3, "temperature": 0.0}, timeout=120)["output_ids"] == want[2][:3]
        assert eng.is_healthy
    finally:
        eng.shutdown()


def test_replica_router_spreads_requests_and_follows_aborts():
    from mllm_b200.engine.io_struct import AbortReq, FlushCacheReq, TokenizedGenerateReqInput
    from mllm_b200.orchestrator.tokenizer_process import ReplicaRouter

    class Sink:
        def __init__(self):
            self.got = []

        def send_pyobj(self, m):
            self.got.append(m)

    sinks = [Sink(), Sink(), Sink()]
    router = ReplicaRouter(sinks)

    def req(rid, n):
        return TokenizedGenerateReqInput(rid=rid, input_text="", input_ids=[1] * n, mm_inputs=None, sampling_params={},
                                         stream=False, return_logprob=False, created_time=0.0)

    where = {f"r{i}": router.route(req(f"r{i}", n))[0] for i, n in enumerate([100, 10, 10, 10, 10, 10])}
    assert where["r0"] == 0 and where["r1"] == 1 and where["r2"] == 2
    assert where["r3"] != 0 and where["r4"] != 0     # the replica holding the long prompt is skipped
    tokens = [sum(len(m.input_ids) for m in s.got) for s in sinks]
    assert max(tokens) == 100 and min(tokens) >= 20
    assert router.route(AbortReq(rid="r1")) == [1]
    assert router.route(AbortReq(rid="unknown")) == [0, 1, 2]
    assert router.route(FlushCacheReq()) == [0, 1, 2]
    assert router.route(None) == [0, 1, 2] and all(s.got[-1] is None for s in sinks)


def test_image_request_takes_the_shared_memory_queue():
    """``enable_shared_queue``: the tokenizer hands an image request's tensors to the scheduler through
    the shared-memory queue (the socket carries only a notice); the answer equals the in-process engine's,
    text requests still use the socket, and no shared-memory segment is left behind."""
    import glob

    import numpy as np

    def cfg(shared):
        return ServerConfig(model_path="preset:qwen3-vl-tiny", dtype="float32", max_running_requests=2,
                            max_total_tokens=1024, context_length=512, log_level="warning", enable_shared_queue=shared)

    img = np.random.default_rng(0).integers(0, 256, (64, 96, 3), dtype=np.uint8)
    sp = {"max_new_tokens": 4, "temperature": 0.0}
    ref = Engine(cfg(False), mode="inproc", device="cpu").launch()
    want_img = ref.generate("describe", sp, image_data=img)["output_ids"]
    want_txt = ref.generate("hello there", sp)["output_ids"]
    ref.shutdown()
    eng = Engine(cfg(True), mode="multiproc", device="cpu").launch()
    try:
        assert eng._tensor_queues is not None and len(eng._tensor_queues) == 1
        assert eng.generate("describe", sp, image_data=img, timeout=180)["output_ids"] == want_img
        assert eng.generate("hello there", sp, timeout=120)["output_ids"] == want_txt
        assert eng.generate("describe", sp, image_data=img, timeout=180)["output_ids"] == want_img
    finally:
        eng.shutdown()
    assert not glob.glob("/dev/shm/mllm_b200_meta_*")


def test_router_sends_tensor_requests_through_the_shared_queue():
    from mllm_b200.engine.io_struct import SharedQueueNotice, TokenizedGenerateReqInput
    from mllm_b200.orchestrator.scheduler_process import _take_from_shared_queue
    from mllm_b200.orchestrator.tokenizer_process import ReplicaRouter

    class Sink:
        def __init__(self):
            self.got = []

        def send_pyobj(self, m):
            self.got.append(m)

    class FakeQueue:
        def __init__(self):
            self.items = []

        def put(self, rid, meta, mm):
            self.items.append((rid, meta, mm))

        def get(self, timeout=None):
            return self.items.pop(0)

    sink, q = Sink(), FakeQueue()
    router = ReplicaRouter([sink], [q])
    mk = lambda rid, mm: TokenizedGenerateReqInput(rid=rid, input_text="", input_ids=[1, 2, 3], mm_inputs=mm,
                                                   sampling_params={}, stream=False, return_logprob=False, created_time=0.0)
    router.route(mk("text", None))
    router.route(mk("img", {"pixel_values": [1.0, 2.0]}))
    assert isinstance(sink.got[0], TokenizedGenerateReqInput) and isinstance(sink.got[1], SharedQueueNotice)
    assert len(q.items) == 1 and q.items[0][1].mm_inputs is None      # the body on the queue, tensors beside it
    back = _take_from_shared_queue(q, sink.got[1])
    assert back.rid == "img" and back.mm_inputs == {"pixel_values": [1.0, 2.0]} and back.input_ids == [1, 2, 3]
    assert "error" in _take_from_shared_queue(None, sink.got[1])


def test_two_pipeline_stages_engine_on_cpu():
    """Two scheduler / model-runner ranks as pipeline stages behind one tokenizer / detokenizer pair:
    requests complete, batches of several requests work, repeated prompts reproduce their tokens, and a
    request for log-probabilities is refused with a clear message (the logits live on the last stage)."""
    cfg = _cfg()
    cfg.pp_size = 2
    eng = Engine(cfg, mode="multiproc", device="cpu").launch()
    try:
        assert len(eng._procs) == 4      # tokenizer, two stages, detokenizer
        sp = {"max_new_tokens": 6, "temperature": 0.0}
        first = eng.generate(["hello", "the quick brown fox", "a"], sp, timeout=180)
        assert all(len(r["output_ids"]) == 6 and r["meta_info"]["finish_reason"] == "length" for r in first)
        again = eng.generate(["hello", "the quick brown fox", "a"], sp, timeout=180)
        assert [r["output_ids"] for r in again] == [r["output_ids"] for r in first]
        with pytest.raises(ValueError, match="pipeline"):
            eng.generate("hello", sp, timeout=60, return_logprob=True)
        assert eng.is_healthy
    finally:
        eng.shutdown()
