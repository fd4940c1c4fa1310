"""OpenAI-compatible endpoints through FastAPI's test client over an in-process CPU engine."""
import json

import pytest

from mllm_b200.configs import GlobalConfig, ServerConfig
from mllm_b200.engine.launch import Engine
from mllm_b200.server.launch import create_app

fastapi_testclient = pytest.importorskip("fastapi.testclient")


@pytest.fixture(scope="module")
def client():
    GlobalConfig.reset()
    sc = ServerConfig(model_path="preset:qwen3-tiny", dtype="float32", max_running_requests=4, max_total_tokens=2048,
                      context_length=256, log_level="warning", api_key="secret", enable_metrics=True,
                      enable_debug_timing=True, reasoning_parser="qwen3", tool_call_parser="qwen25",
                      served_model_name="tiny")
    eng = Engine(sc, mode="inproc", device="cpu").launch()
    with fastapi_testclient.TestClient(create_app(eng)) as c:
        c.headers.update({"Authorization": "Bearer secret"})
        yield c
    eng.shutdown()


def _sse(resp):
    events = [l[6:] for l in resp.text.split("\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    return [json.loads(e) for e in events[:-1]]


def test_health_auth_models(client):
    assert client.get("/health", headers={"Authorization": ""}).status_code == 200
    assert client.get("/v1/models", headers={"Authorization": "Bearer wrong"}).status_code == 401
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    assert client.get("/v1/models/tiny").json()["id"] == "tiny"
    assert client.get("/v1/models/other").status_code == 404
    assert client.get("/model_info").json()["is_generation"] is True
    assert "api_key" not in client.get("/server_info").json()["server"]
    assert client.get("/health_generate").status_code == 200


def test_generate_and_completions(client):
    r = client.post("/generate", json={"text": "hello", "sampling_params": {"max_new_tokens": 4, "temperature": 0}})
    assert r.status_code == 200 and r.json()["meta_info"]["completion_tokens"] == 4
    r = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 5, "temperature": 0})
    body = r.json()
    assert body["object"] == "text_completion" and body["usage"]["completion_tokens"] == 5
    assert body["usage"]["total_tokens"] == body["usage"]["prompt_tokens"] + 5 and "debug_timing" in body
    assert client.post("/v1/completions", json={"prompt": "x", "n": 2, "stream": True}).status_code == 400
    assert client.post("/v1/completions", json={"prompt": "x", "top_p": 7}).status_code == 400
    s = _sse(client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 5, "temperature": 0, "stream": True,
                                                  "stream_options": {"include_usage": True}}))
    assert s[-1]["usage"]["completion_tokens"] == 5 and s[-2]["choices"][0]["finish_reason"] == "length"
    assert "".join(c["choices"][0]["text"] for c in s if c["choices"]) == body["choices"][0]["text"]


def test_chat_completions(client):
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": [{"type": "text", "text": "hi"}]}]
    r = client.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 6, "temperature": 0})
    body = r.json()
    assert body["object"] == "chat.completion" and body["choices"][0]["message"]["role"] == "assistant"
    assert body["usage"]["completion_tokens"] == 6 and "reasoning_content" in body["choices"][0]["message"]
    s = _sse(client.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 6, "temperature": 0, "stream": True}))
    assert s[0]["choices"][0]["delta"]["role"] == "assistant" and s[-1]["choices"][0]["finish_reason"] == "length"
    assert client.post("/v1/chat/completions", json={"messages": msgs, "logprobs": True, "stream": True}).status_code == 400


def test_abort_flush_metrics(client):
    assert client.post("/abort_request", json={"rid": "nope"}).json()["status"] == "ok"
    assert client.post("/flush_cache").status_code == 200
    text = client.get("/metrics").text
    assert "mllm_b200_requests_total" in text and "mllm_b200_ttft_seconds_bucket" in text and "mllm_b200_kv_usage_ratio" in text


def test_logprobs_in_all_three_endpoints(client):
    import math

    r = client.post("/generate", json={"text": "hello", "sampling_params": {"max_new_tokens": 4, "temperature": 0},
                                       "return_logprob": True, "top_logprobs_num": 3}).json()
    lp = r["meta_info"]["output_token_logprobs"]
    assert len(lp["token_logprobs"]) == 4 and len(lp["tokens"]) == 4 and all(len(t) == 3 for t in lp["top_logprobs"])
    for chosen, top in zip(lp["token_logprobs"], lp["top_logprobs"]):
        assert chosen <= 0 and abs(chosen - top[0][1]) < 1e-6        # greedy: the sampled token is the most likely one
        assert top[0][1] >= top[1][1] >= top[2][1]
    assert [t[0][0] for t in lp["top_logprobs"]] == r["output_ids"]

    body = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 4, "temperature": 0, "logprobs": 2}).json()
    clp = body["choices"][0]["logprobs"]
    assert clp["token_logprobs"] == pytest.approx(lp["token_logprobs"], abs=1e-5)
    assert len(clp["top_logprobs"]) == 4 and all(len(d) <= 2 for d in clp["top_logprobs"]) and clp["text_offset"][0] == 0
    assert "".join(clp["tokens"]) == body["choices"][0]["text"]
    plain = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 4, "temperature": 0}).json()
    assert plain["choices"][0]["logprobs"] is None and plain["choices"][0]["text"] == body["choices"][0]["text"]

    chat = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                                     "temperature": 0, "logprobs": True, "top_logprobs": 2}).json()
    content = chat["choices"][0]["logprobs"]["content"]
    assert len(content) == 3 and all(len(c["top_logprobs"]) == 2 and c["logprob"] <= 0 for c in content)
    assert all(bytes(c["bytes"]).decode("utf-8", "ignore") == c["token"] for c in content)
    assert math.isclose(content[0]["logprob"], content[0]["top_logprobs"][0]["logprob"], abs_tol=1e-6)
    assert client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "logprobs": True,
                                                     "stream": True}).status_code == 400
    assert client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                     "top_logprobs": 2}).status_code == 400


def test_n_samples_echo_and_stop(client):
    body = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 5, "temperature": 0.9, "n": 3, "seed": 11}).json()
    assert [c["index"] for c in body["choices"]] == [0, 1, 2] and body["usage"]["completion_tokens"] == 15
    again = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 5, "temperature": 0.9, "n": 3, "seed": 11}).json()
    assert [c["text"] for c in again["choices"]] == [c["text"] for c in body["choices"]]     # seeds are seed, seed+1, seed+2
    assert len({c["text"] for c in body["choices"]}) > 1
    echo = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 3, "temperature": 0, "echo": True}).json()
    plain = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 3, "temperature": 0}).json()
    assert echo["choices"][0]["text"] == "hello" + plain["choices"][0]["text"]
    assert client.post("/v1/completions", json={"prompt": "x", "n": 2, "stream": True}).status_code == 400
    assert client.post("/v1/completions", json={"prompt": "x", "n": 99}).status_code == 400
    chat = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                                                     "temperature": 0, "n": 2}).json()
    assert len(chat["choices"]) == 2 and chat["choices"][0]["message"]["content"] == chat["choices"][1]["message"]["content"]
    assert chat["usage"]["completion_tokens"] == 8
    # stop strings through the HTTP layer
    long = client.post("/v1/completions", json={"prompt": "hello world", "max_tokens": 24, "temperature": 0}).json()["choices"][0]["text"]
    stop = long[6:9]
    cut = client.post("/v1/completions", json={"prompt": "hello world", "max_tokens": 24, "temperature": 0, "stop": stop}).json()
    assert cut["choices"][0]["text"] == long[: long.find(stop)] and cut["choices"][0]["finish_reason"] == "stop"


def test_method_variants_of_generate_and_flush(client):
    r = client.put("/generate", json={"text": "hello", "sampling_params": {"max_new_tokens": 2, "temperature": 0}})
    assert r.status_code == 200 and r.json()["meta_info"]["completion_tokens"] == 2
    assert client.get("/flush_cache").status_code == client.post("/flush_cache").status_code == 200


def test_compat_fields_and_continuous_usage(client):
    msgs = [{"role": "user", "content": "hi"}]
    s = _sse(client.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 4, "temperature": 0, "stream": True,
                                                      "user": "u1", "stream_reasoning": False,
                                                      "stream_options": {"include_usage": True, "continuous_usage_stats": True}}))
    with_usage = [c for c in s if c.get("choices") and "usage" in c]
    assert with_usage and with_usage[-1]["usage"]["completion_tokens"] >= with_usage[0]["usage"]["completion_tokens"]
    assert s[-1]["usage"]["completion_tokens"] == 4
    r = client.post("/generate", json={"text": "hello", "sampling_params": {"max_new_tokens": 2, "temperature": 0},
                                       "logprob_start_len": -1, "lora_path": None, "session_params": None})
    assert r.status_code == 200
    assert client.post("/v1/completions", json={"prompt": "x", "max_tokens": 2, "user": "u"}).status_code == 200
