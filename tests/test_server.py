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
    assert client.post("/v1/completions", json={"prompt": "x", "n": 2}).status_code == 400
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
    assert client.post("/v1/chat/completions", json={"messages": msgs, "logprobs": True}).status_code == 400


def test_abort_flush_metrics(client):
    assert client.post("/abort_request", json={"rid": "nope"}).json()["status"] == "ok"
    assert client.post("/flush_cache").status_code == 200
    text = client.get("/metrics").text
    assert "mllm_b200_requests_total" in text and "mllm_b200_ttft_seconds_bucket" in text and "mllm_b200_kv_usage_ratio" in text
