"""Model locations: directories and presets pass through, anything shaped like ``org/name`` is fetched as a hub
repository (the download call is replaced by a stand-in that writes a snapshot directory: there is no network)."""
import json

import pytest

from mllm_b200.configs import ServerConfig
from mllm_b200.engine.launch import Engine
from mllm_b200.executor import load_hf_config
from mllm_b200.models.presets import preset_to_config_json
from mllm_b200.utils import hub


def test_directories_and_presets_pass_through(tmp_path):
    assert str(hub.resolve_model_path("preset:qwen3-tiny")) == "preset:qwen3-tiny"
    assert hub.resolve_model_path(tmp_path) == tmp_path
    assert hub.resolve_model_path(None) is None
    with pytest.raises(FileNotFoundError, match="does not exist"):
        hub.resolve_model_path(tmp_path / "missing")
    with pytest.raises(FileNotFoundError, match="does not exist"):
        hub.resolve_model_path("just-a-name")


def test_repository_id_is_downloaded_once_and_the_engine_reads_the_snapshot(tmp_path, monkeypatch):
    import huggingface_hub

    calls = []

    def fake_download(repo_id, local_dir=None, allow_patterns=None, **kw):
        calls.append((repo_id, local_dir, tuple(allow_patterns or ())))
        out = tmp_path / "cache" / repo_id.replace("/", "--") if local_dir is None else type(tmp_path)(local_dir)
        out.mkdir(parents=True, exist_ok=True)
        (out / "config.json").write_text(json.dumps(preset_to_config_json("qwen3-tiny")))
        return str(out)

    monkeypatch.setattr(huggingface_hub, "snapshot_download", fake_download)
    eng = Engine(ServerConfig(model_path="someorg/tiny-model", download_dir=tmp_path / "dl"), device="cpu")
    sc = eng.server_config
    assert str(sc.model_path) == str(tmp_path / "dl" / "tiny-model") and str(sc.tokenizer_path) == str(sc.model_path)
    assert calls == [("someorg/tiny-model", str(tmp_path / "dl" / "tiny-model"), tuple(hub._ALLOW))]
    cfg = load_hf_config(sc.model_path)
    assert int(cfg.hidden_size) == 256 and int(cfg.vocab_size) == 1024
    # a separate tokenizer repository is resolved on its own; without download_dir the hub cache is used
    eng2 = Engine(ServerConfig(model_path="someorg/tiny-model", tokenizer_path="otherorg/tok"), device="cpu")
    assert str(eng2.server_config.tokenizer_path).endswith("otherorg--tok")
    assert [c[0] for c in calls[1:]] == ["someorg/tiny-model", "otherorg/tok"]


def test_a_failed_download_names_the_reason(monkeypatch):
    import huggingface_hub

    def boom(**kw):
        raise OSError("no route to host")

    monkeypatch.setattr(huggingface_hub, "snapshot_download", boom)
    with pytest.raises(FileNotFoundError, match="could not be downloaded: OSError: no route to host"):
        hub.resolve_model_path("someorg/tiny-model")


def test_eos_ids_and_default_output_length_follow_the_checkpoint(tmp_path):
    """Precedence of the end-of-sequence ids: config, text_config, generation_config.json; and the output-length
    limit a config declares becomes the default of requests that give none."""
    import types

    from mllm_b200.engine.launch import model_default_max_new_tokens
    from mllm_b200.orchestrator.scheduler_process import resolve_eos_token_ids

    ns = types.SimpleNamespace
    assert resolve_eos_token_ids(ns(eos_token_id=7)) == [7]
    assert resolve_eos_token_ids(ns(eos_token_id=[7, 9])) == [7, 9]
    assert resolve_eos_token_ids(ns(eos_token_id=None, text_config=ns(eos_token_id=11))) == [11]
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [151645, 151643], "temperature": 0.7}))
    assert resolve_eos_token_ids(ns(eos_token_id=None), tmp_path) == [151645, 151643]
    assert resolve_eos_token_ids(ns(eos_token_id=3), tmp_path) == [3]                 # the config wins
    assert resolve_eos_token_ids(ns(eos_token_id=None), "preset:qwen3-tiny") == []
    (tmp_path / "generation_config.json").write_text("{not json")
    assert resolve_eos_token_ids(ns(eos_token_id=None), tmp_path) == []
    assert model_default_max_new_tokens(ns(max_new_tokens=None, max_tokens=512)) == 512
    assert model_default_max_new_tokens(ns(text_config=ns(max_completion_tokens=64))) == 64
    assert model_default_max_new_tokens(ns(max_new_tokens=0)) is None
    # through the engine: a request without a length stops at the model's default
    from mllm_b200.models.presets import get_preset

    eng = Engine(ServerConfig(model_path="preset:qwen3-tiny", dtype="float32", max_running_requests=2, max_total_tokens=512,
                              log_level="warning"), hf_config=get_preset("qwen3-tiny", max_new_tokens=5), device="cpu").launch()
    try:
        out = eng.generate("hello", {"temperature": 0.0, "ignore_eos": True})
        assert len(out["output_ids"]) == 5
        assert len(eng.generate("hello", {"temperature": 0.0, "ignore_eos": True, "max_new_tokens": 2})["output_ids"]) == 2
    finally:
        eng.shutdown()
