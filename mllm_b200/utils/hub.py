"""Model locations: a checkpoint directory, a built-in preset (``preset:<name>``) or a hub repository id.

The reference downloads a repository when ``model_path`` is not a directory (pymllm/engine/launch.py:647-658,
``Engine._maybe_download``).  Here the same rule is one function used by the engine and the command-line tools;
the download itself is ``huggingface_hub.snapshot_download`` (weights, config and tokenizer files only)."""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Optional, Union

logger = logging.getLogger(__name__)

# what a serving process reads: configs, tokenizer files, safetensors shards and their index
_ALLOW = ["*.json", "*.safetensors", "*.txt", "*.model", "*.tiktoken", "*.jinja", "*.mllm"]


def is_preset(path: Union[str, Path, None]) -> bool:
    return path is not None and str(path).startswith("preset:")


def resolve_model_path(path: Union[str, Path, None], download_dir: Optional[Union[str, Path]] = None) -> Optional[Path]:
    """``path`` itself when it is a preset, a directory or a file; otherwise ``path`` is taken as a hub repository
    id (``org/name``) and the local snapshot directory is returned (downloaded under ``download_dir/<name>`` when
    given, else into the hub cache).  Raises ``FileNotFoundError`` with the reason when neither works."""
    if path is None or is_preset(path):
        return None if path is None else Path(str(path))
    p = Path(str(path))
    if p.exists():
        return p
    repo_id = str(path)
    if repo_id.count("/") != 1 or repo_id.startswith((".", "/", "~")):
        raise FileNotFoundError(f"model path {repo_id!r} does not exist (and is not an 'org/name' repository id)")
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:  # pragma: no cover
        raise FileNotFoundError(f"model path {repo_id!r} does not exist and huggingface_hub is not installed") from e
    kwargs = {"allow_patterns": list(_ALLOW)}
    if download_dir is not None:
        kwargs["local_dir"] = str(Path(download_dir) / p.name)
    logger.info("downloading %s ...", repo_id)
    try:
        local = snapshot_download(repo_id=repo_id, **kwargs)
    except Exception as e:
        raise FileNotFoundError(f"model path {repo_id!r} is not a local directory and could not be downloaded: "
                                f"{type(e).__name__}: {e}") from e
    logger.info("downloaded %s to %s", repo_id, local)
    return Path(local)
