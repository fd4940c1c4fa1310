"""Messages that travel between the HTTP layer, tokenizer, scheduler and detokenizer
(same roles and field names as pymllm/engine/io_struct.py:30-205)."""

from __future__ import annotations

import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Union


def new_rid() -> str:
    return uuid.uuid4().hex


@dataclass
class BaseReq:
    rid: Optional[Union[str, List[str]]] = None


@dataclass
class GenerateReqInput(BaseReq):
    """A user request: one prompt or a batch of prompts, as text or as token ids."""

    text: Optional[Union[List[str], str]] = None
    input_ids: Optional[Union[List[List[int]], List[int]]] = None
    sampling_params: Optional[Union[List[Dict[str, Any]], Dict[str, Any]]] = None
    return_logprob: Optional[Union[List[bool], bool]] = None
    logprob_start_len: Optional[Union[List[int], int]] = None
    top_logprobs_num: Optional[Union[List[int], int]] = None
    stream: bool = False
    image_data: Optional[Any] = None
    video_data: Optional[Any] = None
    audio_data: Optional[Any] = None
    lora_path: Optional[Union[List[Optional[str]], str]] = None
    session_params: Optional[Union[List[Dict[str, Any]], Dict[str, Any]]] = None
    extra_options: Dict[str, Any] = field(default_factory=dict)
    is_single: bool = field(default=True, init=False)
    batch_size: int = field(default=1, init=False)

    def normalize_batch_and_arguments(self) -> None:
        if (self.text is None) == (self.input_ids is None):
            raise ValueError("Exactly one of `text` or `input_ids` must be provided.")
        if self.text is not None:
            if isinstance(self.text, str):
                self.is_single, self.batch_size = True, 1
            else:
                if not self.text:
                    raise ValueError("`text` cannot be an empty list.")
                self.is_single, self.batch_size = False, len(self.text)
        else:
            if len(self.input_ids) == 0:
                raise ValueError("`input_ids` cannot be empty.")
            if isinstance(self.input_ids[0], int):
                self.is_single, self.batch_size = True, 1
            else:
                self.is_single, self.batch_size = False, len(self.input_ids)
        if self.rid is None:
            self.rid = new_rid() if self.is_single else [new_rid() for _ in range(self.batch_size)]
        elif not self.is_single and isinstance(self.rid, str):
            self.rid = [f"{self.rid}_{i}" for i in range(self.batch_size)]

    @staticmethod
    def _pick(value: Any, i: int) -> Any:
        return value[i] if isinstance(value, list) else value

    def __getitem__(self, i: int) -> "GenerateReqInput":
        if not 0 <= i < self.batch_size:
            raise IndexError(f"index {i} out of range for batch size {self.batch_size}")
        if self.is_single:
            return self
        one = GenerateReqInput(
            rid=self._pick(self.rid, i), text=self._pick(self.text, i),
            input_ids=self.input_ids[i] if self.input_ids is not None else None,
            sampling_params=self._pick(self.sampling_params, i), return_logprob=self._pick(self.return_logprob, i),
            logprob_start_len=self._pick(self.logprob_start_len, i), top_logprobs_num=self._pick(self.top_logprobs_num, i),
            stream=self.stream, image_data=self._pick(self.image_data, i), video_data=self._pick(self.video_data, i),
            audio_data=self._pick(self.audio_data, i), lora_path=self._pick(self.lora_path, i),
            session_params=self._pick(self.session_params, i), extra_options=dict(self.extra_options),
        )
        one.is_single, one.batch_size = True, 1
        return one

    def to_request_dict(self) -> Dict[str, Any]:
        keys = ("rid", "text", "input_ids", "sampling_params", "return_logprob", "logprob_start_len",
                "top_logprobs_num", "stream", "image_data", "video_data", "audio_data", "lora_path", "session_params")
        out = {k: getattr(self, k) for k in keys if getattr(self, k) is not None}
        out.update(self.extra_options)
        return out


@dataclass
class TokenizedGenerateReqInput(BaseReq):
    input_text: str = ""
    input_ids: List[int] = field(default_factory=list)
    mm_inputs: Optional[Dict[str, Any]] = None
    sampling_params: Dict[str, Any] = field(default_factory=dict)
    stream: bool = False
    return_logprob: bool = False
    logprob_start_len: int = -1
    top_logprobs_num: int = 0
    lora_path: Optional[str] = None
    session_params: Optional[Dict[str, Any]] = None
    created_time: float = 0.0


@dataclass
class SharedQueueNotice:
    """Sent over the control socket in place of a request whose body went through the shared-memory
    queue (``--server.enable_shared_queue``): keeps the arrival order and wakes an idle scheduler."""
    rid: str = ""


@dataclass
class BatchTokenizedGenerateReqInput:
    reqs: List[TokenizedGenerateReqInput]

    def __len__(self) -> int:
        return len(self.reqs)

    def __getitem__(self, i: int) -> TokenizedGenerateReqInput:
        return self.reqs[i]

    def __iter__(self) -> Iterator[TokenizedGenerateReqInput]:
        return iter(self.reqs)


@dataclass
class AbortReq:
    rid: str


@dataclass
class FlushCacheReq:
    pass


@dataclass
class BatchTokenIDOutput:
    """Scheduler -> detokenizer: the state of every request that produced a token this step."""

    rids: List[str]
    finished_reasons: List[Optional[str]]
    output_ids: List[List[int]]           # all generated ids so far, per request
    skip_special_tokens: List[bool]
    prompt_tokens: List[int]
    completion_tokens: List[int]
    cached_tokens: List[int] = field(default_factory=list)
    timing: List[Optional[Dict[str, float]]] = field(default_factory=list)
    # per request: None, or {"token_logprobs": [lp per generated token], "top_logprobs": [[(id, lp), ...] per token]}
    logprobs: List[Optional[Dict[str, Any]]] = field(default_factory=list)
    stop_strs: List[Optional[List[str]]] = field(default_factory=list)   # the text is cut at the first of these


@dataclass
class BatchStrOutput:
    """Detokenizer -> front end."""

    rids: List[str]
    finished_reasons: List[Optional[str]]
    output_strs: List[str]                # full text so far
    deltas: List[str]                     # text added since the previous message
    output_ids: List[List[int]]
    prompt_tokens: List[int]
    completion_tokens: List[int]
    cached_tokens: List[int] = field(default_factory=list)
    timing: List[Optional[Dict[str, float]]] = field(default_factory=list)
    logprobs: List[Optional[Dict[str, Any]]] = field(default_factory=list)
