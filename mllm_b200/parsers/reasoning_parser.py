"""Split model output into reasoning (``<think> ... </think>``) and answer text.

Covers the model families of pymllm/parsers/reasoning_parser.py:30-212 — ``deepseek-r1`` and
``qwen3-thinking`` (the model starts inside a reasoning block even without an opening tag),
``qwen3``, ``glm45`` and ``kimi`` (reasoning only after an explicit opening tag) — for whole strings
and for streams, where a tag may arrive split over several chunks.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class _Family:
    open_tag: str
    close_tag: str
    starts_in_reasoning: bool


FAMILIES: Dict[str, _Family] = {
    "deepseek-r1": _Family("<think>", "</think>", True),
    "qwen3": _Family("<think>", "</think>", False),
    "qwen3-thinking": _Family("<think>", "</think>", True),
    "glm45": _Family("<think>", "</think>", False),
    "kimi": _Family("◁think▷", "◁/think▷", False),
}


def _held_back(text: str, tag: str) -> int:
    """Length of the longest suffix of ``text`` that is a proper prefix of ``tag``."""
    for n in range(min(len(tag) - 1, len(text)), 0, -1):
        if tag.startswith(text[-n:]):
            return n
    return 0


class ReasoningParser:
    def __init__(self, model_type: str, stream_reasoning: bool = True) -> None:
        if model_type not in FAMILIES:
            raise ValueError(f"unknown reasoning parser {model_type!r}; have {sorted(FAMILIES)}")
        self.family = FAMILIES[model_type]
        self.stream_reasoning = stream_reasoning
        self._in_reasoning = self.family.starts_in_reasoning
        self._seen_open = False
        self._done = False
        self._pending = ""
        self._reasoning_buf = ""
        self._strip_nl = False

    def parse_non_stream(self, text: str) -> Tuple[Optional[str], str]:
        """(reasoning or None, answer)."""
        f = self.family
        body = text
        had_open = False
        if f.open_tag in body:
            before, _, body = body.partition(f.open_tag)
            had_open = True
            if before.strip() and not f.starts_in_reasoning:
                # text before the opening tag is answer text
                reasoning, _, after = body.partition(f.close_tag)
                return (reasoning.strip() or None), (before + after).strip()
        if not had_open and not f.starts_in_reasoning:
            return None, text
        if f.close_tag in body:
            reasoning, _, answer = body.partition(f.close_tag)
            return (reasoning.strip() or None), answer.lstrip("\n")
        return (body.strip() or None), ""  # reasoning never closed: all of it is reasoning

    def parse_stream_chunk(self, delta: str) -> Tuple[str, str]:
        """(reasoning delta, answer delta) for the next piece of a stream."""
        f = self.family
        self._pending += delta
        reasoning_out, answer_out = "", ""
        while self._pending:
            if self._done:
                if self._strip_nl:  # newlines right after the closing tag are not part of the answer
                    self._pending = self._pending.lstrip("\n")
                    if not self._pending:
                        break
                    self._strip_nl = False
                answer_out += self._pending
                self._pending = ""
                break
            if not self._in_reasoning:
                idx = self._pending.find(f.open_tag)
                if idx >= 0 and not self._seen_open:
                    answer_out += self._pending[:idx]
                    self._pending = self._pending[idx + len(f.open_tag):]
                    self._in_reasoning = self._seen_open = True
                    continue
                keep = _held_back(self._pending, f.open_tag) if not self._seen_open else 0
                answer_out += self._pending[: len(self._pending) - keep]
                self._pending = self._pending[len(self._pending) - keep:]
                break
            # inside reasoning
            if not self._seen_open and self._pending.startswith(f.open_tag):
                self._pending = self._pending[len(f.open_tag):]
                self._seen_open = True
                continue
            if not self._seen_open and f.open_tag.startswith(self._pending):
                break  # may still become an opening tag
            idx = self._pending.find(f.close_tag)
            if idx >= 0:
                reasoning_out += self._pending[:idx]
                self._pending = self._pending[idx + len(f.close_tag):]
                self._in_reasoning, self._done, self._strip_nl = False, True, True
                continue
            keep = _held_back(self._pending, f.close_tag)
            reasoning_out += self._pending[: len(self._pending) - keep]
            self._pending = self._pending[len(self._pending) - keep:]
            break
        if not self.stream_reasoning:
            self._reasoning_buf += reasoning_out
            if self._done and self._reasoning_buf:
                reasoning_out, self._reasoning_buf = self._reasoning_buf, ""
            else:
                reasoning_out = ""
        return reasoning_out, answer_out
