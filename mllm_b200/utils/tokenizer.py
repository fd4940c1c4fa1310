"""Tokenizer access: HF ``AutoTokenizer`` for checkpoint directories, and a small self-contained
byte-level tokenizer for presets / directories without tokenizer files (benchmarks and tests run
without any download)."""

from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence


class ByteTokenizer:
    """UTF-8 bytes as token ids 0..255 plus a few specials; decodes any id sequence."""

    def __init__(self, vocab_size: int = 1024) -> None:
        self.vocab_size = max(int(vocab_size), 260)
        self.bos_token_id, self.eos_token_id, self.pad_token_id = 256, 257, 258
        self.eos_token = "<|endoftext|>"
        self.chat_template = None
        self.name_or_path = "byte-tokenizer"

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        return list(text.encode("utf-8"))

    def __call__(self, text, **kw) -> Dict[str, Any]:
        if isinstance(text, str):
            return {"input_ids": self.encode(text)}
        return {"input_ids": [self.encode(t) for t in text]}

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True, **kw) -> str:
        out = bytearray()
        for i in ids:
            i = int(i)
            if i < 256:
                out.append(i)
            elif not skip_special_tokens:
                out.extend(f"<|{i}|>".encode())
            else:  # ids beyond the byte range print as a replacement so lengths stay visible
                if i >= 260:
                    out.extend(b"?")
        return out.decode("utf-8", errors="replace")

    def batch_decode(self, batch, **kw) -> List[str]:
        return [self.decode(x, **kw) for x in batch]

    def apply_chat_template(self, messages, tokenize: bool = False, add_generation_prompt: bool = True, **kw):
        text = render_chatml(messages, add_generation_prompt)
        return self.encode(text) if tokenize else text


def render_chatml(messages: List[Dict[str, Any]], add_generation_prompt: bool = True) -> str:
    """ChatML rendering used when a tokenizer has no chat template."""
    parts = []
    for m in messages:
        content = m.get("content", "")
        if isinstance(content, list):
            content = "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type") == "text")
        parts.append(f"<|im_start|>{m.get('role', 'user')}\n{content}<|im_end|>\n")
    if add_generation_prompt:
        parts.append("<|im_start|>assistant\n")
    return "".join(parts)


def get_tokenizer(path: Optional[Any], vocab_size: int = 1024, mode: str = "auto", trust_remote_code: bool = False):
    s = str(path) if path is not None else ""
    has_files = s and not s.startswith("preset:") and os.path.isdir(s) and any(
        os.path.exists(os.path.join(s, f)) for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json"))
    if not has_files:
        return ByteTokenizer(vocab_size)
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(s, use_fast=(mode != "slow"), trust_remote_code=trust_remote_code)
