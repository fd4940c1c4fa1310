"""Weight-only block quantisation of a checkpoint into a ``.mllm`` V2 file (role of the reference's
``mllm-quantizer`` tool with its GGUF schemas).

    python -m mllm_b200.io.quantize --input <model.mllm | dir with *.safetensors> --output q.mllm \\
        --scheme q4_0 [--include REGEX] [--exclude REGEX] [--keep-dtype bf16]

Matrices (2-D tensors whose row length is a multiple of 32) whose names match ``--include`` and not
``--exclude`` are stored as GGUF ``Q4_0`` or ``Q8_0`` blocks of 32 values; everything else is stored
as it is (or cast to ``--keep-dtype``).  The engine's loader expands such blocks when it reads the file.

Block layouts (little endian):

* ``Q8_0``: fp16 scale ``d = max|x| / 127`` followed by 32 int8 values ``round(x / d)`` — 34 bytes.
* ``Q4_0``: fp16 scale ``d = m / -8`` where ``m`` is the value of largest magnitude (sign kept), then
  16 bytes; byte ``j`` holds code ``j`` in its low nibble and code ``j + 16`` in its high nibble, a
  code being ``clip(round(x / d) + 8, 0, 15)`` — 18 bytes.
"""

from __future__ import annotations

import argparse
import os
import re
from typing import Iterator, Optional, Tuple

import numpy as np
import torch

from ..mem_cache.native import host_ext
from .mllm_file import DTYPE_IDS, iter_mllm_tensors

SCHEMES = {"q4_0": 2, "q8_0": 8}
_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
DEFAULT_EXCLUDE = r"(norm|embed_tokens|lm_head|bias|A_log|dt_bias|conv1d)"


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    blk = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    d = (np.abs(blk).max(axis=1) / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df > 0, 1.0 / np.where(df > 0, df, 1.0), 0.0).astype(np.float32)
    q = np.clip(np.rint(blk * inv[:, None]), -127, 127).astype(np.int8)
    out = np.empty((blk.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    blk = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    idx = np.abs(blk).argmax(axis=1)
    m = blk[np.arange(blk.shape[0]), idx]
    d = (m / -8.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1.0), 0.0).astype(np.float32)
    q = np.clip(np.rint(blk * inv[:, None]) + 8, 0, 15).astype(np.uint8)
    out = np.empty((blk.shape[0], 18), dtype=np.uint8)
    out[:, :2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


_QUANT = {"q4_0": quantize_q4_0, "q8_0": quantize_q8_0}


def _source(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    if os.path.isdir(path) or path.endswith(".safetensors"):
        from .convert import iter_safetensors

        return iter_safetensors(path)
    return iter_mllm_tensors(path)


def quantize_file(src: str, dst: str, scheme: str = "q4_0", include: str = r"\.weight$",
                  exclude: str = DEFAULT_EXCLUDE, keep_dtype: Optional[torch.dtype] = None, model_name: str = "") -> dict:
    if scheme not in SCHEMES:
        raise ValueError(f"scheme must be one of {sorted(SCHEMES)}")
    inc, exc = re.compile(include), re.compile(exclude) if exclude else None
    entries, stats = [], {"quantized": 0, "kept": 0, "bytes_in": 0, "bytes_out": 0}
    for name, t in _source(src):
        t = t.detach().cpu().contiguous()
        stats["bytes_in"] += t.numel() * t.element_size()
        take = (t.dim() == 2 and t.is_floating_point() and t.shape[1] % 32 == 0 and inc.search(name)
                and not (exc is not None and exc.search(name)))
        if take:
            raw = _QUANT[scheme](t.float().numpy())
            entries.append((name, SCHEMES[scheme], [int(s) for s in t.shape], raw))
            stats["quantized"] += 1
        else:
            if keep_dtype is not None and t.is_floating_point():
                t = t.to(keep_dtype)
            if t.dtype not in DTYPE_IDS:
                raise ValueError(f"{name}: dtype {t.dtype} has no .mllm id")
            raw = t.view(torch.uint8).reshape(-1).numpy() if t.numel() else np.empty(0, dtype=np.uint8)
            entries.append((name, DTYPE_IDS[t.dtype], [int(s) for s in t.shape], raw))
            stats["kept"] += 1
        stats["bytes_out"] += int(entries[-1][3].size)
    host_ext().write_mllm_v2(str(dst), model_name, entries)
    return stats


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--scheme", choices=sorted(SCHEMES), default="q4_0")
    ap.add_argument("--include", default=r"\.weight$")
    ap.add_argument("--exclude", default=DEFAULT_EXCLUDE)
    ap.add_argument("--keep-dtype", choices=sorted(_DTYPES), default=None)
    ap.add_argument("--model-name", default="")
    a = ap.parse_args(argv)
    st = quantize_file(a.input, a.output, a.scheme, a.include, a.exclude,
                       _DTYPES[a.keep_dtype] if a.keep_dtype else None, a.model_name)
    print(f"{a.output}: {st['quantized']} tensors as {a.scheme}, {st['kept']} kept; "
          f"{st['bytes_in'] / 2 ** 20:.1f} MiB -> {st['bytes_out'] / 2 ** 20:.1f} MiB")


if __name__ == "__main__":
    main()
