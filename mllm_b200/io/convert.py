"""Checkpoint conversion between HF safetensors and the ``.mllm`` V2 container (role of the reference's
``pymllm/mobile/convertor`` command line: model_file_v2.py, ``mllm-convertor``).

    python -m mllm_b200.io.convert --input <dir with *.safetensors> --output model.mllm [--model-name NAME] [--dtype bf16]
    python -m mllm_b200.io.convert --input model.mllm --output out_dir --to-safetensors
"""

from __future__ import annotations

import argparse
import glob
import os
from typing import Iterator, Optional, Tuple

import torch

from .mllm_file import MllmFileReader, iter_mllm_tensors, write_mllm

_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def iter_safetensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    from safetensors import safe_open

    files = sorted(glob.glob(os.path.join(path, "*.safetensors"))) if os.path.isdir(path) else [path]
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {path}")
    for f in files:
        with safe_open(f, framework="pt", device="cpu") as fh:
            for k in fh.keys():
                yield k, fh.get_tensor(k)


def safetensors_to_mllm(src: str, dst: str, model_name: str = "", dtype: Optional[torch.dtype] = None) -> int:
    def cast(it):
        for name, t in it:
            yield name, (t.to(dtype) if dtype is not None and t.is_floating_point() else t)

    items = list(cast(iter_safetensors(src)))
    write_mllm(dst, items, model_name=model_name)
    return len(items)


def mllm_to_safetensors(src: str, dst_dir: str, gguf_dtype: torch.dtype = torch.bfloat16) -> int:
    from safetensors.torch import save_file

    os.makedirs(dst_dir, exist_ok=True)
    tensors = {name: t.clone().contiguous() for name, t in iter_mllm_tensors(src, gguf_dtype)}
    save_file(tensors, os.path.join(dst_dir, "model.safetensors"))
    return len(tensors)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--model-name", default="")
    ap.add_argument("--dtype", choices=sorted(_DTYPES), default=None, help="cast floating-point tensors while converting")
    ap.add_argument("--to-safetensors", action="store_true")
    ap.add_argument("--list", action="store_true", help="print the parameters of a .mllm file and exit")
    a = ap.parse_args(argv)
    if a.list:
        r = MllmFileReader(a.input)
        print(f"version {r.version} model_name {r.model_name!r}")
        for n in r.names():
            dt, shape, size, off = r.info(n)
            print(f"{n}\tdtype_id={dt}\tshape={list(shape)}\tbytes={size}\toffset={off}")
        return
    if a.to_safetensors:
        n = mllm_to_safetensors(a.input, a.output, _DTYPES.get(a.dtype or "bf16"))
    else:
        n = safetensors_to_mllm(a.input, a.output, a.model_name, _DTYPES.get(a.dtype) if a.dtype else None)
    print(f"wrote {n} tensors to {a.output}")


if __name__ == "__main__":
    main()
