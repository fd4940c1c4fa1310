"""Build / load the native extensions in-tree.

Two extensions live under ``mllm_b200/csrc``:

* ``mllm_b200_C``    — the sm_100a CUDA kernels plus their PyTorch binding;
* ``mllm_b200_host`` — host-only C++ (radix tree, page allocator, ``.mllm`` file reader).

They are compiled with ``torch.utils.cpp_extension.load`` into ``mllm_b200/_ext`` so the
shared objects sit beside the package (not in a user cache) and travel with the source
tree.  A content hash of the sources is stored next to each ``.so``; at import time a
``.so`` whose hash matches is loaded directly, without invoking ninja.
"""

from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading
from pathlib import Path
from types import ModuleType
from typing import Dict, List, Optional

_PKG = Path(__file__).resolve().parent
_CSRC = _PKG / "csrc"
_OUT = _PKG / "_ext"

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17"]

EXTENSIONS: Dict[str, Dict[str, List[str]]] = {
    "mllm_b200_C": {
        "sources": ["bindings.cpp", "elementwise.cu", "gemm_tcgen05.cu", "attention.cu", "sampling.cu", "moe.cu",
                    "comm.cu", "gemm_w4a16.cu", "vision.cu", "gdn.cu", "gdn_chunk.cu", "no_alloc.cu", "ep_a2a.cu", "gemm_smallm.cu", "gemm_smallm_w4.cu"],
        "headers": ["common.cuh", "kernels.h", "no_alloc.h"],
        "cuda": True,
    },
    "mllm_b200_host": {
        "sources": ["host/host_bindings.cpp", "host/radix_tree.cpp", "host/page_allocator.cpp", "host/mllm_file.cpp", "host/cpu_oracle.cpp", "host/symm_heap.cpp"],
        "headers": ["host/radix_tree.h", "host/page_allocator.h", "host/mllm_file.h", "host/cpu_oracle.h", "host/symm_heap.h"],
        "cuda": False,
    },
}

_loaded: Dict[str, ModuleType] = {}
_lock = threading.Lock()


def _existing(names: List[str]) -> List[Path]:
    return [(_CSRC / n) for n in names if (_CSRC / n).exists()]


def _source_hash(name: str) -> str:
    spec = EXTENSIONS[name]
    h = hashlib.sha256()
    for p in sorted(_existing(spec["sources"]) + _existing(spec["headers"])):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(CUDA_FLAGS if spec["cuda"] else CXX_FLAGS).encode())
    return h.hexdigest()


def _so_path(name: str) -> Path:
    return _OUT / name / f"{name}.so"


def _hash_path(name: str) -> Path:
    return _OUT / name / "source.sha256"


def _import_so(name: str) -> ModuleType:
    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location(name, _so_path(name))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[name] = mod
    return mod


def is_built(name: str) -> bool:
    return _so_path(name).exists() and _hash_path(name).exists() and _hash_path(name).read_text().strip() == _source_hash(name)


def build_extension(name: str, verbose: bool = False) -> ModuleType:
    """Compile ``name`` (if its sources changed) and import it."""
    from torch.utils import cpp_extension

    spec = EXTENSIONS[name]
    out = _OUT / name
    out.mkdir(parents=True, exist_ok=True)
    sources = [str(p) for p in _existing(spec["sources"])]
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 1)))
    mod = cpp_extension.load(
        name=name,
        sources=sources,
        extra_cflags=CXX_FLAGS,
        extra_cuda_cflags=CUDA_FLAGS if spec["cuda"] else None,
        extra_include_paths=[str(_CSRC)],
        build_directory=str(out),
        with_cuda=spec["cuda"],
        verbose=verbose,
    )
    _hash_path(name).write_text(_source_hash(name))
    sys.modules[name] = mod
    return mod


def load_extension(name: str, build_if_missing: bool = True) -> Optional[ModuleType]:
    """Import ``name`` from the in-tree ``.so``; compile first when it is missing or stale."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
        mod: Optional[ModuleType] = None
        if is_built(name):
            mod = _import_so(name)
        elif build_if_missing:
            mod = build_extension(name)
        if mod is not None:
            _loaded[name] = mod
        return mod


def build_all(verbose: bool = False) -> None:
    for name in EXTENSIONS:
        if not _existing(EXTENSIONS[name]["sources"]):
            continue
        if not is_built(name):
            build_extension(name, verbose=verbose)
        load_extension(name)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print("built:", {n: str(_so_path(n)) for n in EXTENSIONS})
