"""Tracing helpers: NVTX ranges around engine phases and a ``torch.profiler`` context that writes a
Chrome trace (role of the ``--profile`` switches of pymllm/bench_one_batch.py:96-111, 405-446)."""

from __future__ import annotations

import contextlib
import os
import time
from typing import Iterable, Iterator, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str) -> Iterator[None]:
    """NVTX range when CUDA is present (shows up in Nsight timelines); no-op otherwise."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


@contextlib.contextmanager
def torch_profiler(enabled: bool, activities: Iterable[str] = ("CPU", "GPU"), record_shapes: bool = False,
                   output_dir: Optional[str] = None, filename_prefix: str = "mllm_b200", tag: str = "",
                   exported: Optional[list] = None) -> Iterator[Optional[object]]:
    """``with torch_profiler(True, ...) as prof:`` profiles the block and exports
    ``<output_dir>/<prefix>_<tag>_<time>.trace.json.gz`` (the path is appended to ``exported`` when given).
    ``"CUDA_PROFILER"`` in ``activities`` brackets the block with cudaProfilerStart/Stop instead (for
    external tools)."""
    if not enabled:
        yield None
        return
    acts = set(a.upper() for a in activities)
    if "CUDA_PROFILER" in acts and torch.cuda.is_available():
        torch.cuda.cudart().cudaProfilerStart()
        try:
            yield None
        finally:
            torch.cuda.cudart().cudaProfilerStop()
        return
    from torch.profiler import ProfilerActivity, profile

    pa = []
    if "CPU" in acts:
        pa.append(ProfilerActivity.CPU)
    if "GPU" in acts and torch.cuda.is_available():
        pa.append(ProfilerActivity.CUDA)
    out_dir = output_dir or os.environ.get("MLLM_B200_PROFILE_DIR", "/tmp")
    os.makedirs(out_dir, exist_ok=True)
    with profile(activities=pa, record_shapes=record_shapes) as prof:
        yield prof
    name = "_".join(x for x in (filename_prefix, tag, str(int(time.time()))) if x)
    path = os.path.join(out_dir, name + ".trace.json.gz")
    prof.export_chrome_trace(path)
    prof.exported_path = path
    if exported is not None:
        exported.append(path)
