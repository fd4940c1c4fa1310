"""ZMQ plumbing of the multi-process engine (role of pymllm/orchestrator/ipc_utils.py:15-105):
``ipc://`` endpoints under a per-engine temp directory, PUSH/PULL sockets with no linger."""

from __future__ import annotations

import logging
import os
import tempfile
from typing import List


def ipc_dir() -> str:
    d = os.path.join(tempfile.gettempdir(), "mllm_b200_ipc")
    os.makedirs(d, exist_ok=True)
    return d


def make_ipc_address(name: str, unique: str) -> str:
    return f"ipc://{ipc_dir()}/mllm_b200_{name}_{unique}"


def make_socket(ctx, sock_type, addr: str, bind: bool):
    import zmq

    s = ctx.socket(sock_type)
    s.setsockopt(zmq.LINGER, 0)
    if sock_type == zmq.PUSH:
        s.setsockopt(zmq.SNDHWM, 0)
    else:
        s.setsockopt(zmq.RCVHWM, 0)
    if bind:
        s.bind(addr)
    else:
        s.connect(addr)
    return s


def cleanup_ipc(addresses: List[str]) -> None:
    for a in addresses:
        path = a.replace("ipc://", "")
        try:
            os.unlink(path)
        except OSError:
            pass


def setup_subprocess_logging(level: str = "info") -> None:
    logging.basicConfig(level=getattr(logging, str(level).upper(), logging.INFO),
                        format=f"%(asctime)s [pid {os.getpid()}] %(name)s %(levelname)s %(message)s")
