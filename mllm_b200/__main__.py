"""``python -m mllm_b200 <command>`` — helper commands (role of ``pymllm show-config`` in the reference).

    show-config   versions, CUDA / GPU facts, which compiled extensions load, supported architectures and
                  quantisation methods
    models        the supported architecture names, one per line
"""

from __future__ import annotations

import argparse
import json


def show_config() -> dict:
    import torch

    from . import ops
    from .models import supported_architectures
    from .quantization import list_quantization_methods

    info = {"torch": torch.__version__, "cuda_runtime": torch.version.cuda, "cuda_available": torch.cuda.is_available(),
            "architectures": supported_architectures(), "quantization": list_quantization_methods()}
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        info["gpu"] = {"name": p.name, "capability": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                       "memory_gib": round(p.total_memory / 2 ** 30, 1), "count": torch.cuda.device_count()}
    ext = {}
    try:
        ext["mllm_b200_C"] = ops.ext() is not None
    except Exception as exc:
        ext["mllm_b200_C"] = f"not loaded: {exc}"
    try:
        from .mem_cache.native import host_ext

        ext["mllm_b200_host"] = host_ext() is not None
    except Exception as exc:
        ext["mllm_b200_host"] = f"not loaded: {exc}"
    info["extensions"] = ext
    return info


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="python -m mllm_b200", description="mllm_b200 helper commands.")
    ap.add_argument("command", nargs="?", choices=["show-config", "models"])
    a = ap.parse_args(argv)
    if a.command == "show-config":
        print(json.dumps(show_config(), indent=1))
    elif a.command == "models":
        from .models import supported_architectures

        print("\n".join(supported_architectures()))
    else:
        ap.print_help()


if __name__ == "__main__":
    main()
