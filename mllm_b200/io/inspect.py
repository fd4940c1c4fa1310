"""Lists what a ``.mllm`` parameter file holds (role of the reference's ``mllm-params-inspector`` tool).

    python -m mllm_b200.io.inspect model.mllm [--filter REGEX] [--json]
"""

from __future__ import annotations

import argparse
import json
import re
from typing import Dict, List

from .mllm_file import _ID_TO_DTYPE, GGUF_IDS, MllmFileReader


def dtype_name(dtype_id: int) -> str:
    if dtype_id in GGUF_IDS:
        return f"gguf_{GGUF_IDS[dtype_id].lower()}"
    if dtype_id in _ID_TO_DTYPE:
        return str(_ID_TO_DTYPE[dtype_id]).replace("torch.", "")
    return f"id{dtype_id}"


def describe(path: str, pattern: str = "") -> Dict:
    r = MllmFileReader(path)
    rx = re.compile(pattern) if pattern else None
    rows: List[Dict] = []
    for name in r.names():
        if rx is not None and not rx.search(name):
            continue
        dtype_id, shape, size, offset = r.info(name)
        rows.append({"name": name, "dtype": dtype_name(dtype_id), "shape": list(shape), "bytes": size, "offset": offset})
    by_dtype: Dict[str, int] = {}
    for row in rows:
        by_dtype[row["dtype"]] = by_dtype.get(row["dtype"], 0) + row["bytes"]
    return {"path": str(path), "version": r.version, "model_name": r.model_name, "tensors": rows,
            "total_bytes": sum(x["bytes"] for x in rows), "bytes_by_dtype": by_dtype}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("path")
    ap.add_argument("--filter", default="", help="only names matching this regular expression")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    d = describe(a.path, a.filter)
    if a.json:
        print(json.dumps(d))
        return
    print(f"{d['path']}: .mllm V{d['version']}  model_name={d['model_name']!r}  {len(d['tensors'])} tensors, "
          f"{d['total_bytes'] / 2 ** 20:.1f} MiB")
    width = max([len(x["name"]) for x in d["tensors"]] + [4])
    for x in d["tensors"]:
        print(f"  {x['name']:<{width}}  {x['dtype']:<10} {str(tuple(x['shape'])):<22} {x['bytes']:>12d} B")
    for k, v in sorted(d["bytes_by_dtype"].items()):
        print(f"  [{k}] {v / 2 ** 20:.1f} MiB")


if __name__ == "__main__":
    main()
