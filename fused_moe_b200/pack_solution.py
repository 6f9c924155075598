"""Packs this implementation into the contest's ``solution.json`` wire format.

The reference ships its kernels to the benchmark harness as one JSON document (scripts/pack_solution_simple.py:58-75;
schema as in the reference's own solution.json): ``name``, ``definition``, ``author``, ``spec`` (language, target
hardware, entry point ``kernel.py::kernel``, destination-passing style) and ``sources`` = a list of ``{path, content}``
text files that the harness writes to a directory and imports.  This module emits the same document for this
repository's code:

* ``kernel.py`` at the top level is a shim (imported by the harness as a submodule of a generated package): it builds ``libb200moe.so`` with nvcc on first import (the JSON format
  carries text only, so the library cannot travel prebuilt) and re-exports ``fused_moe_b200.kernel.kernel``;
* the package (``fused_moe_b200/*.py``, ``fused_moe_b200/csrc/*``) and ``include/b200moe.h`` keep their relative paths,
  which is what ``fused_moe_b200/build.py`` expects.

Usage:  python -m fused_moe_b200.pack_solution [-o solution.json] [--name NAME] [--author AUTHOR]
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Dict, List

ROOT = Path(__file__).resolve().parent.parent
DEFINITION = "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048"

# The harness writes the sources under <cache>/<pkg>/ and imports <pkg>.kernel (flashinfer_bench
# compile/builders/python_builder.py), so the shim reaches the package with relative imports.
SHIM = '''"""Entry point for the benchmark harness: builds the CUDA library once, then forwards to the package."""
from .fused_moe_b200 import build as _build

_build.build()          # nvcc, sm_100a; raises if the toolkit is missing: there is no fallback
from .fused_moe_b200.kernel import kernel  # noqa: E402,F401
'''

# what the operator needs at run time; tests, oracle, bench and the expert-parallel plumbing stay out
PACKAGE_FILES = ["__init__.py", "_lib.py", "build.py", "kernel.py"]


def gather_sources() -> List[Dict[str, str]]:
    files = [(ROOT / "fused_moe_b200" / f) for f in PACKAGE_FILES]
    files += sorted((ROOT / "fused_moe_b200" / "csrc").glob("*.cu")) + sorted((ROOT / "fused_moe_b200" / "csrc").glob("*.cuh"))
    files.append(ROOT / "include" / "b200moe.h")
    sources = [{"path": "kernel.py", "content": SHIM}]
    for p in files:
        sources.append({"path": p.relative_to(ROOT).as_posix(), "content": p.read_text(encoding="utf-8")})
    return sources


def pack(name: str = "b200-fused-moe", author: str = "b200-fused-moe") -> Dict:
    return {
        "name": name,
        "definition": DEFINITION,
        "author": author,
        "spec": {
            "language": "python",
            "target_hardware": ["cuda"],
            "entry_point": "kernel.py::kernel",
            "dependencies": [],
            "destination_passing_style": True,
            "binding": None,
        },
        "sources": gather_sources(),
        "description": "DeepSeek-V3 FP8 block-scale fused MoE layer, hand-written sm_100a CUDA behind a C ABI",
    }


def unpack(doc: Dict, dest: Path) -> List[Path]:
    """Writes the sources of a packed document under ``dest`` (what the harness's builder does) -> written paths."""
    out = []
    for s in doc["sources"]:
        p = dest / s["path"]
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text(s["content"], encoding="utf-8")
        out.append(p)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-o", "--output", default="solution.json")
    ap.add_argument("--name", default="b200-fused-moe")
    ap.add_argument("--author", default="b200-fused-moe")
    args = ap.parse_args()
    doc = pack(args.name, args.author)
    Path(args.output).write_text(json.dumps(doc, indent=2), encoding="utf-8")
    print(f"{args.output}: {len(doc['sources'])} sources, entry {doc['spec']['entry_point']}")


if __name__ == "__main__":
    main()
