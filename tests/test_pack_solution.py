"""CPU: the solution.json packer emits the reference's wire format (scripts/pack_solution_simple.py:58-75) and the
unpacked tree is importable source (no build, no GPU here)."""
import importlib
import json
import os
import py_compile
import shutil
import sys

import pytest

from fused_moe_b200 import pack_solution


def load_like_the_harness(tmp_path, pkg="_fib_py_b200_fused_moe_test"):
    """What the harness's Python builder does with a solution (flashinfer_bench compile/builders/python_builder.py:
    write the sources under <tmp>/<pkg>/, put <tmp> on sys.path, import <pkg>.<entry file>, take the entry function),
    restated here because the wheel is not installed.  The library built in this checkout is copied next to the
    unpacked sources (newer than them), so the shim's build step finds it up to date instead of running nvcc again."""
    from fused_moe_b200 import _lib
    doc = pack_solution.pack()
    pkg_dir = tmp_path / pkg
    pack_solution.unpack(doc, pkg_dir)
    (pkg_dir / "__init__.py").write_text("")
    lib_dst = pkg_dir / "fused_moe_b200" / _lib.LIB_PATH.name
    shutil.copy2(_lib.LIB_PATH, lib_dst)
    os.utime(lib_dst, None)
    entry_file, entry_func = doc["spec"]["entry_point"].split("::")
    sys.path.insert(0, str(tmp_path))
    try:
        mod = importlib.import_module(pkg + "." + entry_file[:-3])
        return getattr(mod, entry_func)
    finally:
        sys.path.remove(str(tmp_path))


def test_document_has_the_reference_schema():
    doc = pack_solution.pack()
    assert set(doc) == {"name", "definition", "author", "spec", "sources", "description"}
    assert doc["definition"] == "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048"
    spec = doc["spec"]
    assert spec["language"] == "python" and spec["entry_point"] == "kernel.py::kernel"
    assert spec["destination_passing_style"] is True and spec["target_hardware"] == ["cuda"]
    json.loads(json.dumps(doc))  # plain JSON types only
    paths = [s["path"] for s in doc["sources"]]
    assert len(paths) == len(set(paths))
    for needed in ("kernel.py", "fused_moe_b200/kernel.py", "fused_moe_b200/_lib.py", "fused_moe_b200/build.py",
                   "fused_moe_b200/csrc/api.cu", "fused_moe_b200/csrc/gemm.cu", "fused_moe_b200/csrc/gemm_skinny.cu",
                   "fused_moe_b200/csrc/common.cuh", "include/b200moe.h"):
        assert needed in paths
    assert not any(p.startswith(("oracle/", "tests/", "_work/")) for p in paths)


def test_unpacked_tree_matches_the_repository(tmp_path):
    doc = pack_solution.pack()
    written = pack_solution.unpack(doc, tmp_path)
    assert len(written) == len(doc["sources"])
    for p in written:
        if p.suffix == ".py":
            py_compile.compile(str(p), doraise=True)
    # every source the build lists is present in the unpacked tree, at the place build.py looks for it
    from fused_moe_b200 import build
    for src in build.SOURCES:
        assert (tmp_path / "fused_moe_b200" / "csrc" / src).is_file()
    for hdr in build.HEADERS:
        assert (tmp_path / hdr.relative_to(pack_solution.ROOT)).is_file()


def test_entry_point_imports_the_way_the_harness_imports_it(tmp_path):
    from fused_moe_b200 import _lib
    if not _lib.LIB_PATH.exists():
        pytest.skip("libb200moe.so not built")
    fn = load_like_the_harness(tmp_path)
    assert callable(fn) and fn.__name__ == "kernel"
    assert fn.__module__.startswith("_fib_py_b200_fused_moe_test.fused_moe_b200")


@pytest.mark.gpu
def test_harness_call_site_matches_direct_call(tmp_path):
    """The packed solution, loaded and called as the harness calls it (keyword arguments named like the definition's
    inputs; compile/runnable.py), gives the bytes of the in-tree kernel()."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fused_moe_b200 import kernel as direct, synth
    fn = load_like_the_harness(tmp_path, pkg="_fib_py_b200_fused_moe_gpu")
    inp = synth.make_inputs(7, 32, seed=0, device="cuda")
    a = fn(**inp)
    b = direct.kernel(**inp)
    torch.cuda.synchronize()
    assert a.dtype == torch.bfloat16 and a.shape == (7, 7168)
    assert torch.equal(a, b)
    out = torch.empty_like(a)
    assert fn(**inp, output=out) is out and torch.equal(out, b)   # destination-passing style
