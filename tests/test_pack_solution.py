"""CPU: the solution.json packer emits the reference's wire format (scripts/pack_solution_simple.py:58-75) and the
unpacked tree is importable source (no build, no GPU here)."""
import json
import py_compile

from fused_moe_b200 import pack_solution


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
