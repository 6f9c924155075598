"""CPU: the C-ABI library loads, exports every symbol include/b200moe.h declares, and its host-only entry points
(sizing, carving, error strings) behave; the Python entry point validates arguments and refuses to run without CUDA."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

from fused_moe_b200 import _lib, build, kernel as K, synth

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_header_symbols_exported(lib):
    header = (ROOT / "include" / "b200moe.h").read_text()
    declared = set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SYMBOLS), f"binding and header differ: {declared ^ set(_lib.SYMBOLS)}"
    for name in declared:
        assert hasattr(lib, name), f"{name} not exported by libb200moe.so"


def test_struct_mirrors_match_header():
    header = (ROOT / "include" / "b200moe.h").read_text()
    for cls, cname in ((_lib.Problem, "b200moe_problem"), (_lib.Workspace, "b200moe_workspace"),
                       (_lib.EpPeers, "b200moe_ep_peers")):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = re.findall(r"(\w+)\s*(?:\[\d+\])?;", body)
        assert names == [f[0] for f in cls._fields_]


def test_version_and_strerror(lib):
    assert lib.b200moe_version() >= 100
    assert lib.b200moe_strerror(0) == b"ok"
    for code in range(-6, 0):
        assert lib.b200moe_strerror(code) not in (b"ok", b"unknown error")
    assert lib.b200moe_strerror(-99) == b"unknown error"


def test_workspace_sizing_and_carving(lib):
    n = C.c_size_t(0)
    assert lib.b200moe_workspace_bytes(80, 32, C.byref(n)) == 0
    small = n.value
    assert lib.b200moe_workspace_bytes(16384, 32, C.byref(n)) == 0
    assert n.value > small > 0
    # R_max rows of fp8 activations + two-term intermediate + bf16 expert rows dominate
    r_max = (8 * 16384 // 128 + 32) * 128
    assert n.value >= r_max * (7168 + 2 * 2048 + 2 * 7168)
    assert lib.b200moe_workspace_bytes(-1, 32, C.byref(n)) == _lib.EINVAL
    assert lib.b200moe_workspace_bytes(8, 0, C.byref(n)) == _lib.EINVAL
    assert lib.b200moe_workspace_bytes(8, 257, C.byref(n)) == _lib.EINVAL
    assert lib.b200moe_workspace_bytes(8, 32, None) == _lib.EINVAL

    ws = _lib.Workspace()
    need = K.workspace_bytes(7, 4)
    base = 1 << 20  # carving only does pointer arithmetic
    assert lib.b200moe_workspace_carve(base, need, 7, 4, C.byref(ws)) == 0
    assert (ws.T, ws.E_local, ws.n_chunks) == (7, 4, 1)
    assert ws.R_max == (8 * 7 // 128 + 4) * 128
    assert _lib.Workspace._fields_[-1][0] == "status_mirror" and not ws.status_mirror   # the caller's to set
    ptrs = [getattr(ws, f[0]) for f in _lib.Workspace._fields_[4:-1]]
    assert ptrs == sorted(ptrs) and all(p % 256 == 0 for p in ptrs)
    assert ptrs[0] == base and ptrs[-1] + 2 * ws.R_max * 7168 <= base + need
    assert lib.b200moe_workspace_carve(base, need - 1, 7, 4, C.byref(ws)) == _lib.EWORKSPACE
    assert lib.b200moe_workspace_carve(base + 8, need, 7, 4, C.byref(ws)) == _lib.EWORKSPACE
    assert lib.b200moe_workspace_carve(None, need, 7, 4, C.byref(ws)) == _lib.EINVAL


def test_problem_workspace_mismatch_is_rejected(lib):
    ws = _lib.Workspace()
    need = K.workspace_bytes(7, 4)
    assert lib.b200moe_workspace_carve(1 << 20, need, 7, 4, C.byref(ws)) == 0
    p = _lib.Problem()
    p.T, p.E_local, p.local_expert_offset = 8, 4, 0
    assert lib.b200moe_forward(C.byref(p), C.byref(ws), None) == _lib.EWORKSPACE
    p.T, p.local_expert_offset = 7, 254
    assert lib.b200moe_forward(C.byref(p), C.byref(ws), None) == _lib.EINVAL
    p.local_expert_offset = 0  # null tensors
    assert lib.b200moe_forward(C.byref(p), C.byref(ws), None) == _lib.EINVAL


def test_check_raises():
    with pytest.raises(ValueError):
        _lib.check(_lib.EINVAL, "x")
    with pytest.raises(RuntimeError):
        _lib.check(_lib.EWORKSPACE, "x")
    _lib.check(0, "x")


def test_kernel_refuses_cpu_tensors_and_bad_arguments():
    inp = synth.make_inputs(3, 1, seed=2, only_experts=[])
    with pytest.raises(RuntimeError, match="no CPU path"):
        K.kernel(**inp)
    bad = dict(inp)
    bad["routing_bias"] = inp["routing_bias"].float()
    with pytest.raises(TypeError):
        K.kernel(**bad)
    bad = dict(inp)
    bad["gemm2_weights_scale"] = inp["gemm2_weights_scale"][:, :, :8]
    with pytest.raises(ValueError):
        K.kernel(**bad)
    bad = dict(inp)
    bad["routing_logits"] = inp["routing_logits"][0]
    with pytest.raises(ValueError):
        K.kernel(**bad)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_synth_is_reproducible_and_shaped():
    a = synth.make_inputs(5, 2, seed=9, local_expert_offset=10, only_experts=[1])
    b = synth.make_inputs(5, 2, seed=9, local_expert_offset=10, only_experts=[1])
    for k, v in a.items():
        if torch.is_tensor(v):
            assert torch.equal(v.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else v,
                               b[k].view(torch.uint8) if v.dtype == torch.float8_e4m3fn else b[k])
    assert a["hidden_states_scale"].shape == (56, 5) and a["gemm1_weights"].shape == (2, 4096, 7168)
    assert not a["gemm1_weights"][0].view(torch.uint8).any() and a["gemm1_weights"][1].view(torch.uint8).any()
    # dequantised activations reproduce the bf16 source to fp8 precision
    deq = a["hidden_states"].float().view(5, 56, 128) * a["hidden_states_scale"].t().unsqueeze(2)
    assert deq.abs().max() < 6 and 0.8 < deq.std() < 1.2
    assert a["hidden_states"].float().abs().max() <= 448


def test_ctypes_mirrors_match_the_header_layout(tmp_path):
    """Every structure of include/b200moe.h, as laid out by the C compiler (sizeof and the offset of every field), equals
    the package's ctypes mirror of it: what crosses the boundary is read the same way on both sides."""
    import ctypes as C
    import shutil
    import subprocess
    from pathlib import Path
    from fused_moe_b200 import _lib
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    root = Path(__file__).resolve().parent.parent
    pairs = {"b200moe_problem": _lib.Problem, "b200moe_workspace": _lib.Workspace, "b200moe_ep_peers": _lib.EpPeers,
             "b200moe_ep_plan": _lib.EpPlan}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "b200moe.h"', 'int main(void) {']
    for cname, mirror in pairs.items():
        lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
        for field, _ in mirror._fields_:
            lines.append(f'  printf("{cname}.{field} %zu\\n", offsetof({cname}, {field}));')
    # the constants the package repeats on the Python side
    consts = {"B200MOE_SORT_STATIC_MAX_ENTRIES": _lib.SORT_STATIC_MAX_ENTRIES, "B200MOE_EP_RECORD_BYTES": _lib.EP_RECORD_BYTES,
              "B200MOE_DECODE_MAX_T": _lib.DECODE_MAX_T, "B200MOE_DECODE_MAX_WORK": _lib.DECODE_MAX_WORK,
              "B200MOE_SKINNY_MAX_T": _lib.SKINNY_MAX_T, "B200MOE_PROLOGUE_MAX_T": _lib.PROLOGUE_MAX_T,
              "B200MOE_PARTIAL_F32": _lib.PARTIAL_F32, "B200MOE_PARTIAL_HALF": _lib.PARTIAL_HALF,
              "B200MOE_HALF_ROW_BYTES": _lib.HALF_ROW_BYTES}
    for cname in consts:
        lines.append(f'  printf("{cname} %d\\n", (int){cname});')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([cc, "-I", str(root / "include"), str(src), "-o", str(exe)], check=True)
    got = dict(l.split() for l in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, value in consts.items():
        assert int(got[cname]) == value, cname
    assert _lib.HALF_ROW_BYTES == 7168 * 2 + 7168 // 8
    for cname, mirror in pairs.items():
        assert int(got[cname]) == C.sizeof(mirror), cname
        for field, _ in mirror._fields_:
            assert int(got[f"{cname}.{field}"]) == getattr(mirror, field).offset, f"{cname}.{field}"
