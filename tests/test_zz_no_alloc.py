"""GPU: b200moe_sort_static — the token sort for callers that cannot allocate device memory — against the regular
b200moe_topk_bits + b200moe_sort path, through the C ABI, on two calls in a row.

Who needs it: a process that has given every byte of HBM to its own pool and must never reach cudaMalloc, a plugin
whose device-memory budget is fixed when it is loaded, code inside a region where allocating is forbidden.  The entry
point keeps its scratch tables in a fixed array inside the library; the second call below runs on a different problem
size so that whatever the first call left in that array would show up if anything depended on it.  This file sorts last
in the collection order on purpose.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sorted_reference(lib, K, idx, w, T, E, off):
    """Existing entry points, workspace-backed."""
    from fused_moe_b200 import _lib
    from fused_moe_b200.kernel import _workspace
    dev = idx.device
    stream = torch.cuda.current_stream().cuda_stream
    ws = _workspace(dev, T, E, stream)
    p = _lib.Problem()
    p.T, p.E_local, p.local_expert_offset = T, E, off
    p.topk_idx_in, p.topk_w_in = idx.data_ptr(), w.data_ptr()
    _lib.check(lib.b200moe_topk_bits(C.byref(p), C.byref(ws.struct), stream), "topk_bits")
    _lib.check(lib.b200moe_sort(C.byref(p), C.byref(ws.struct), stream), "sort")
    torch.cuda.synchronize()
    R = ws.struct.R_max
    tb = int(ws.view("total_blocks", torch.int32, (1,)).item())
    return dict(counts=ws.view("counts", torch.int32, (E,)).clone(),
                block_offsets=ws.view("block_offsets", torch.int32, (E + 1,)).clone(), total_blocks=tb,
                sorted_token_ids=ws.view("sorted_token_ids", torch.int32, (R,))[:tb * 128].clone(),
                sorted_weights=ws.view("sorted_weights", torch.float32, (R,))[:tb * 128].clone(),
                scatter_map=ws.view("scatter_map", torch.int32, (T, 8)).clone())


def _sorted_static(lib, idx, w, T, E, off):
    """New entry point: every buffer is the caller's, the library allocates nothing."""
    from fused_moe_b200 import _lib
    dev = idx.device
    R = (8 * T // 128 + E) * 128
    counts = torch.full((E,), -1, dtype=torch.int32, device=dev)
    offs = torch.full((E + 1,), -1, dtype=torch.int32, device=dev)
    total = torch.full((1,), -1, dtype=torch.int32, device=dev)
    ids = torch.full((R,), -1, dtype=torch.int32, device=dev)
    sw = torch.full((R,), float("nan"), dtype=torch.float32, device=dev)
    smap = torch.full((T, 8), -7, dtype=torch.int32, device=dev)
    before = torch.cuda.memory_allocated(dev)
    rc = lib.b200moe_sort_static(idx.data_ptr(), w.data_ptr(), T, E, off, counts.data_ptr(), offs.data_ptr(),
                                 total.data_ptr(), ids.data_ptr(), sw.data_ptr(), smap.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "b200moe_sort_static")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    tb = int(total.item())
    return dict(counts=counts, block_offsets=offs, total_blocks=tb, sorted_token_ids=ids[:tb * 128],
                sorted_weights=sw[:tb * 128], scatter_map=smap)


def test_sort_static_matches_sort_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fused_moe_b200 import _lib, kernel as K, synth
    lib = _lib.load()
    # second call: fewer tokens, more experts, another offset — it reuses the array the first call filled.  The third
    # and fourth have more than 32 chunks of 32 tokens, where the sort uses BOTH tables of the fixed array (the bit
    # matrix and the per-chunk prefix) and a separate scan kernel; they run right after a smaller call, and the last is
    # smaller again, so leftovers of every size are in the array at some point.
    for T, E, off, seed, skew in ((300, 32, 64, 4, True), (77, 64, 128, 9, False), (1100, 8, 16, 2, True),
                                  (2000, 16, 208, 6, False), (33, 256, 0, 7, True)):
        inp = synth.make_inputs(T, E, seed=seed, local_expert_offset=off, skew=skew, device="cuda", only_experts=[])
        idx, w = K.route(inp["routing_logits"], inp["routing_bias"], 2.5)
        want = _sorted_reference(lib, K, idx, w, T, E, off)
        got = _sorted_static(lib, idx, w, T, E, off)
        assert got["total_blocks"] == want["total_blocks"] > 0
        for name in ("counts", "block_offsets", "sorted_token_ids", "sorted_weights", "scatter_map"):
            assert torch.equal(got[name], want[name]), f"{name} differs (T={T}, E={E})"  # integers and copied weights: exact


def test_sort_static_rejects_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fused_moe_b200 import _lib
    lib = _lib.load()
    d = torch.zeros(64, dtype=torch.int32, device="cuda")
    args = lambda T, E, off: (d.data_ptr(), d.data_ptr(), T, E, off) + (d.data_ptr(),) * 6 + (None,)
    T_big = 32 * (_lib.SORT_STATIC_MAX_ENTRIES // 32) + 1          # one chunk too many at 32 local experts
    assert lib.b200moe_sort_static(*args(T_big, 32, 0)) == _lib.ETOOLARGE
    assert lib.b200moe_strerror(_lib.ETOOLARGE) != b"unknown error"
    assert lib.b200moe_sort_static(*args(8, 0, 0)) == _lib.EINVAL
    assert lib.b200moe_sort_static(*args(8, 32, 240)) == _lib.EINVAL
