"""GPU: the failure paths of the library, exercised without harming the device.

A bounded wait is made to run out by waiting for a flag nobody sets, with the wait limit lowered to a few tens of
milliseconds (b200moe_set_wait_limit_cycles): the kernel returns, the status word says what happened, and the same
process goes on to compute a correct layer.  Nothing here traps, faults or spins without a limit.  The reference has no
device-side waits (its kernels never wait for one another), so there is no reference behaviour to compare with; the
contract tested is the one stated in include/b200moe.h."""
import ctypes as C

import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu

KEYS = ["routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
        "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset", "routed_scaling_factor"]


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fused_moe_b200 import _lib
    return _lib.load()


def _layer_still_correct(oracle, seed):
    from fused_moe_b200 import kernel as K, synth
    inp = synth.make_inputs(40, 8, seed=seed, local_expert_offset=96, skew=True, device="cuda")
    out = K.kernel(**inp)
    K.check_status()
    ref = oracle.kernel(*[inp[k] for k in KEYS])
    assert ref["pairs"] > 0
    assert_close(out.float().cpu(), ref["out_bf16"].float(), what="layer after a failed wait")


def test_barrier_wait_runs_out_and_the_gpu_stays_usable(lib, oracle):
    """A two-rank flag barrier whose second rank never arrives: both flag arrays are plain local buffers and nothing
    ever writes rank 1's flag.  With the limit at ~50 ms the kernel gives up, records (code 2, rank, missing rank,
    epoch) and returns; the next layer call is correct."""
    from fused_moe_b200 import _lib
    flags = torch.zeros((2, 64), dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    peers = _lib.EpPeers()
    peers.world, peers.rank = 2, 0
    peers.flags[0], peers.flags[1] = flags[0].data_ptr(), flags[1].data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.b200moe_set_wait_limit_cycles(100_000_000) == 0      # about 50 ms at B200 clocks
    try:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        _lib.check(lib.b200moe_ep_barrier(C.byref(peers), 7, status.data_ptr(), stream), "b200moe_ep_barrier")
        t1.record()
        torch.cuda.synchronize()
    finally:
        assert lib.b200moe_set_wait_limit_cycles(0) == 0            # back to the default
    assert status.cpu().tolist() == [2, 0, 1, 7]
    assert 5.0 < t0.elapsed_time(t1) < 2000.0                       # it waited for about the limit, not for seconds
    assert flags[0].cpu().tolist()[:2] == [7, 0] and flags[1].cpu().tolist()[0] == 7   # its own arrival was published
    assert lib.b200moe_set_wait_limit_cycles(-1) == _lib.EINVAL
    _layer_still_correct(oracle, seed=3)


def test_count_exchange_refuses_counts_that_do_not_fit(lib):
    """One rank, local buffers: 10 records announced but the receive buffer holds 8 -> status code 3, plan.ok = 0 and
    every count zero, so the kernels that follow store nothing."""
    from fused_moe_b200 import _lib
    hdr = torch.zeros(256, dtype=torch.int32, device="cuda")
    back = torch.zeros(16, dtype=torch.float32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    plan = torch.full((512,), 0xEE, dtype=torch.uint8, device="cuda")
    counts = torch.tensor([10], dtype=torch.int32, device="cuda")
    peers = _lib.EpPeers()
    peers.world, peers.rank, peers.cap_recv, peers.cap_back = 1, 0, 8, 64
    peers.flags[0], peers.counts[0], peers.back_rows[0] = hdr.data_ptr(), hdr[64:].data_ptr(), back.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.b200moe_ep_exchange_counts(C.byref(peers), counts.data_ptr(), 1, plan.data_ptr(),
                                              status.data_ptr(), stream), "b200moe_ep_exchange_counts")
    torch.cuda.synchronize()
    pl = _lib.EpPlan.from_buffer_copy(bytes(plan.cpu().numpy().tobytes())[:C.sizeof(_lib.EpPlan)])
    assert status.cpu().tolist() == [3, 0, 8, 64]
    assert (pl.ok, pl.n_recv, pl.n_send, pl.matrix[0]) == (0, 0, 0, 0)
    # the same counts with room for them
    status.zero_()
    peers.cap_recv = 16
    _lib.check(lib.b200moe_ep_exchange_counts(C.byref(peers), counts.data_ptr(), 2, plan.data_ptr(),
                                              status.data_ptr(), stream), "b200moe_ep_exchange_counts")
    torch.cuda.synchronize()
    pl = _lib.EpPlan.from_buffer_copy(bytes(plan.cpu().numpy().tobytes())[:C.sizeof(_lib.EpPlan)])
    assert status.cpu().tolist() == [0, 0, 0, 0]
    assert (pl.ok, pl.n_recv, pl.n_send, pl.seg_count, pl.seg_start[0], pl.seg_start[1]) == (1, 10, 10, 1, 0, 10)
    assert pl.seg_base[0] == back.data_ptr() and pl.dst_row0[0] == 0


def test_failed_call_is_reported_by_the_next_call_without_a_sync(oracle):
    """kernel() never synchronises, so a call whose device status word is non-zero is reported by a LATER call: the
    last kernel of every layer call copies a non-zero status into pinned host memory, which kernel() looks at on entry.
    The failure is staged by writing the status word from the host (no kernel is made to fail)."""
    from fused_moe_b200 import kernel as K, synth
    inp = synth.make_inputs(40, 8, seed=8, local_expert_offset=96, skew=True, device="cuda")
    good = K.kernel(**inp).clone()
    K.check_status()
    ws = K.last_workspace()
    ws.view("status", torch.int32, (4,)).copy_(torch.tensor([1, 17, 3, 9], dtype=torch.int32))
    K.kernel(**inp)                      # runs; its last kernel publishes the status word
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match=r"code=1 block=17 role=3 detail=9"):
        K.kernel(**inp)
    out = K.kernel(**inp)                # the workspace is re-initialised: the library works again
    K.check_status()
    assert torch.equal(out, good)
    _layer_still_correct(oracle, seed=8)
