"""CPU, world_size 2, gloo: the expert-parallel dispatch / combine plumbing (fused_moe_b200/ep.py).

Routing is the CPU oracle's; the expert path is a cheap stand-in that is linear in the routing weights and depends on
token row, expert id and the receiving rank's expert range, so a wrong destination, a dropped or duplicated row, a
mis-ordered combine or a bad split size all change the result."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle"))

T_GLOBAL = 48
H = 7168


def _dequant(hs, scales):
    n = hs.shape[0]
    return (hs.float().view(n, 56, 128) * scales.t().unsqueeze(2)).reshape(n, H)


def _standin_expert(idx, w, hs, scales, lo, hi):
    local = (idx >= lo) & (idx < hi)
    coeff = (w * (idx.float() + 1.0) * local).sum(dim=1, keepdim=True)
    return coeff * _dequant(hs, scales)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from fused_moe_b200 import ep, synth
        inp = synth.make_inputs(T_GLOBAL, 1, seed=17, skew=True, only_experts=[])
        t_loc = T_GLOBAL // world
        sl = slice(rank * t_loc, (rank + 1) * t_loc)
        e_l = 256 // world

        def route_fn(logits, bias, scale):
            return oracle.route(logits, bias, scale)

        def expert_fn(idx, w, hs, scales):
            return _standin_expert(idx, w, hs, scales, rank * e_l, (rank + 1) * e_l)

        shard = ep.ExpertParallelMoE(route_fn, expert_fn, rank, world)
        out = shard.forward(inp["routing_logits"][sl].contiguous(), inp["routing_bias"],
                            inp["hidden_states"][sl].contiguous(), inp["hidden_states_scale"][:, sl].contiguous(), 2.5)
        # unsharded expectation for this rank's tokens
        idx, w = oracle.route(inp["routing_logits"][sl].contiguous(), inp["routing_bias"], 2.5)
        want = _standin_expert(idx, w, inp["hidden_states"][sl], inp["hidden_states_scale"][:, sl].contiguous(), 0, 256)
        err = (out.float() - want).abs().max().item() / want.abs().max().item()
        plan = shard.last_plan
        dest = (idx.long() // e_l)
        per_rank = [int((dest == d).any(dim=1).sum()) for d in range(world)]
        ok = err < 1e-2 and plan.send_splits == per_rank and sum(plan.send_splits) == plan.send_token.numel()
        # rows sent to one rank are in ascending token order
        off = 0
        for n in plan.send_splits:
            seg = plan.send_token[off:off + n]
            ok = ok and bool((seg[1:] > seg[:-1]).all())
            off += n
        ret[rank] = (ok, err, plan.send_splits, plan.recv_splits)
    finally:
        dist.destroy_process_group()


def test_dispatch_combine_world2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        ok, err, send, recv = ret[r]
        assert ok, f"rank {r}: err={err} send={send} recv={recv}"
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0, and vice versa
    assert ret[0][2][1] == ret[1][3][0] and ret[1][2][0] == ret[0][3][1]


def _faulty_worker(rank, world, port, ret, fault):
    """Host-side failures only (no GPU, nothing is made to hang for longer than the group's timeout):
    "short_send"  rank 1 hands the dispatch all-to-all fewer rows than the split sizes it announced;
    "leaves"      rank 1 completes one step and then leaves the job; rank 0 starts a second step alone.
    The other rank must get an exception from the collective, not a wrong result and not an endless wait."""
    from datetime import timedelta
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=8))
    outcome = "no error"
    try:
        import oracle
        from fused_moe_b200 import ep, synth
        inp = synth.make_inputs(T_GLOBAL, 1, seed=17, skew=True, only_experts=[])
        t_loc = T_GLOBAL // world
        sl = slice(rank * t_loc, (rank + 1) * t_loc)
        e_l = 256 // world
        shard = ep.ExpertParallelMoE(lambda l, b, sc: oracle.route(l, b, sc),
                                     lambda idx, w, hs, scales: _standin_expert(idx, w, hs, scales, rank * e_l,
                                                                                (rank + 1) * e_l), rank, world)
        args = (inp["routing_logits"][sl].contiguous(), inp["routing_bias"], inp["hidden_states"][sl].contiguous(),
                inp["hidden_states_scale"][:, sl].contiguous(), 2.5)
        if fault == "short_send" and rank == 1:
            real_pack = ep.pack_rows
            ep.pack_rows = lambda tokens, *a: real_pack(tokens[:-3], *a)     # three rows short of the announced count
        shard.forward(*args)
        if fault == "leaves":
            if rank == 1:
                outcome = "left"
                return
            shard.forward(*args)          # the peer is gone
    except Exception as exc:               # what the test is about: the failure surfaces as an exception
        outcome = type(exc).__name__
    finally:
        ret[rank] = outcome
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("fault", ["short_send", "leaves"])
def test_host_side_failures_raise_instead_of_hanging(fault):
    world = 2
    ret = mp.Manager().dict()
    port = 29300 + (os.getpid() + (7 if fault == "leaves" else 0)) % 300
    ctx = mp.spawn(_faulty_worker, args=(world, port, ret, fault), nprocs=world, join=False)
    import time
    deadline = time.time() + 120
    while not ctx.join(timeout=5) and time.time() < deadline:     # join() returns once every rank has exited
        pass
    for proc in ctx.processes:
        assert not proc.is_alive(), "a rank is still waiting two minutes after its peer failed"
    assert len(ret) == world
    if fault == "short_send":
        assert any(v not in ("no error", "left") for v in ret.values()), dict(ret)
    else:
        assert ret[1] == "left" and ret[0] not in ("no error", "left"), dict(ret)


def test_pack_unpack_roundtrip():
    from fused_moe_b200 import ep, synth
    inp = synth.make_inputs(9, 1, seed=5, only_experts=[])
    idx = torch.randint(0, 256, (9, 8), dtype=torch.int32)
    w = torch.rand(9, 8)
    tokens = torch.tensor([0, 3, 3, 8])
    buf = ep.pack_rows(tokens, inp["hidden_states"], inp["hidden_states_scale"], idx, w)
    assert buf.shape == (4, ep.ROW_BYTES) and ep.ROW_BYTES % 16 == 0
    hs, scales, idx2, w2 = ep.unpack_rows(buf)
    assert torch.equal(hs.view(torch.uint8), inp["hidden_states"].view(torch.uint8)[tokens])
    assert torch.equal(scales, inp["hidden_states_scale"][:, tokens])
    assert torch.equal(idx2, idx[tokens]) and torch.equal(w2, w[tokens])


def test_world_must_divide_experts():
    from fused_moe_b200 import ep
    with pytest.raises(ValueError):
        ep.ExpertParallelMoE(None, None, 0, 3)
