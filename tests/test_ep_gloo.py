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
