"""GPU, the prefill sizes of the benchmark configurations (T = 4096 and 16384, 32 local experts, skewed router; and the bench's headline
configuration, T = 16384 with all 256 experts local): the oracle cannot run the
whole layer at these sizes in seconds, so parity is checked through size-independent properties —
  * routing and the complete sort metadata bit-exact against the oracle (both are cheap on the CPU);
  * a random sample of token rows against the oracle run on just those tokens (routing and experts are per token);
  * permutation: shuffling the tokens shuffles the output rows bit for bit (a row's result does not depend on which
    128-row tile or position it lands in);
  * scaling: doubling routed_scaling_factor doubles every output element exactly;
  * sharding: the outputs of the two 16-expert halves of the shard, run separately, add up to the 32-expert output.
"""
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu

KEYS = ["routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
        "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset", "routed_scaling_factor"]


@pytest.fixture(scope="module")
def setup():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fused_moe_b200 import kernel as K, synth
    inp = synth.make_inputs(16384, 32, seed=0, skew=True, device="cuda")
    return K, inp


def _slice(inp, sel):
    out = dict(inp)
    out["routing_logits"] = inp["routing_logits"][sel].contiguous()
    out["hidden_states"] = inp["hidden_states"][sel].contiguous()
    out["hidden_states_scale"] = inp["hidden_states_scale"][:, sel].contiguous()
    return out


@pytest.mark.parametrize("T", [4096, 16384])
def test_metadata_exact_and_sampled_rows(setup, oracle, T):
    K, full = setup
    inp = _slice(full, slice(0, T))
    out = K.kernel(**inp)
    K.check_status()
    ws = K.last_workspace()
    idx = ws.view("topk_idx", torch.int32, (T, 8)).cpu()
    w = ws.view("topk_w", torch.float32, (T, 8)).cpu()
    ridx, rw = oracle.route(inp["routing_logits"], inp["routing_bias"], 2.5)
    assert torch.equal(idx, ridx) and torch.equal(w, rw)
    s = oracle.sort(ridx, rw, 32, 0)
    n = s["total_blocks"] * 128
    assert int(ws.view("total_blocks", torch.int32, (1,)).item()) == s["total_blocks"]
    assert torch.equal(ws.view("counts", torch.int32, (32,)).cpu(), s["counts"])
    assert torch.equal(ws.view("block_offsets", torch.int32, (33,)).cpu(), s["block_offsets"])
    assert torch.equal(ws.view("sorted_token_ids", torch.int32, (ws.struct.R_max,))[:n].cpu(), s["sorted_token_ids"])
    assert torch.equal(ws.view("sorted_weights", torch.float32, (ws.struct.R_max,))[:n].cpu(), s["sorted_weights"])
    assert torch.equal(ws.view("scatter_map", torch.int32, (T, 8)).cpu(), s["scatter_map"])
    assert torch.isfinite(out.float()).all()
    # sampled rows: tokens that do reach local experts, plus a few that may not
    local = ((ridx >= 0) & (ridx < 32)).any(dim=1).nonzero().flatten()
    g = torch.Generator().manual_seed(T)
    pick = torch.cat([local[torch.randperm(local.numel(), generator=g)[:20]],
                      torch.randint(0, T, (4,), generator=g)]).sort().values
    sub = _slice(inp, pick.to("cuda"))
    ref = oracle.kernel(*[sub[k] for k in KEYS])
    assert torch.equal(ref["topk_idx"], ridx[pick])
    assert ref["pairs"] >= 20
    assert_close(out[pick.to("cuda")].float().cpu(), ref["out_bf16"].float(), what=f"sampled rows at T={T}")


def test_permutation_scaling_and_sharding(setup):
    K, full = setup
    T = 16384
    out = K.kernel(**full).clone()
    perm = torch.randperm(T, generator=torch.Generator().manual_seed(1)).to("cuda")
    out_p = K.kernel(**_slice(full, perm))
    assert torch.equal(out_p, out[perm]), "output rows depend on the position of their tokens"
    doubled = dict(full)
    doubled["routed_scaling_factor"] = 2.0 * full["routed_scaling_factor"]
    out_2 = K.kernel(**doubled)
    assert torch.equal(out_2.float(), 2.0 * out.float()), "output is not linear in routed_scaling_factor"
    # two 16-expert shards of the same weights
    parts = []
    for lo in (0, 16):
        shard = dict(full)
        for k in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale"):
            shard[k] = full[k][lo:lo + 16].contiguous()
        shard["local_expert_offset"] = lo
        parts.append(K.kernel(**shard).float())
    K.check_status()
    # each shard rounds to bf16 once more than the joint run: agree to bf16 precision of the parts
    assert_close(parts[0] + parts[1], out.float(), atol=2e-2, rtol=1.6e-2, what="sum of expert shards")
    nonzero_rows = (out.float().abs().sum(dim=1) > 0).sum().item()
    assert nonzero_rows > T // 4


def test_headline_configuration_all_experts_local(oracle):
    """bench.py's N = 1 workload (T = 16384, 256 local experts, N(0,1) router: 131 072 pairs, every token sums eight
    expert rows): metadata bit-exact, and sampled rows against the oracle.  The oracle gets only the experts the
    sampled tokens use, renumbered 0..n-1 (it takes the routing as given through forward_from_topk)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fused_moe_b200 import kernel as K, synth
    T, E = 16384, 256
    inp = synth.make_inputs(T, E, seed=0, skew=False, device="cuda")
    out = K.kernel(**inp)
    K.check_status()
    ws = K.last_workspace()
    idx = ws.view("topk_idx", torch.int32, (T, 8)).cpu()
    w = ws.view("topk_w", torch.float32, (T, 8)).cpu()
    ridx, rw = oracle.route(inp["routing_logits"], inp["routing_bias"], 2.5)
    assert torch.equal(idx, ridx) and torch.equal(w, rw)
    s = oracle.sort(ridx, rw, E, 0)
    n = s["total_blocks"] * 128
    assert int(s["counts"].sum()) == T * 8
    assert int(ws.view("total_blocks", torch.int32, (1,)).item()) == s["total_blocks"]
    assert torch.equal(ws.view("counts", torch.int32, (E,)).cpu(), s["counts"])
    assert torch.equal(ws.view("block_offsets", torch.int32, (E + 1,)).cpu(), s["block_offsets"])
    assert torch.equal(ws.view("sorted_token_ids", torch.int32, (ws.struct.R_max,))[:n].cpu(), s["sorted_token_ids"])
    assert torch.equal(ws.view("scatter_map", torch.int32, (T, 8)).cpu(), s["scatter_map"])
    pick = torch.randint(0, T, (6,), generator=torch.Generator().manual_seed(5)).sort().values
    used = torch.unique(ridx[pick]).tolist()
    renumber = {e: i for i, e in enumerate(used)}
    sub_idx = torch.tensor([[renumber[int(e)] for e in row] for row in ridx[pick]], dtype=torch.int32)
    sel = torch.tensor(used, device="cuda")
    ref32, ref16, pairs = oracle.forward_from_topk(
        sub_idx, rw[pick], inp["hidden_states"][pick.to("cuda")], inp["hidden_states_scale"][:, pick.to("cuda")],
        inp["gemm1_weights"][sel], inp["gemm1_weights_scale"][sel], inp["gemm2_weights"][sel],
        inp["gemm2_weights_scale"][sel], 0)
    assert pairs == 48
    assert_close(out[pick.to("cuda")].float().cpu(), ref16.float(), what="sampled rows, 256 local experts")
