"""GPU: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded inputs.

Integer results (expert ids, permutation, offsets) must be bit-exact; the bf16 output must satisfy
|x - y| <= 1e-2 + 2e-2 |y| against the fp32-dequant oracle (tests/conftest.py: ATOL, RTOL).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import assert_close, assert_close_rowscaled, golden_names, load_golden, matched_ratio

pytestmark = pytest.mark.gpu

KEYS = ["routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
        "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset", "routed_scaling_factor"]


@pytest.fixture(scope="module")
def moe():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fused_moe_b200 import kernel as k
    from fused_moe_b200 import _lib
    _lib.load()  # raises if libb200moe.so is missing: there is no fallback to test
    return k


_weights_cache = {}


def gpu_inputs(T, E_local, seed, offset, skew, heavy=False):
    from fused_moe_b200 import synth
    key = (E_local, seed, offset)
    w = _weights_cache.get(key)
    if w is None:
        _weights_cache.clear()
    inp = synth.make_inputs(T, E_local, seed=seed, local_expert_offset=offset, skew=skew, device="cuda", weights=w,
                            heavy_tail=heavy)
    _weights_cache[key] = inp
    return inp


def poison_workspace(moe, T, E_local):
    """Fill the scratch buffer with 0xFF so that reads of rows the kernels never wrote show up as NaN / nonsense."""
    from fused_moe_b200.kernel import _devices, workspace_bytes
    st = _devices.get(torch.cuda.current_device())
    if st is not None and st.buffer is not None:
        st.buffer.fill_(0xFF)
        st.active = None


def run_and_check(moe, oracle, T, E_local, seed, offset, skew, poison=True):
    inp = gpu_inputs(T, E_local, seed, offset, skew)
    if poison:
        moe.kernel(**inp)  # sizes the buffer
        torch.cuda.synchronize()
        poison_workspace(moe, T, E_local)
    out = moe.kernel(**inp)
    moe.check_status()
    ws = moe.last_workspace()
    assert out.shape == (T, 7168) and out.dtype == torch.bfloat16
    ref = oracle.kernel(*[inp[k] for k in KEYS])

    # routing: bit-exact ids (order included) and weights
    idx = ws.view("topk_idx", torch.int32, (T, 8)).cpu()
    w = ws.view("topk_w", torch.float32, (T, 8)).cpu()
    assert torch.equal(idx, ref["topk_idx"]), "expert ids differ from the oracle"
    assert torch.equal(w, ref["topk_w"]), "routing weights differ from the oracle"

    # sort metadata: bit-exact, as the forward call left it (for 2 < T <= 32 that is the fused single-launch prologue,
    # above it the separate sort kernels).  The decode path (few expected pairs) does not sort, so the stage is run here
    # explicitly.
    from fused_moe_b200._lib import uses_decode_path
    if uses_decode_path(T, E_local):
        from fused_moe_b200 import _lib
        from fused_moe_b200.kernel import _problem
        p = _problem(T, E_local, offset, float(inp["routed_scaling_factor"]), inp["routing_logits"],
                     inp["routing_bias"], inp["hidden_states"], inp["hidden_states_scale"], inp["gemm1_weights"],
                     inp["gemm1_weights_scale"], inp["gemm2_weights"], inp["gemm2_weights_scale"], out)
        _lib.check(_lib.load().b200moe_sort(C.byref(p), C.byref(ws.struct), torch.cuda.current_stream().cuda_stream),
                   "sort")
        torch.cuda.synchronize()
    s = oracle.sort(ref["topk_idx"], ref["topk_w"], E_local, offset)
    tb = int(ws.view("total_blocks", torch.int32, (1,)).item())
    assert tb == s["total_blocks"]
    assert torch.equal(ws.view("counts", torch.int32, (E_local,)).cpu(), s["counts"])
    assert torch.equal(ws.view("block_offsets", torch.int32, (E_local + 1,)).cpu(), s["block_offsets"])
    n = tb * 128
    assert torch.equal(ws.view("sorted_token_ids", torch.int32, (ws.struct.R_max,))[:n].cpu(), s["sorted_token_ids"])
    assert torch.equal(ws.view("sorted_weights", torch.float32, (ws.struct.R_max,))[:n].cpu(), s["sorted_weights"])
    assert torch.equal(ws.view("scatter_map", torch.int32, (T, 8)).cpu(), s["scatter_map"])

    ratio = assert_close(out.float().cpu(), ref["out_bf16"].float(), what=f"T={T} E={E_local} off={offset}")
    return out, ref, ratio


@pytest.mark.parametrize("T,E_local,seed,offset,skew", [
    (7, 32, 0, 0, False),      # the reference's CPU-runnable configuration
    (1, 32, 5, 96, False),     # decode path (matrix-vector kernels)
    (2, 32, 9, 0, False),      # decode path, two tokens
    (4, 32, 14, 0, True),      # last batch size on the decode path for 32 local experts, skewed: shared experts
    (5, 32, 14, 0, True),      # first batch size past it
    (8, 16, 14, 32, True),     # decode path at its token limit (16 local experts)
    (9, 8, 14, 32, True),      # nine tokens: never the decode path
    (1, 256, 15, 0, False),    # all experts local, one token (eight pairs): fused prologue + token-minor GEMMs
    (1, 128, 15, 64, False),   # 128 local experts: decode path for one token only
    (80, 32, 1, 0, False),     # small batch
    (33, 8, 3, 60, False),     # E_local below one warp, non-zero offset, two token chunks
    (40, 3, 13, 253, True),    # last experts, skewed router
    (3, 2, 21, 100, False),    # no token reaches a local expert: all-zero output
    (300, 32, 4, 64, True),    # an expert with more than one 128-row block
    (12, 256, 6, 0, True),     # all 256 experts local: every token sums eight expert rows
    (32, 32, 7, 32, False),    # largest batch of the fused prologue: one full token chunk
    (31, 256, 8, 0, True),     # fused prologue, ragged chunk, every pair local (248 gathered rows)
    (33, 32, 7, 32, False),    # first batch size on the separate route / sort / gather kernels
    (112, 32, 10, 0, True),    # largest batch on the token-minor GEMMs, experts with more than one 64-row sub-block
    (113, 32, 10, 0, True),    # first batch size on the 128-token-tile GEMMs
    (256, 32, 10, 0, True),    # eight full token chunks
    (1000, 32, 11, 0, True),   # 32 token chunks, ragged; experts with several 128-row blocks
    (1025, 8, 11, 40, False),  # one token into the 33rd chunk
])
def test_layer_matches_oracle(moe, oracle, T, E_local, seed, offset, skew):
    out, ref, _ = run_and_check(moe, oracle, T, E_local, seed, offset, skew)
    if ref["pairs"] == 0:
        assert not out.any()


@pytest.mark.parametrize("name", golden_names(full=True))
def test_layer_matches_reference_golden(moe, name):
    """Straight against the reference's own outputs (tests/golden, made by solution/cuda/binding.py)."""
    g = load_golden(name)
    inp = gpu_inputs(g["T"], g["E_local"], g["seed"], g["offset"], g["skew"], g["heavy"])
    out = moe.kernel(**inp)
    moe.check_status()
    ws = moe.last_workspace()
    idx = ws.view("topk_idx", torch.int32, (g["T"], 8)).cpu().long()
    assert np.array_equal(idx.sort(dim=1).values.numpy(), g["topk_idx"])
    ref = torch.from_numpy(g["out_f32"]).bfloat16().float()
    if g["heavy"]:
        # Heavy-tailed activations (rows from 1e-2 to 3e4, elements that cancel to ~0): an element-wise 1e-2 + 2e-2 |y|
        # cannot hold for any FP8 product there.  Checked instead: the contest's own criterion for real traces, and an
        # error bound relative to each row's largest value, which is what the two-term FP8 intermediate must deliver.
        assert matched_ratio(out.float().cpu(), ref) >= 0.999
        assert_close_rowscaled(out.float().cpu(), ref, rel=1e-2, what=name)
        return
    assert_close(out.float().cpu(), ref, what=name)


def test_routing_large_skewed(moe, oracle):
    """Routing + sort alone at prefill size: bit-exact against the oracle, sets equal to the reference's torch code."""
    from fused_moe_b200 import _lib, synth
    from fused_moe_b200.kernel import _problem, _workspace
    g = load_golden("route_t4096_skew")
    T, E_local, off = g["T"], 32, 0
    inp = synth.make_inputs(T, E_local, seed=g["seed"], skew=True, device="cuda", only_experts=[])
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream().cuda_stream
    ws = _workspace(dev, T, E_local, stream)
    out = torch.empty((T, 7168), dtype=torch.bfloat16, device=dev)
    p = _problem(T, E_local, off, 2.5, inp["routing_logits"], inp["routing_bias"], inp["hidden_states"],
                 inp["hidden_states_scale"], inp["gemm1_weights"], inp["gemm1_weights_scale"], inp["gemm2_weights"],
                 inp["gemm2_weights_scale"], out)
    lib = _lib.load()
    _lib.check(lib.b200moe_route(C.byref(p), C.byref(ws.struct), stream), "route")
    _lib.check(lib.b200moe_sort(C.byref(p), C.byref(ws.struct), stream), "sort")
    torch.cuda.synchronize()
    idx = ws.view("topk_idx", torch.int32, (T, 8)).cpu()
    w = ws.view("topk_w", torch.float32, (T, 8)).cpu()
    ridx, rw = oracle.route(inp["routing_logits"], inp["routing_bias"], 2.5)
    assert torch.equal(idx, ridx) and torch.equal(w, rw)
    assert np.array_equal(idx.long().sort(dim=1).values.numpy(), g["topk_idx"])
    s = oracle.sort(ridx, rw, E_local, off)
    n = s["total_blocks"] * 128
    assert torch.equal(ws.view("block_offsets", torch.int32, (E_local + 1,)).cpu(), s["block_offsets"])
    assert torch.equal(ws.view("sorted_token_ids", torch.int32, (ws.struct.R_max,))[:n].cpu(), s["sorted_token_ids"])
    assert torch.equal(ws.view("scatter_map", torch.int32, (T, 8)).cpu(), s["scatter_map"])
    # chunk_bits from topk_idx alone (the expert-parallel receiver's path) equals the fused routing's
    bits = ws.view("chunk_bits", torch.int32, (ws.struct.n_chunks, E_local)).clone()
    ws.view("chunk_bits", torch.int32, (ws.struct.n_chunks, E_local)).fill_(-1)
    p.routing_logits = None
    p.topk_idx_in = ws.struct.topk_idx
    p.topk_w_in = ws.struct.topk_w
    _lib.check(lib.b200moe_topk_bits(C.byref(p), C.byref(ws.struct), stream), "topk_bits")
    torch.cuda.synchronize()
    assert torch.equal(ws.view("chunk_bits", torch.int32, (ws.struct.n_chunks, E_local)), bits)


@pytest.mark.parametrize("T,E_local,seed,offset,skew", [
    (7, 32, 3, 0, False),       # every tile shared by several CTAs (fewer tiles than SMs)
    (150, 32, 3, 0, True),      # experts just above one 64-row sub-block
    (300, 32, 3, 64, True),     # a left-over round with fewer chunk units than CTAs
    (700, 32, 3, 0, True),      # experts with five sub-blocks, whole rounds plus a left-over round
    (40, 3, 3, 253, True),      # one real row
    (64, 256, 3, 0, False),     # all experts local
    (2000, 8, 3, 0, True),      # above the batch size at which b200moe_forward picks these kernels
])
def test_token_minor_gemms_match_tile_gemms(moe, T, E_local, seed, offset, skew):
    """b200moe_gemm1_skinny / b200moe_gemm2_skinny against b200moe_gemm1 / b200moe_gemm2 on the same sorted rows, and
    twice in a row (the tile tickets must be back at zero after a launch).  Tiles one CTA computes alone are bit-equal;
    tiles shared between CTAs add the same fp32 products in another association, hence the small tolerance."""
    from fused_moe_b200 import _lib
    from fused_moe_b200.kernel import _problem
    lib = _lib.load()
    inp = gpu_inputs(T, E_local, seed, offset, skew)
    out = moe.kernel(**inp)
    torch.cuda.synchronize()
    ws = moe.last_workspace()
    R = ws.struct.R_max
    stream = torch.cuda.current_stream().cuda_stream
    p = _problem(T, E_local, offset, float(inp["routed_scaling_factor"]), inp["routing_logits"], inp["routing_bias"],
                 inp["hidden_states"], inp["hidden_states_scale"], inp["gemm1_weights"], inp["gemm1_weights_scale"],
                 inp["gemm2_weights"], inp["gemm2_weights_scale"], out)
    # the sorted rows both GEMM pairs read (the forward call above may have taken the decode path, which does not sort)
    for stage in ("route", "sort", "gather"):
        _lib.check(getattr(lib, "b200moe_" + stage)(C.byref(p), C.byref(ws.struct), stream), stage)
    torch.cuda.synchronize()
    rows = int(ws.view("total_blocks", torch.int32, (1,)).item()) * 128
    real = ws.view("sorted_token_ids", torch.int32, (R,))[:rows] < T

    def run(tag):
        ws.view("inter_q", torch.uint8, (2, R, 2048)).fill_(0x11)
        ws.view("expert_out", torch.float32, (R, 7168)).fill_(7.0)
        _lib.check(getattr(lib, "b200moe_gemm1" + tag)(C.byref(p), C.byref(ws.struct), stream), "gemm1" + tag)
        _lib.check(getattr(lib, "b200moe_gemm2" + tag)(C.byref(p), C.byref(ws.struct), stream), "gemm2" + tag)
        torch.cuda.synchronize()
        moe.check_status()
        return ws.view("expert_out", torch.float32, (R, 7168))[:rows][real].clone()

    ref = run("")
    first = run("_skinny")
    second = run("_skinny")
    assert torch.equal(first, second), "token-minor GEMMs are not repeatable"
    assert int(ws.view("gemm_tile_ctr", torch.int32, (R // 64 * 28,)).abs().sum().item()) == 0
    if ref.numel():
        tol = 5e-4 * float(ref.abs().max())
        assert float((first - ref).abs().max()) <= tol


def test_gemm2_rows_in_half_form(moe, oracle):
    """b200moe_gemm2_half leaves the rows of b200moe_gemm2 in the half form (every value within 2^-11 of itself, rows of
    pad tokens untouched), and b200moe_reduce_half over them gives the bytes of the whole call."""
    from fused_moe_b200 import _lib
    from fused_moe_b200.kernel import _problem
    lib = _lib.load()
    T, E_local = 700, 32
    inp = gpu_inputs(T, E_local, 3, 32, True)
    out = moe.kernel(**inp).clone()
    torch.cuda.synchronize()
    ws = moe.last_workspace()
    R = ws.struct.R_max
    stream = torch.cuda.current_stream().cuda_stream
    again = torch.empty_like(out)
    p = _problem(T, E_local, 32, float(inp["routed_scaling_factor"]), inp["routing_logits"], inp["routing_bias"],
                 inp["hidden_states"], inp["hidden_states_scale"], inp["gemm1_weights"], inp["gemm1_weights_scale"],
                 inp["gemm2_weights"], inp["gemm2_weights_scale"], again)
    rows = int(ws.view("total_blocks", torch.int32, (1,)).item()) * 128
    real = ws.view("sorted_token_ids", torch.int32, (R,))[:rows] < T
    _lib.check(lib.b200moe_gemm2(C.byref(p), C.byref(ws.struct), stream), "gemm2")
    torch.cuda.synchronize()
    full = ws.view("expert_out", torch.float32, (R, 7168))[:rows].clone()
    ws.view("expert_out", torch.uint8, (R * 7168 * 4,)).fill_(0x5A)
    _lib.check(lib.b200moe_gemm2_half(C.byref(p), C.byref(ws.struct), stream), "gemm2_half")
    torch.cuda.synchronize()
    half = ws.view("expert_out", torch.uint8, (R * 7168 * 4,))[:rows * 15232].view(rows, 15232).clone()
    assert np.array_equal(half[real].cpu().numpy(), oracle.encode_half_rows(full[real].cpu().numpy()))
    dec = decode_half_rows(half[real])
    f3 = full[real].view(-1, 896, 8)
    gmax = f3.abs().amax(dim=2, keepdim=True)
    assert ((dec.view(-1, 896, 8) - f3).abs() <= f3.abs() * 2.0 ** -11 + gmax * 2.0 ** -39).all()
    assert (half[~real] == 0x5A).all()          # rows of pad tokens are not written
    _lib.check(lib.b200moe_reduce_half(C.byref(p), C.byref(ws.struct), stream), "reduce_half")
    torch.cuda.synchronize()
    moe.check_status()
    assert torch.equal(again, out)


def test_from_topk_equals_routed(moe):
    """kernel_from_topk with the routing's own (ids, weights) reproduces kernel() bit for bit."""
    inp = gpu_inputs(80, 32, 1, 0, False)
    out = moe.kernel(**inp).clone()
    ws = moe.last_workspace()
    idx = ws.view("topk_idx", torch.int32, (80, 8)).clone()
    w = ws.view("topk_w", torch.float32, (80, 8)).clone()
    out2 = moe.kernel_from_topk(idx, w, inp["hidden_states"], inp["hidden_states_scale"], inp["gemm1_weights"],
                                inp["gemm1_weights_scale"], inp["gemm2_weights"], inp["gemm2_weights_scale"], 0)
    moe.check_status()
    assert torch.equal(out, out2)


def test_destination_passing_and_scalar_tensors(moe):
    """output= is filled and returned; 0-d device tensors are accepted for the two scalars
    (reference: solution/python/pure_triton_impl.py:2012-2020, scripts/diag_precision_modal.py:106-107)."""
    inp = gpu_inputs(7, 32, 0, 0, False)
    ref = moe.kernel(**inp).clone()
    dst = torch.full((7, 7168), 3.0, dtype=torch.bfloat16, device="cuda")
    args = dict(inp)
    args["local_expert_offset"] = torch.tensor(0, dtype=torch.int32, device="cuda")
    args["routed_scaling_factor"] = torch.tensor(2.5, dtype=torch.float32, device="cuda")
    ret = moe.kernel(*[args[k] for k in KEYS], dst)
    assert ret is dst and torch.equal(dst, ref)


def test_argument_errors(moe):
    inp = gpu_inputs(7, 32, 0, 0, False)
    bad = dict(inp)
    bad["routing_logits"] = inp["routing_logits"].double()
    with pytest.raises(TypeError):
        moe.kernel(**bad)
    bad = dict(inp)
    bad["hidden_states_scale"] = inp["hidden_states_scale"].t().contiguous()
    with pytest.raises(ValueError):
        moe.kernel(**bad)
    bad = dict(inp)
    bad["local_expert_offset"] = 250
    with pytest.raises(ValueError):
        moe.kernel(**bad)
    bad = dict(inp)
    bad["hidden_states"] = inp["hidden_states"].cpu()
    with pytest.raises(RuntimeError):
        moe.kernel(**bad)


def test_empty_batch(moe):
    inp = gpu_inputs(7, 32, 0, 0, False)
    z = dict(inp)
    z["routing_logits"] = inp["routing_logits"][:0]
    z["hidden_states"] = inp["hidden_states"][:0]
    z["hidden_states_scale"] = inp["hidden_states_scale"][:, :0].contiguous()
    out = moe.kernel(**z)
    assert out.shape == (0, 7168)


def _world1_weights(inp):
    """A world-1 shard owns all 256 experts: the 32 generated experts at their global position, zeros elsewhere."""
    E = 256
    w13 = torch.zeros((E, 4096, 7168), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    w13s = torch.zeros((E, 32, 56), dtype=torch.float32, device="cuda")
    w2 = torch.zeros((E, 7168, 2048), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    w2s = torch.zeros((E, 56, 16), dtype=torch.float32, device="cuda")
    w13[64:96], w13s[64:96], w2[64:96], w2s[64:96] = (inp["gemm1_weights"], inp["gemm1_weights_scale"],
                                                      inp["gemm2_weights"], inp["gemm2_weights_scale"])
    return dict(gemm1_weights=w13, gemm1_weights_scale=w13s, gemm2_weights=w2, gemm2_weights_scale=w2s)


def test_expert_parallel_half_rows_world1(moe):
    """Partial rows in the half form through both transports with one rank: the two transports give the same bits (same
    kernels encode and decode), and the result is kernel()'s within the layer's tolerance — a token's row passes
    through float16 with 11 significant bits once before the final bfloat16 rounding."""
    from fused_moe_b200 import ep, synth
    inp = gpu_inputs(300, 32, 4, 64, True)
    wts = _world1_weights(inp)
    _half_rows_world1(moe, ep, synth, inp, wts, 512, ((300, 4), (150, 9), (412, 12)))
    # more than 512 rows: the reduce and the combine then take four groups per thread (one token per CTA)
    _half_rows_world1(moe, ep, synth, inp, wts, 2048, ((1200, 5), (700, 6)))


def _half_rows_world1(moe, ep, synth, inp, wts, capacity, batches):
    shards = {t: ep.make_cuda_shard(wts, rank=0, world=1, transport=t, max_tokens_per_rank=capacity, partial_rows="half")
              for t in ("nccl", "peer")}
    # batches above the token-minor GEMM limit, where the shard's 256-expert layer adds in kernel()'s order
    for T, seed in batches:
        cur = synth.make_inputs(T, 32, seed=seed, local_expert_offset=64, skew=True, device="cuda", weights=inp)
        want = moe.kernel(**cur).float()
        got = {}
        for t, shard in shards.items():
            if t == "peer" and shard._peer is not None:
                shard._peer["slab"][shard._peer["off_back"]:].fill_(0xFF)     # stale bytes in the return buffer
            got[t] = shard.forward(cur["routing_logits"], cur["routing_bias"], cur["hidden_states"],
                                   cur["hidden_states_scale"], cur["routed_scaling_factor"]).clone()
            moe.check_status()
            shard.check_status()
        assert torch.equal(got["nccl"], got["peer"]), f"T={T}"
        err = (got["peer"].float() - want).abs()
        assert (err <= 1e-2 + 2e-2 * want.abs()).all(), f"T={T}"
        # one extra rounding at 2^-11 of the value, then bfloat16: at most one bfloat16 step from kernel() (values
        # below 2^-28 of their group's maximum lose bits: they only matter at the absolute level)
        bad = err > want.abs() * 2.0 ** -7 + 1e-6
        assert not bad.any(), (f"T={T}: {int(bad.sum())} values, e.g. got {got['peer'].float()[bad][:4].tolist()} "
                               f"want {want[bad][:4].tolist()}")
        assert (got["peer"].float() != want).float().mean().item() < 0.2


@pytest.mark.parametrize("transport", ["nccl", "peer"])
def test_expert_parallel_shard_world1(moe, transport):
    """The expert-parallel plumbing with one rank reproduces kernel() bit for bit.  "nccl": dispatch and combine are
    local copies.  "peer": the whole device-side protocol on a local slab — count exchange and plan on the device,
    records packed into the receive buffer, the layer over a receive buffer LARGER than what arrived (capacity 512
    tokens; the rows beyond the count are poisoned and, on the later calls, hold the previous call's records), partial
    rows placed through the plan, combine.  Three calls with different batches share the buffers."""
    from fused_moe_b200 import ep, synth
    inp = gpu_inputs(300, 32, 4, 64, True)
    shard = ep.make_cuda_shard(_world1_weights(inp), rank=0, world=1, transport=transport, max_tokens_per_rank=512)
    # batches above the token-minor GEMM limit: the 128-row tile kernels give the same bits whatever the expert count
    for T, seed in ((300, 4), (150, 11), (412, 12)):
        cur = synth.make_inputs(T, 32, seed=seed, local_expert_offset=64, skew=(seed != 11), device="cuda", weights=inp)
        want = moe.kernel(**cur).clone()
        if transport == "peer" and shard._peer is not None:
            shard._peer["recv"][T:].fill_(0xFF)     # stale / poisoned rows past the received count must select nothing
        got = shard.forward(cur["routing_logits"], cur["routing_bias"], cur["hidden_states"],
                            cur["hidden_states_scale"], cur["routed_scaling_factor"])
        moe.check_status()
        shard.check_status()
        # experts outside 64..95 have zero weights and add nothing: same sums, same single rounding
        assert torch.equal(got, want), f"T={T}"
        send, recv = shard.last_splits
        assert send == [T] and recv == [T] and shard.last_records.shape == (T, 7456)
    # the same (last) batch from pinned host memory, two runs pipelined over the copy streams: identical rows
    host = {k: cur[k].cpu().pin_memory() for k in ("routing_logits", "hidden_states", "hidden_states_scale")}
    out_h = shard.forward_host(host["routing_logits"], cur["routing_bias"], host["hidden_states"],
                               host["hidden_states_scale"], cur["routed_scaling_factor"], slices=2)
    torch.cuda.synchronize()
    shard.check_status()
    assert out_h.is_pinned() and torch.equal(out_h, want.cpu())
    # and three calls queued back to back, each with its own event instead of a wait on the caller's stream
    outs = [torch.empty((412, 7168), dtype=torch.bfloat16).pin_memory().fill_(3.0) for _ in range(3)]
    evs = [torch.cuda.Event() for _ in outs]
    for o, ev, sl in zip(outs, evs, (1, 2, 1)):
        shard.forward_host(host["routing_logits"], cur["routing_bias"], host["hidden_states"],
                           host["hidden_states_scale"], cur["routed_scaling_factor"], o, slices=sl, ready_event=ev)
    for o, ev in zip(outs, evs):
        ev.synchronize()
        assert torch.equal(o, want.cpu())
    torch.cuda.synchronize()
    shard.check_status()
    shard.forward_host(host["routing_logits"], cur["routing_bias"], host["hidden_states"],
                       host["hidden_states_scale"], cur["routed_scaling_factor"], slices=2)
    torch.cuda.synchronize()
    if transport == "peer":
        # a receive buffer of more than 32 chunks of 32 rows: the sort then runs its separate scan kernel, and both it and
        # the scatter must ignore the rows past the received count
        big = ep.make_cuda_shard(shard.weights, rank=0, world=1, transport="peer", max_tokens_per_rank=2048)
        cur = synth.make_inputs(1200, 32, seed=21, local_expert_offset=64, skew=True, device="cuda", weights=inp)
        want = moe.kernel(**cur).clone()
        for _ in range(2):
            big._peer_setup(1200, torch.device("cuda", torch.cuda.current_device()))
            big._peer["recv"][1200:].fill_(0xFF)
            got = big.forward(cur["routing_logits"], cur["routing_bias"], cur["hidden_states"],
                              cur["hidden_states_scale"], cur["routed_scaling_factor"])
            moe.check_status()
            big.check_status()
            assert torch.equal(got, want)
        pl = shard.read_plan()
        # the shard's last step was the second run of forward_host: 206 of the 412 tokens
        assert pl.ok == 1 and pl.n_recv == 206 and pl.n_send == 206 and pl.seg_start[1] == 206 and pl.dst_row0[0] == 0
        with pytest.raises(ValueError):             # beyond the capacity agreed at the first call
            big = synth.make_inputs(513, 32, seed=1, local_expert_offset=64, device="cuda", weights=inp)
            shard.forward(big["routing_logits"], big["routing_bias"], big["hidden_states"], big["hidden_states_scale"],
                          big["routed_scaling_factor"])


def test_synth_cpu_and_cuda_generate_identical_bytes(moe):
    """The golden fixtures were generated on a CPU; the GPU tests regenerate their inputs on the device."""
    from fused_moe_b200 import synth
    a = synth.make_inputs(5, 2, seed=9, local_expert_offset=10, skew=True, only_experts=[1], device="cpu")
    b = synth.make_inputs(5, 2, seed=9, local_expert_offset=10, skew=True, only_experts=[1], device="cuda")
    for k, v in a.items():
        if torch.is_tensor(v):
            x = v.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else v
            y = b[k].cpu()
            y = y.view(torch.uint8) if y.dtype == torch.float8_e4m3fn else y
            assert torch.equal(x, y), k


@pytest.mark.parametrize("T,heavy", [(1, False), (33, True), (1000, False)])
def test_quantize_activations_matches_oracle(moe, oracle, T, heavy):
    """b200moe_quantize_act against the CPU restatement of its specification (oracle/quant.c: s = max(amax/448, 1e-12),
    q = e4m3(x * (1/s))): identical bytes and scales, including an all-zero row (scale clamps to 1e-12, codes 0) and
    heavy-tailed rows.  Against the input generator, which divides instead (x / s), the scales are still identical and
    a code may differ by one step where the two roundings straddle a boundary of e4m3."""
    from fused_moe_b200 import synth
    x = synth.normal(T * 7168, 77, 1, device="cuda").view(T, 7168)
    if heavy:
        x = x * torch.exp(2.3 * synth.normal(T, 77, 7, device="cuda").clamp(-2, 2)).view(T, 1)
        x[T // 2].zero_()
    xb = x.bfloat16()
    q, s = moe.quantize_activations(xb)
    torch.cuda.synchronize()
    q_ref, s_ref = oracle.quantize_act(xb)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.view(torch.uint8).cpu(), q_ref.view(torch.uint8))      # bytes: exact
    q_gen, s_gen = synth.quantize_act(xb.float())
    assert torch.equal(s, s_gen)
    differs = q.view(torch.uint8) != q_gen.view(torch.uint8)
    assert differs.float().mean().item() < 1e-3
    assert ((q.float() - q_gen.float()).abs() <= 0.125 * q_gen.float().abs() + 2.0 ** -9)[differs].all()
    with pytest.raises(TypeError):
        moe.quantize_activations(x)           # float32 input
    with pytest.raises(ValueError):
        moe.quantize_activations(xb[:, :128])  # wrong width


@pytest.mark.parametrize("T,slices", [(8192, None), (9001, 4), (300, None)])
def test_host_memory_entry_point_equals_device_call(moe, T, slices):
    """kernel_host (pinned host activations, copies pipelined over token slices) gives the bytes of kernel()."""
    inp = gpu_inputs(T, 32, 0, 0, True)
    want = moe.kernel(**inp).cpu()
    host = {k: inp[k].cpu().pin_memory() for k in ("routing_logits", "hidden_states", "hidden_states_scale")}
    args = dict(inp)
    args.update(host)
    got = moe.kernel_host(**args, slices=slices)
    again = torch.empty((T, 7168), dtype=torch.bfloat16).pin_memory()
    assert moe.kernel_host(**args, output=again, slices=slices) is again    # back to back on the same staging buffers
    torch.cuda.synchronize()
    moe.check_status()
    assert got.is_pinned() and torch.equal(got, want) and torch.equal(again, want)
    with pytest.raises(RuntimeError):
        moe.kernel_host(**inp)    # device activations


def decode_half_rows(rows: torch.Tensor) -> torch.Tensor:
    """uint8 [n, 15232] in the half form of b200moe_problem.partial_format -> float32 [n, 7168]."""
    n = rows.shape[0]
    halves = rows[:, :14336].contiguous().view(torch.float16).view(n, 896, 8).float()
    scale = torch.pow(2.0, rows[:, 14336:].to(torch.float32) - 141.0)
    return (halves * scale.view(n, 896, 1)).view(n, 7168)


@pytest.mark.parametrize("T", [40, 700])
def test_half_partial_rows(moe, oracle, T):
    """The half form of the un-rounded rows (eight float16 sharing a power-of-two scale byte): every value within
    2^-11 of ITSELF of the float32 row the same call produces otherwise, all-zero groups stay zero, and the combine
    kernel adds decoded rows in slot order with one rounding."""
    from fused_moe_b200 import _lib, ep
    inp = gpu_inputs(T, 32, 5, 64, True)
    idx, w = moe.route(inp["routing_logits"], inp["routing_bias"], inp["routed_scaling_factor"])
    recs = ep.pack_rows(torch.arange(T, device="cuda"), inp["hidden_states"], inp["hidden_states_scale"], idx, w)
    args = [inp[k] for k in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale")]
    full = moe.kernel_from_records(recs, *args, 64)
    half = moe.kernel_from_records(recs, *args, 64, half_rows=True)
    moe.check_status()
    assert half.dtype == torch.uint8 and tuple(half.shape) == (T, 15232)
    # byte for byte the CPU restatement of the format applied to the float32 rows
    assert np.array_equal(half.cpu().numpy(), oracle.encode_half_rows(full.cpu().numpy()))
    dec = decode_half_rows(half)
    gmax = full.view(T, 896, 8).abs().amax(dim=2, keepdim=True)
    # float16 keeps its own exponent per value: 11 significant bits of every value down to 2^-28 of the group maximum
    f3 = full.view(T, 896, 8)
    assert ((dec.view(T, 896, 8) - f3).abs() <= f3.abs() * 2.0 ** -11 + gmax * 2.0 ** -39).all()
    zero_groups = gmax.squeeze(2) == 0
    assert (half[:, 14336:][zero_groups] == 14).all() and (dec.view(T, 896, 8)[zero_groups] == 0).all()
    nz = ~zero_groups
    exp_of_max = torch.frexp(gmax.squeeze(2)[nz])[1] - 1 + 127          # biased exponent of the group maximum
    assert torch.equal(half[:, 14336:][nz].to(torch.int32), exp_of_max.to(torch.int32))
    # combine: token t adds rows t, (t + 3) % T and one missing slot
    slot = torch.full((T, 8), -1, dtype=torch.int32, device="cuda")
    slot[:, 0] = torch.arange(T, device="cuda")
    slot[:, 5] = (torch.arange(T, device="cuda") + 3) % T
    out = torch.empty((T, 7168), dtype=torch.bfloat16, device="cuda")
    lib = _lib.load()
    _lib.check(lib.b200moe_ep_combine_half(half.data_ptr(), slot.data_ptr(), T, out.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream), "b200moe_ep_combine_half")
    want = (dec + dec[(torch.arange(T, device="cuda") + 3) % T]).bfloat16()
    assert torch.equal(out, want)


def test_host_memory_calls_overlap_with_ready_events(moe):
    """kernel_host with ready_event: five batches of different sizes and contents are queued back to back without any
    wait in between (copy-in of one under the layer of the previous, copy-out under the next); each output, read after
    its own event, has the bytes of kernel() on that batch."""
    from fused_moe_b200 import synth
    base = gpu_inputs(1500, 32, 0, 0, True)
    batches = []
    for i, (T, seed, slices) in enumerate(((1500, 3, None), (700, 4, 2), (1500, 5, None), (64, 6, None), (1300, 7, 3))):
        cur = synth.make_inputs(T, 32, seed=seed, local_expert_offset=0, skew=bool(i & 1), device="cuda", weights=base)
        want = moe.kernel(**cur).cpu()
        args = dict(cur)
        args.update({k: cur[k].cpu().pin_memory() for k in ("routing_logits", "hidden_states", "hidden_states_scale")})
        batches.append((args, want, slices, torch.empty((T, 7168), dtype=torch.bfloat16).pin_memory().fill_(7.0)))
    torch.cuda.synchronize()
    events = [torch.cuda.Event() for _ in batches]
    for (args, _, slices, out), ev in zip(batches, events):
        assert moe.kernel_host(**args, output=out, slices=slices, ready_event=ev) is out
    for (args, want, _, out), ev in zip(batches, events):
        ev.synchronize()
        assert torch.equal(out, want)
    torch.cuda.synchronize()
    moe.check_status()
    # an empty batch records the event at once
    empty = {k: (v[:0] if k in ("routing_logits", "hidden_states") else v) for k, v in batches[0][0].items()}
    empty["hidden_states_scale"] = torch.empty((56, 0), dtype=torch.float32).pin_memory()
    empty["routing_logits"] = torch.empty((0, 256), dtype=torch.float32).pin_memory()
    empty["hidden_states"] = torch.empty((0, 7168), dtype=torch.float8_e4m3fn).pin_memory()
    ev = torch.cuda.Event()
    assert moe.kernel_host(**empty, ready_event=ev).shape == (0, 7168)
    ev.synchronize()


def test_interleaved_batch_sizes_share_one_workspace(moe):
    """Calls of different batch sizes alternate on one device (one shared scratch buffer, re-carved per size; every
    dispatch class of b200moe_forward; tile tickets that must be back at zero): each repeats its first result bit for
    bit, without any synchronisation between the calls."""
    sizes = [1, 7, 9, 16, 33, 80, 112, 256, 300, 1000]
    inputs = {T: gpu_inputs(T, 32, 0, 0, True) for T in sizes}
    first = {T: moe.kernel(**inputs[T]).clone() for T in sizes}
    torch.cuda.synchronize()
    order = torch.randint(0, len(sizes), (40,), generator=torch.Generator().manual_seed(3)).tolist()
    outs = [(sizes[i], moe.kernel(**inputs[sizes[i]]).clone()) for i in order]
    torch.cuda.synchronize()
    moe.check_status()
    for T, out in outs:
        assert torch.equal(out, first[T]), f"T={T} changed between calls"
