"""CPU: the oracle (oracle/) against the golden outputs of the reference's own PyTorch path (tests/golden)."""
import numpy as np
import pytest
import torch

from conftest import assert_close, assert_close_rowscaled, golden_names, load_golden
from fused_moe_b200 import synth


def _sorted_by_expert(idx, w):
    order = idx.argsort(dim=1)
    return torch.gather(idx, 1, order), torch.gather(w, 1, order)


@pytest.mark.parametrize("name", golden_names())
def test_routing_matches_reference(oracle, name):
    g = load_golden(name)
    inp = synth.make_inputs(g["T"], g["E_local"], seed=g["seed"], local_expert_offset=g["offset"], skew=g["skew"],
                            only_experts=[], heavy_tail=g["heavy"])
    idx, w = oracle.route(inp["routing_logits"], inp["routing_bias"], inp["routed_scaling_factor"])
    # every token's eight experts are distinct and come in descending biased score, ties to the lower id
    s = torch.sigmoid(inp["routing_logits"]) + inp["routing_bias"].float()
    picked = torch.gather(s, 1, idx.long())
    assert (picked[:, :-1] >= picked[:, 1:] - 1e-6).all()
    sidx, sw = _sorted_by_expert(idx.long(), w)
    assert (sidx[:, 1:] > sidx[:, :-1]).all()
    # the expert SET per token is exactly the reference's (torch.topk leaves the order unspecified)
    assert np.array_equal(sidx.numpy(), g["topk_idx"]), "expert sets differ from the reference"
    np.testing.assert_allclose(sw.numpy(), g["topk_w"], rtol=2e-6, atol=1e-7)
    np.testing.assert_allclose(w.sum(dim=1).numpy(), inp["routed_scaling_factor"], rtol=1e-5)


@pytest.mark.parametrize("name", golden_names(full=True))
def test_forward_matches_reference(oracle, name):
    g = load_golden(name)
    inp = synth.make_inputs(g["T"], g["E_local"], seed=g["seed"], local_expert_offset=g["offset"], skew=g["skew"],
                            only_experts=g["hit_experts"], heavy_tail=g["heavy"])
    res = oracle.kernel(inp["routing_logits"], inp["routing_bias"], inp["hidden_states"], inp["hidden_states_scale"],
                        inp["gemm1_weights"], inp["gemm1_weights_scale"], inp["gemm2_weights"],
                        inp["gemm2_weights_scale"], inp["local_expert_offset"], inp["routed_scaling_factor"])
    ref = torch.from_numpy(g["out_f32"])
    if g["heavy"]:
        # rows up to 3e4 with elements that cancel to ~0: float32 rounding is relative to the row's largest value
        assert_close_rowscaled(res["out_f32"], ref, rel=2e-5, what=f"{name} fp32")
        assert_close_rowscaled(res["out_bf16"].float(), ref.bfloat16().float(), rel=8e-3, what=f"{name} bf16")
        return
    # float32 sums in a different order: agree to float32 rounding, far inside the acceptance bound
    assert_close(res["out_f32"], ref, atol=2e-5, rtol=2e-5, what=f"{name} fp32")
    # and the bf16 rounding is the reference's cast (binding.py:185): equal up to a neighbouring bf16 value
    assert_close(res["out_bf16"].float(), ref.bfloat16().float(), atol=3e-5, rtol=1.6e-2, what=f"{name} bf16")
    if not g["hit_experts"]:
        assert res["pairs"] == 0 and not res["out_f32"].any()


def test_sigmoid_close_to_torch(oracle):
    x = np.concatenate([np.linspace(-30, 30, 4001), [-100.0, 100.0, 0.0, -87.5, 88.5]]).astype(np.float32)
    ours = oracle.sigmoid(x)
    ref = torch.sigmoid(torch.from_numpy(x)).numpy()
    np.testing.assert_allclose(ours, ref, rtol=4e-7, atol=1e-37)


def test_sort_properties(oracle):
    T, E, off = 300, 32, 64
    inp = synth.make_inputs(T, E, seed=4, local_expert_offset=off, skew=True, only_experts=[])
    idx, w = oracle.route(inp["routing_logits"], inp["routing_bias"], 2.5)
    s = oracle.sort(idx, w, E, off)
    counts, offs = s["counts"].numpy(), s["block_offsets"].numpy()
    local = (idx >= off) & (idx < off + E)
    assert counts.sum() == int(local.sum())
    assert np.array_equal(offs[1:] - offs[:-1], (counts + 127) // 128)
    ids, smap = s["sorted_token_ids"].numpy(), s["scatter_map"].numpy()
    assert ((smap >= 0) == local.numpy()).all()
    # stable order = the reference's argsort(stable=True) of the local pair list (binding.py:138-150)
    flat_e = (idx.reshape(-1) - off)[local.reshape(-1)]
    flat_t = torch.arange(T).repeat_interleave(8)[local.reshape(-1)]
    order = flat_e.argsort(stable=True)
    ref_tokens = flat_t[order].numpy()
    got = np.concatenate([ids[offs[e] * 128: offs[e] * 128 + counts[e]] for e in range(E)])
    assert np.array_equal(got, ref_tokens)
    for e in range(E):
        pad = ids[offs[e] * 128 + counts[e]: offs[e + 1] * 128]
        assert (pad == T).all()
    # scatter_map inverts the placement
    for t, k in zip(*np.nonzero(smap >= 0)):
        assert ids[smap[t, k]] == t and s["sorted_weights"][smap[t, k]] == w[t, k]


def test_e4m3_conversion_matches_torch(oracle):
    """Pins oracle/quant.c's float32 -> e4m3 conversion (round to nearest even) against torch's own on the CPU, over the
    whole range the quantiser produces (|x| <= 448) including subnormals, ties and both zeros."""
    torch.manual_seed(0)
    x = torch.cat([torch.randn(100000) * 100, torch.randn(50000) * 0.01, torch.linspace(-448, 448, 50001),
                   torch.tensor([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9, 2.0 ** -6,
                                 0.0146484375, 447.9, 2.5 * 2.0 ** -9, 17.0, 18.0, 19.0, 0.40625])]).float()
    x = x[x.abs() <= 448]
    want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = oracle.f32_to_e4m3(x.numpy())
    assert np.array_equal(want, got)
    assert oracle.f32_to_e4m3(np.array([1e9, -470.0], dtype=np.float32)).tolist() == [0x7E, 0xFE]   # saturating


def test_quantiser_restatement_matches_torch_formula(oracle):
    """oracle.quantize_act against the same specification written with torch ops on the CPU."""
    x = (synth.normal(9 * 7168, 5, 1).view(9, 7168) * torch.exp(2.0 * synth.normal(9, 5, 7)).view(9, 1)).bfloat16()
    x[4].zero_()
    q, s = oracle.quantize_act(x)
    xb = x.float().view(9, 56, 128)
    s_t = (xb.abs().amax(dim=2) * (1.0 / 448.0)).clamp_min(1e-12)
    q_t = (xb * (1.0 / s_t).unsqueeze(2)).to(torch.float8_e4m3fn).view(9, 7168)
    assert torch.equal(s, s_t.t().contiguous())
    assert torch.equal(q.view(torch.uint8), q_t.view(torch.uint8))


def test_half_row_restatement(oracle):
    """The numpy restatement of the half form of un-rounded rows (include/b200moe.h, ``partial_format``): layout, scale
    byte = exponent of the group maximum, 11 significant bits per value, zero and tiny groups, and agreement with
    torch's own float32 -> float16 conversion.  The GPU tests require the library's bytes to equal this restatement."""
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((6, 7168)) * np.exp(rng.uniform(-30, 30, (6, 896)).repeat(8, axis=1))).astype(np.float32)
    x[0, :16] = 0.0                                   # all-zero groups
    x[1, 8:16] = [3e-38, 0, 0, 0, 0, 0, 0, 0]         # below 2^-113: flushed to zero by the clamp at 14
    x[2, 0:8] = [1.0, 2.0 ** -10, 2.0 ** -20, -(2.0 ** -27), 0.3, -0.7, 2.0 ** -30, 0.0]
    enc = oracle.encode_half_rows(x)
    assert enc.shape == (6, 15232) and enc.dtype == np.uint8
    eb = enc[:, 14336:].astype(np.int64)
    g = x.reshape(6, 896, 8)
    gmax = np.abs(g).max(axis=2)
    big = gmax >= 2.0 ** -113
    assert (eb[big] == (np.frexp(gmax[big])[1] - 1 + 127)).all() and (eb[~big] == 14).all()
    dec = oracle.decode_half_rows(enc).reshape(6, 896, 8)
    assert (dec[~big] == 0).all()
    err = np.abs(dec - g)[big]
    bound = (np.abs(g) * 2.0 ** -11 + gmax[:, :, None] * 2.0 ** -39)[big]
    assert (err <= bound).all()
    # the scaled values are what torch converts to float16 as well
    k = np.ldexp(np.float32(1.0), (141 - eb)).astype(np.float32)
    want = torch.from_numpy(g * k[:, :, None]).to(torch.float16).numpy().view(np.uint8).reshape(6, 14336)
    assert (enc[:, :14336] == want).all()
    # the largest magnitude of a group lands in [2^14, 2^15]
    top = np.abs(enc[:, :14336].copy().view(np.float16).reshape(6, 896, 8).astype(np.float32)).max(axis=2)
    assert ((top[big] >= 2.0 ** 14) & (top[big] <= 2.0 ** 15)).all()
