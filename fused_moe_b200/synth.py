"""Seeded synthetic inputs with the operator's shapes, dtypes and value distributions.

The contest workloads the reference was measured on are not distributed with it, so tests and benchmarks use these
stand-ins: hidden states ~N(0,1) rounded to bf16 then quantised to e4m3 with one fp32 scale per token per 128 columns
(amax/448, stored [56,T]); router logits ~N(0,1) (optionally plus a per-expert offset ~N(0,1.5) for skewed, "hot
expert" traffic); bias ~N(0,0.1) in bf16; W13 and W2 ~N(0,0.02) quantised to e4m3 with fp32 128x128 block scales
(recipe as in the reference's profiling script, scripts/yjl_ncu.py:413-416).

Values come from a counter-based integer hash, not from torch's RNG: every element is a pure function of
(seed, tensor tag, expert, element index) computed with wrapping int64 arithmetic and exactly-rounded float32
operations, so a CPU run and a CUDA run — or two different machines — produce bit-identical tensors.  The normal
deviate is the centred sum of eight uniform 16-bit fields (Irwin-Hall, |z| <= 4.9).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

H = 7168
I = 2048
E_GLOBAL = 256
_FP8 = torch.float8_e4m3fn
_M64 = (1 << 64) - 1


def _i64(x: int) -> int:
    x &= _M64
    return x - (1 << 64) if x >= (1 << 63) else x


def _mix_scalar(x: int) -> int:
    x &= _M64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _M64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _M64
    x ^= x >> 31
    return x


def _lsr(x: torch.Tensor, k: int) -> torch.Tensor:
    return (x >> k) & ((1 << (64 - k)) - 1)


def _mix(x: torch.Tensor) -> torch.Tensor:
    x = x ^ _lsr(x, 30)
    x = x * _i64(0xBF58476D1CE4E5B9)
    x = x ^ _lsr(x, 27)
    x = x * _i64(0x94D049BB133111EB)
    x = x ^ _lsr(x, 31)
    return x


def _fields_sum(h: torch.Tensor) -> torch.Tensor:
    return (h & 0xFFFF) + (_lsr(h, 16) & 0xFFFF) + (_lsr(h, 32) & 0xFFFF) + _lsr(h, 48)


_INV_STD = 1.0 / 53509.6  # std of the sum of eight uniform{0..65535}
# amax/448 written as a multiplication: torch divides by a scalar exactly on the CPU but multiplies by the reciprocal on
# CUDA, which would make the two devices disagree in the last bit of the scale
_INV_448 = 1.0 / 448.0


def normal(n: int, seed: int, tag: int, sub: int = 0, device="cpu") -> torch.Tensor:
    """n approximately-N(0,1) float32 values, a pure function of (seed, tag, sub, index)."""
    key = _mix_scalar(_mix_scalar(seed * 0x9E3779B97F4A7C15 + tag) + sub)
    idx = torch.arange(n, dtype=torch.int64, device=device)
    base = idx * _i64(0x9E3779B97F4A7C15) + _i64(key)
    s = _fields_sum(_mix(base)) + _fields_sum(_mix(base ^ _i64(0xD1B54A32D192ED03)))
    return (s - 262140).to(torch.float32) * _INV_STD


def quantize_act(x: torch.Tensor):
    """[T,7168] float32 -> (e4m3 [T,7168], scales [56,T] float32), one scale per token per 128 columns."""
    T = x.shape[0]
    xb = x.view(T, H // 128, 128)
    s = (xb.abs().amax(dim=2) * _INV_448).clamp_min(1e-12)
    q = (xb / s.unsqueeze(2)).to(_FP8).view(T, H)
    return q, s.t().contiguous()


def quantize_weight(w: torch.Tensor):
    """[N,K] float32 -> (e4m3 [N,K], scales [N/128, K/128] float32), one scale per 128x128 block."""
    N, K = w.shape
    wb = w.view(N // 128, 128, K // 128, 128)
    s = (wb.abs().amax(dim=(1, 3)) * _INV_448).clamp_min(1e-12)
    q = (wb / s[:, None, :, None]).to(_FP8).view(N, K)
    return q, s.contiguous()


def make_inputs(T: int, E_local: int = 32, seed: int = 0, local_expert_offset: int = 0, skew: bool = False,
                device="cpu", routed_scaling_factor: float = 2.5, weights: Optional[Dict] = None,
                only_experts=None, heavy_tail: bool = False) -> Dict:
    """Keyword arguments for ``kernel(**inputs)``.  ``weights`` (a previous result) lets callers reuse the expert
    weights, which dominate generation time; expert e of the result is GLOBAL expert local_expert_offset+e, so
    shards of an expert-parallel run see consistent weights.  ``only_experts`` (local ids) generates just those
    experts and leaves the others zero — CPU tests use it to skip experts no token reaches.  ``heavy_tail`` gives the
    activations a log-normal magnitude per token (x 0.01 .. x 100) and 20x outliers on ~0.3 % of the elements, so the
    SwiGLU intermediates span the range reported for real traces (p99 above 1e4) instead of staying near 1."""
    dev = torch.device(device)
    hs = normal(T * H, seed, 1, device=dev).view(T, H)
    if heavy_tail:
        mag = torch.exp(2.3 * normal(T, seed, 7, device=dev).clamp(-2.0, 2.0)).view(T, 1)
        spike = normal(T * H, seed, 8, device=dev).view(T, H).abs() > 3.0
        hs = hs * mag * torch.where(spike, 20.0, 1.0)
    hs = hs.bfloat16().float()
    hs_q, hs_s = quantize_act(hs)
    logits = normal(T * E_GLOBAL, seed, 2, device=dev).view(T, E_GLOBAL)
    if skew:
        logits = logits + 1.5 * normal(E_GLOBAL, seed, 3, device=dev).view(1, E_GLOBAL)
    bias = (0.1 * normal(E_GLOBAL, seed, 4, device=dev)).bfloat16()
    out = {
        "routing_logits": logits.contiguous(),
        "routing_bias": bias,
        "hidden_states": hs_q,
        "hidden_states_scale": hs_s,
        "local_expert_offset": local_expert_offset,
        "routed_scaling_factor": routed_scaling_factor,
    }
    if weights is not None:
        for k in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale"):
            out[k] = weights[k]
        return out
    w13 = torch.zeros((E_local, 2 * I, H), dtype=torch.uint8, device=dev).view(_FP8)
    w13s = torch.zeros((E_local, 2 * I // 128, H // 128), dtype=torch.float32, device=dev)
    w2 = torch.zeros((E_local, H, I), dtype=torch.uint8, device=dev).view(_FP8)
    w2s = torch.zeros((E_local, H // 128, I // 128), dtype=torch.float32, device=dev)
    for e in (range(E_local) if only_experts is None else sorted(set(int(x) for x in only_experts))):
        ge = local_expert_offset + e
        a = 0.02 * normal(2 * I * H, seed, 5, ge, dev).view(2 * I, H)
        w13[e], w13s[e] = quantize_weight(a)
        b = 0.02 * normal(H * I, seed, 6, ge, dev).view(H, I)
        w2[e], w2s[e] = quantize_weight(b)
    out.update(gemm1_weights=w13, gemm1_weights_scale=w13s, gemm2_weights=w2, gemm2_weights_scale=w2s)
    return out
