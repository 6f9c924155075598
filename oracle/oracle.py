"""TEST INFRASTRUCTURE — not part of the product.

ctypes wrapper of the CPU oracle (oracle/route_sort.c, oracle/forward.c, oracle/quant.c): the reference's routing
(solution/cuda/binding.py:38-61), sort metadata (solution/cuda/binding.py:134-154 and
solution/python/pure_triton_impl.py:512-531) and fp32-dequant expert path (solution/cuda/binding.py:96-185) restated
for the host, plus the activation-quantiser recipe of its profiling script (scripts/yjl_ncu.py:413-416).  Only the
tests, the driver's smoke check and bench.py's CPU-baseline legs import this module; nothing in ``fused_moe_b200`` does.

Parity pin: tests/golden/*.npz hold outputs of the reference's own ``binding.py`` run on seeded inputs
(tests/golden/make_golden.py); tests/test_oracle.py checks this oracle against them.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np
import torch

ORACLE_DIR = Path(__file__).resolve().parent
LIB_PATH = ORACLE_DIR / "liboracle.so"
TOP_K = 8
H = 7168
BLOCK_M = 128

_lib = None


def build(force: bool = False) -> Path:
    srcs = [ORACLE_DIR / "route_sort.c", ORACLE_DIR / "forward.c", ORACLE_DIR / "quant.c", ORACLE_DIR / "Makefile"]
    stale = force or not LIB_PATH.exists() or any(s.stat().st_mtime > LIB_PATH.stat().st_mtime for s in srcs)
    if stale:
        if force:
            subprocess.run(["make", "-C", str(ORACLE_DIR), "clean"], check=True, capture_output=True)
        subprocess.run(["make", "-C", str(ORACLE_DIR)], check=True, capture_output=True)
    return LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = C.CDLL(str(LIB_PATH))
        lib.oracle_sigmoid.restype = C.c_float
        lib.oracle_sigmoid.argtypes = [C.c_float]
        lib.oracle_route.restype = None
        lib.oracle_route.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
        lib.oracle_sort.restype = C.c_int
        lib.oracle_sort.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 5
        lib.oracle_forward.restype = C.c_long
        lib.oracle_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 8 + [C.c_int]
        lib.oracle_f32_to_e4m3.restype = C.c_uint8
        lib.oracle_f32_to_e4m3.argtypes = [C.c_float]
        lib.oracle_quantize_act.restype = None
        lib.oracle_quantize_act.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        _lib = lib
    return _lib


def _cpu(t: torch.Tensor) -> torch.Tensor:
    return t.detach().cpu().contiguous()


def _bytes(t: torch.Tensor) -> torch.Tensor:
    t = _cpu(t)
    return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t


def route(routing_logits: torch.Tensor, routing_bias: torch.Tensor, routed_scaling_factor: float):
    """-> (topk_idx int32 [T,8], topk_w float32 [T,8]); descending biased score, ties to the lower expert id."""
    logits = _cpu(routing_logits).float()
    bias = _cpu(routing_bias).reshape(-1).view(torch.int16)
    T = logits.shape[0]
    idx = torch.empty((T, TOP_K), dtype=torch.int32)
    w = torch.empty((T, TOP_K), dtype=torch.float32)
    _load().oracle_route(logits.data_ptr(), bias.data_ptr(), T, float(routed_scaling_factor), idx.data_ptr(),
                         w.data_ptr())
    return idx, w


def sort(topk_idx: torch.Tensor, topk_w: torch.Tensor, E_local: int, local_expert_offset: int, block_m: int = BLOCK_M):
    """-> dict(counts, block_offsets, total_blocks, sorted_token_ids, sorted_weights, scatter_map); the sorted arrays
    are cut to total_blocks*block_m rows."""
    idx = _cpu(topk_idx).to(torch.int32)
    w = _cpu(topk_w).float()
    T = idx.shape[0]
    r_max = (8 * T // block_m + E_local) * block_m
    counts = torch.zeros(E_local, dtype=torch.int32)
    offs = torch.zeros(E_local + 1, dtype=torch.int32)
    ids = torch.full((max(r_max, 1),), -7, dtype=torch.int32)
    sw = torch.zeros(max(r_max, 1), dtype=torch.float32)
    smap = torch.zeros(max(T * TOP_K, 1), dtype=torch.int32)
    tb = _load().oracle_sort(idx.data_ptr(), w.data_ptr(), T, E_local, local_expert_offset, block_m, counts.data_ptr(),
                             offs.data_ptr(), ids.data_ptr(), sw.data_ptr(), smap.data_ptr())
    n = tb * block_m
    return dict(counts=counts, block_offsets=offs, total_blocks=tb, sorted_token_ids=ids[:n], sorted_weights=sw[:n],
                scatter_map=smap[:T * TOP_K].view(T, TOP_K))


def forward_from_topk(topk_idx, topk_w, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
                      gemm2_weights, gemm2_weights_scale, local_expert_offset, num_threads: int = 0):
    """fp32-dequant expert path -> (out_f32 [T,7168], out_bf16 [T,7168], local_pairs)."""
    idx = _cpu(topk_idx).to(torch.int32)
    w = _cpu(topk_w).float()
    T = idx.shape[0]
    E_local = gemm1_weights.shape[0]
    hs, hss = _bytes(hidden_states), _cpu(hidden_states_scale).float()
    w13, w13s = _bytes(gemm1_weights), _cpu(gemm1_weights_scale).float()
    w2, w2s = _bytes(gemm2_weights), _cpu(gemm2_weights_scale).float()
    out32 = torch.empty((T, H), dtype=torch.float32)
    out16 = torch.empty((T, H), dtype=torch.int16)
    threads = num_threads or (os.cpu_count() or 1)
    pairs = _load().oracle_forward(idx.data_ptr(), w.data_ptr(), T, E_local, int(local_expert_offset), hs.data_ptr(),
                                   hss.data_ptr(), w13.data_ptr(), w13s.data_ptr(), w2.data_ptr(), w2s.data_ptr(),
                                   out32.data_ptr(), out16.data_ptr(), threads)
    if pairs < 0:
        raise MemoryError("oracle_forward: out of memory")
    return out32, out16.view(torch.bfloat16), int(pairs)


def kernel(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
           gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor, num_threads: int = 0):
    """Whole layer on the CPU -> dict(topk_idx, topk_w, out_f32, out_bf16, pairs)."""
    idx, w = route(routing_logits, routing_bias, float(routed_scaling_factor))
    out32, out16, pairs = forward_from_topk(idx, w, hidden_states, hidden_states_scale, gemm1_weights,
                                            gemm1_weights_scale, gemm2_weights, gemm2_weights_scale,
                                            int(local_expert_offset), num_threads)
    return dict(topk_idx=idx, topk_w=w, out_f32=out32, out_bf16=out16, pairs=pairs)


def quantize_act(x_bf16: torch.Tensor):
    """bf16 [T,7168] -> (e4m3 [T,7168], float32 scales [56,T]): s = max(amax/448, 1e-12), q = e4m3(x * (1/s))."""
    x = _cpu(x_bf16)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == H
    T = x.shape[0]
    q = torch.empty((T, H), dtype=torch.uint8)
    s = torch.empty((H // 128, T), dtype=torch.float32)
    _load().oracle_quantize_act(x.view(torch.int16).data_ptr(), T, q.data_ptr(), s.data_ptr())
    return q.view(torch.float8_e4m3fn), s


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    lib = _load()
    return np.array([lib.oracle_f32_to_e4m3(float(v)) for v in np.asarray(x, dtype=np.float32).ravel()], dtype=np.uint8)


def sigmoid(x: np.ndarray) -> np.ndarray:
    lib = _load()
    return np.array([lib.oracle_sigmoid(float(v)) for v in np.asarray(x, dtype=np.float32).ravel()], dtype=np.float32)


def encode_half_rows(x: np.ndarray) -> np.ndarray:
    """float32 [n, 7168] -> uint8 [n, 15232]: the half form of un-rounded result rows that the library uses between
    GEMM2 and the reduce and for the partial rows an expert-parallel shard returns (no reference counterpart; the
    format is stated in include/b200moe.h at ``partial_format``).  Group g = columns 8g..8g+7: scale byte b = biased
    float32 exponent of the group's largest magnitude, clamped to [14, 254]; the eight values times 2^(141 - b),
    rounded to float16 (nearest even); 896 x 16 bytes of float16, then the 896 scale bytes."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.shape[0]
    g = x.reshape(n, 896, 8)
    m = np.abs(g).max(axis=2)
    eb = (m.view(np.uint32) >> 23).astype(np.int64)
    eb = np.clip(eb, 14, 254)
    k = ((268 - eb) << 23).astype(np.uint32).view(np.float32)           # 2^(141 - eb), exact
    halves = (g * k[:, :, None]).astype(np.float16)                     # a power-of-two factor: the product is exact
    out = np.empty((n, 15232), dtype=np.uint8)
    out[:, :14336] = halves.reshape(n, 7168).view(np.uint8).reshape(n, 14336)
    out[:, 14336:] = eb.astype(np.uint8)
    return out


def decode_half_rows(rows: np.ndarray) -> np.ndarray:
    """uint8 [n, 15232] -> float32 [n, 7168]: value = float16 * 2^(b - 141) (b = 14 decodes to zero)."""
    rows = np.ascontiguousarray(rows, dtype=np.uint8)
    n = rows.shape[0]
    halves = rows[:, :14336].copy().view(np.float16).reshape(n, 896, 8).astype(np.float32)
    eb = rows[:, 14336:].astype(np.int64)
    k = ((eb - 14) << 23).astype(np.uint32).view(np.float32)
    return (halves * k[:, :, None]).reshape(n, 7168)
