"""ctypes binding of libb200moe.so (the C ABI declared in include/b200moe.h).

The library is the only compute path of this package: if it is missing or does not load, importing callers get a
RuntimeError — there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libb200moe.so"

OK, EINVAL, EWORKSPACE, ECUDA, EDEVICE, EUNSUPPORTED, ETOOLARGE = 0, -1, -2, -3, -4, -5, -6
SORT_STATIC_MAX_ENTRIES = 32768
EP_RECORD_BYTES = 7456
DECODE_MAX_T = 8
DECODE_MAX_WORK = 128


def uses_decode_path(T: int, E_local: int) -> bool:
    """Whether b200moe_forward takes the matrix-vector stages for a routed call with dense inputs (the weights are then
    streamed once per (token, expert) pair, which wins while pairs rarely share an expert: about 4 expected pairs)."""
    return T <= DECODE_MAX_T and T * E_local <= DECODE_MAX_WORK

PROLOGUE_MAX_T = 32
SKINNY_MAX_T = 112


PARTIAL_F32, PARTIAL_HALF = 0, 1      # b200moe_problem.partial_format
HALF_ROW_BYTES = 15232                # bytes of one row in the half form


class Problem(C.Structure):
    """Mirror of ``b200moe_problem``."""

    _fields_ = [
        ("T", C.c_int32),
        ("E_local", C.c_int32),
        ("local_expert_offset", C.c_int32),
        ("routed_scaling_factor", C.c_float),
        ("routing_logits", C.c_void_p),
        ("routing_bias", C.c_void_p),
        ("hidden_states", C.c_void_p),
        ("hidden_states_scale", C.c_void_p),
        ("gemm1_weights", C.c_void_p),
        ("gemm1_weights_scale", C.c_void_p),
        ("gemm2_weights", C.c_void_p),
        ("gemm2_weights_scale", C.c_void_p),
        ("output", C.c_void_p),
        ("topk_idx_in", C.c_void_p),
        ("topk_w_in", C.c_void_p),
        ("output_f32", C.c_void_p),
        ("hidden_row_stride", C.c_int64),
        ("scale_token_stride", C.c_int64),
        ("scale_block_stride", C.c_int64),
        ("topk_row_stride", C.c_int64),
        ("out_seg_count", C.c_int32),
        ("out_seg_start", C.c_int32 * 9),
        ("out_seg_base", C.c_void_p * 8),
        ("plan", C.c_void_p),
        ("partial_format", C.c_int32),
    ]


class EpPeers(C.Structure):
    """Mirror of ``b200moe_ep_peers``."""

    _fields_ = [
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("recv_records", C.c_void_p * 8),
        ("flags", C.c_void_p * 8),
        ("counts", C.c_void_p * 8),
        ("back_rows", C.c_void_p * 8),
        ("cap_recv", C.c_int32),
        ("cap_back", C.c_int32),
        ("back_row_bytes", C.c_int32),
    ]


class EpPlan(C.Structure):
    """Mirror of ``b200moe_ep_plan`` (lives in device memory; this mirror is for reading it back in tests and tools)."""

    _fields_ = [
        ("ok", C.c_int32),
        ("n_recv", C.c_int32),
        ("n_send", C.c_int32),
        ("seg_count", C.c_int32),
        ("seg_start", C.c_int32 * 9),
        ("dst_row0", C.c_int32 * 8),
        ("rank", C.c_int32),
        ("seg_base", C.c_void_p * 8),
        ("matrix", C.c_int32 * 64),
    ]


class Workspace(C.Structure):
    """Mirror of ``b200moe_workspace``."""

    _fields_ = [
        ("T", C.c_int32),
        ("E_local", C.c_int32),
        ("R_max", C.c_int32),
        ("n_chunks", C.c_int32),
        ("topk_idx", C.c_void_p),
        ("topk_w", C.c_void_p),
        ("chunk_bits", C.c_void_p),
        ("chunk_base", C.c_void_p),
        ("counts", C.c_void_p),
        ("block_offsets", C.c_void_p),
        ("total_blocks", C.c_void_p),
        ("status", C.c_void_p),
        ("sorted_token_ids", C.c_void_p),
        ("sorted_weights", C.c_void_p),
        ("scatter_map", C.c_void_p),
        ("a_sorted", C.c_void_p),
        ("a_scale_sorted", C.c_void_p),
        ("inter_q", C.c_void_p),
        ("inter_scale", C.c_void_p),
        ("expert_out", C.c_void_p),
        ("gemm_tile_ctr", C.c_void_p),
        ("gemm_partial", C.c_void_p),
        ("status_mirror", C.c_void_p),
    ]


# name -> (restype, argtypes); every symbol include/b200moe.h declares.
_PW = (C.POINTER(Problem), C.POINTER(Workspace), C.c_void_p)
SYMBOLS = {
    "b200moe_version": (C.c_int, ()),
    "b200moe_strerror": (C.c_char_p, (C.c_int,)),
    "b200moe_last_cuda_error": (C.c_char_p, ()),
    "b200moe_workspace_bytes": (C.c_int, (C.c_int32, C.c_int32, C.POINTER(C.c_size_t))),
    "b200moe_workspace_carve": (C.c_int, (C.c_void_p, C.c_size_t, C.c_int32, C.c_int32, C.POINTER(Workspace))),
    "b200moe_workspace_init": (C.c_int, (C.POINTER(Workspace), C.c_void_p)),
    "b200moe_forward": (C.c_int, _PW),
    "b200moe_quantize_act": (C.c_int, (C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p)),
    "b200moe_route": (C.c_int, _PW),
    "b200moe_route_topk": (C.c_int, (C.c_void_p, C.c_void_p, C.c_int32, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p)),
    "b200moe_topk_bits": (C.c_int, _PW),
    "b200moe_sort": (C.c_int, _PW),
    "b200moe_gather": (C.c_int, _PW),
    "b200moe_prologue_small": (C.c_int, _PW),
    "b200moe_gemm1_skinny": (C.c_int, _PW),
    "b200moe_gemm2_skinny": (C.c_int, _PW),
    "b200moe_gemm1": (C.c_int, _PW),
    "b200moe_gemm2": (C.c_int, _PW),
    "b200moe_gemm2_half": (C.c_int, _PW),
    "b200moe_reduce": (C.c_int, _PW),
    "b200moe_reduce_half": (C.c_int, _PW),
    "b200moe_gemv1": (C.c_int, _PW),
    "b200moe_gemv2": (C.c_int, _PW),
    "b200moe_sort_static": (C.c_int, (C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32) + (C.c_void_p,) * 7),
    "b200moe_ep_scratch_bytes": (C.c_int, (C.c_int32, C.c_int32, C.POINTER(C.c_size_t))),
    "b200moe_ep_dispatch": (C.c_int, (C.c_void_p,) * 4 + (C.c_int32, C.c_int32, C.c_void_p, C.c_size_t) + (C.c_void_p,) * 4),
    "b200moe_ep_record_layout": (C.c_int, (C.c_void_p, C.c_int32, C.POINTER(Problem))),
    "b200moe_ep_rank": (C.c_int, (C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p,
                                  C.c_void_p)),
    "b200moe_ep_pack_peers": (C.c_int, (C.c_void_p,) * 4 + (C.c_int32, C.POINTER(EpPeers), C.POINTER(C.c_int32),
                                                           C.c_void_p, C.c_size_t, C.c_void_p)),
    "b200moe_ep_barrier": (C.c_int, (C.POINTER(EpPeers), C.c_int32, C.c_void_p, C.c_void_p)),
    "b200moe_ep_exchange_counts": (C.c_int, (C.POINTER(EpPeers), C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p,
                                             C.c_void_p)),
    "b200moe_ep_pack_peers_planned": (C.c_int, (C.c_void_p,) * 4 + (C.c_int32, C.POINTER(EpPeers), C.c_void_p,
                                                                   C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p)),
    "b200moe_set_wait_limit_cycles": (C.c_int, (C.c_int64,)),
    "b200moe_ep_combine": (C.c_int, (C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p)),
    "b200moe_ep_combine_half": (C.c_int, (C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p)),
    "b200moe_read_status": (C.c_int, (C.POINTER(Workspace), C.c_void_p, C.POINTER(C.c_int32 * 4))),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library once; raises RuntimeError when it is absent (build it with
    ``python -m fused_moe_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: run `python -m fused_moe_b200.build` (needs nvcc); "
            "this package has no fallback path")
    try:
        lib = C.CDLL(str(LIB_PATH))
    except OSError as exc:  # pragma: no cover - depends on the machine
        raise RuntimeError(f"cannot load {LIB_PATH}: {exc}") from exc
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError here = header/library mismatch
        fn.restype = res
        fn.argtypes = list(args)
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    """Raises RuntimeError / ValueError for a non-zero library return code."""
    if rc == OK:
        return
    lib = load()
    msg = lib.b200moe_strerror(rc).decode()
    if rc == ECUDA:
        msg += ": " + lib.b200moe_last_cuda_error().decode()
    if rc == EINVAL:
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg}")
