"""Drop-in entry point: the DeepSeek-V3 FP8 block-scale fused MoE layer on B200.

``kernel(...)`` keeps the signature, argument meaning and return convention of the reference entry point
(solution/python/kernel.py:71-83; host orchestration solution/python/pure_triton_impl.py:2125-2403): ten inputs plus
an optional destination ``output``; the bf16 ``[T, 7168]`` result is always returned.  Everything on the device is
done by libb200moe.so through its C ABI (include/b200moe.h); PyTorch only provides device memory and the stream.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch

from . import _lib

H = 7168
I = 2048
E_GLOBAL = 256
TOP_K = 8
BLOCK_M = 128
H_BLOCKS = H // 128
I_BLOCKS = I // 128

_FP8 = torch.float8_e4m3fn


@dataclass
class _Workspace:
    """One carved view of the per-device scratch buffer, for exactly (T, E_local)."""

    struct: _lib.Workspace
    base_ptr: int
    buffer: torch.Tensor

    def view(self, name: str, dtype: torch.dtype, shape: Tuple[int, ...]) -> torch.Tensor:
        """Torch view (no copy) of one workspace array; for tests and debugging."""
        ptr = getattr(self.struct, name)
        off = ptr - self.base_ptr
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.buffer[off:off + nbytes].view(dtype).view(*shape)


@dataclass
class _DeviceState:
    """Per-device scratch: ONE buffer, carved per (T, E_local), shared by every call on that device.  One workspace
    serves one stream at a time: calls issued on different streams of a device must be ordered by the caller."""

    buffer: Optional[torch.Tensor] = None
    carved: Dict[Tuple[int, int], _Workspace] = field(default_factory=dict)
    active: Optional[Tuple[int, int]] = None
    mirror: Optional[torch.Tensor] = None   # pinned host int32[4]: the device copies a non-zero status word here
    mirror_np: object = None                # numpy view of it (a plain memory read per call)


_devices: Dict[int, _DeviceState] = {}
_host_scalar_cache: Dict[tuple, object] = {}


def _host_scalar(x, cast):
    """Python scalar from a scalar or a 0-d tensor; a device tensor is read back once per (address, dtype), as the
    reference does (solution/python/pure_triton_impl.py:2012-2020)."""
    if torch.is_tensor(x):
        key = (x.data_ptr(), str(x.device), str(x.dtype), cast.__name__)
        if key not in _host_scalar_cache:
            _host_scalar_cache[key] = cast(x.item())
        return _host_scalar_cache[key]
    return cast(x)


def workspace_bytes(T: int, E_local: int) -> int:
    n = C.c_size_t(0)
    _lib.check(_lib.load().b200moe_workspace_bytes(T, E_local, C.byref(n)), "b200moe_workspace_bytes")
    return n.value


def _raise_if_failed(st: _DeviceState) -> None:
    """Looks at the host-visible mirror of the device status word (a read of host memory, no synchronisation).  The last
    kernel of a layer call copies a non-zero status there, so a call whose bounded wait ran out is reported by the next
    call on that device at the latest (``check_status`` reports it at once, at the price of a synchronisation)."""
    m = st.mirror_np
    if m is None or m[0] == 0:
        return
    code, block, role, detail = (int(x) for x in m)
    m[:] = 0
    st.active = None    # next call clears the device status word and the tile tickets (b200moe_workspace_init)
    raise RuntimeError(f"an earlier layer call failed on the device: status code={code} block={block} role={role} "
                       f"detail={detail}; its output is invalid")


def _workspace(device: torch.device, T: int, E_local: int, stream_ptr: int) -> _Workspace:
    lib = _lib.load()
    st = _devices.setdefault(device.index, _DeviceState())
    if st.mirror is None:
        st.mirror = torch.zeros(4, dtype=torch.int32).pin_memory()
        st.mirror_np = st.mirror.numpy()
    _raise_if_failed(st)
    need = workspace_bytes(T, E_local)
    if st.buffer is None or st.buffer.numel() < need:
        st.buffer = torch.empty(need, dtype=torch.uint8, device=device)
        st.carved.clear()
        st.active = None
    key = (T, E_local)
    ws = st.carved.get(key)
    if ws is None:
        s = _lib.Workspace()
        base = st.buffer.data_ptr()
        _lib.check(lib.b200moe_workspace_carve(base, st.buffer.numel(), T, E_local, C.byref(s)),
                   "b200moe_workspace_carve")
        # pinned host memory is addressable from the device at the same address (unified addressing)
        s.status_mirror = st.mirror.data_ptr()
        ws = _Workspace(struct=s, base_ptr=base, buffer=st.buffer)
        st.carved[key] = ws
    if st.active != key:
        # the status word and the tile tickets sit at (T, E_local)-dependent offsets of the shared buffer: clear them
        # when the layout changes (and after a failed call, which may have left tickets behind)
        _lib.check(lib.b200moe_workspace_init(C.byref(ws.struct), stream_ptr), "b200moe_workspace_init")
        st.active = key
    return ws


def _require(t: torch.Tensor, name: str, dtype: torch.dtype, shape: Tuple[int, ...]) -> torch.Tensor:
    if not torch.is_tensor(t):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if tuple(t.shape) != shape:
        raise ValueError(f"{name} must have shape {shape}, got {tuple(t.shape)}")
    return t if t.is_contiguous() else t.contiguous()


def _require_cuda(**tensors) -> None:
    for name, t in tensors.items():
        if t is not None and not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU path")


def _problem(T, E_local, offset, scale, logits, bias, hs, hs_scale, w13, w13s, w2, w2s, out, topk_idx=None,
             topk_w=None) -> _lib.Problem:
    p = _lib.Problem()
    p.T, p.E_local, p.local_expert_offset, p.routed_scaling_factor = T, E_local, offset, scale
    p.routing_logits = logits.data_ptr() if logits is not None else None
    p.routing_bias = bias.data_ptr() if bias is not None else None
    p.hidden_states = hs.data_ptr()
    p.hidden_states_scale = hs_scale.data_ptr()
    p.gemm1_weights = w13.data_ptr()
    p.gemm1_weights_scale = w13s.data_ptr()
    p.gemm2_weights = w2.data_ptr()
    p.gemm2_weights_scale = w2s.data_ptr()
    if out.dtype == torch.float32:
        p.output, p.output_f32 = None, out.data_ptr()
    else:
        p.output, p.output_f32 = out.data_ptr(), None
    p.topk_idx_in = topk_idx.data_ptr() if topk_idx is not None else None
    p.topk_w_in = topk_w.data_ptr() if topk_w is not None else None
    return p


def _check_weights(hidden_states, gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale):
    if not torch.is_tensor(gemm1_weights) or gemm1_weights.dim() != 3:
        raise ValueError("gemm1_weights must be [E_local, 4096, 7168]")
    E_local = int(gemm1_weights.shape[0])
    if not 1 <= E_local <= E_GLOBAL:
        raise ValueError(f"E_local must be in 1..{E_GLOBAL}, got {E_local}")
    w13 = _require(gemm1_weights, "gemm1_weights", _FP8, (E_local, 2 * I, H))
    w13s = _require(gemm1_weights_scale, "gemm1_weights_scale", torch.float32, (E_local, 2 * I_BLOCKS, H_BLOCKS))
    w2 = _require(gemm2_weights, "gemm2_weights", _FP8, (E_local, H, I))
    w2s = _require(gemm2_weights_scale, "gemm2_weights_scale", torch.float32, (E_local, H_BLOCKS, I_BLOCKS))
    return E_local, w13, w13s, w2, w2s


def _run(T, E_local, offset, scale, logits, bias, hs, hs_scale, w13, w13s, w2, w2s, output, topk_idx, topk_w,
         out_dtype=torch.bfloat16):
    _require_cuda(routing_logits=logits, routing_bias=bias, hidden_states=hs, hidden_states_scale=hs_scale,
                  gemm1_weights=w13, gemm1_weights_scale=w13s, gemm2_weights=w2, gemm2_weights_scale=w2s,
                  topk_idx=topk_idx, topk_weights=topk_w)
    device = hs.device
    if offset < 0 or offset + E_local > E_GLOBAL:
        raise ValueError(f"local_expert_offset {offset} with {E_local} local experts exceeds {E_GLOBAL} experts")
    if output is None:
        output = torch.empty((T, H), dtype=out_dtype, device=device)
    else:
        if output.dtype != out_dtype or tuple(output.shape) != (T, H) or not output.is_contiguous():
            raise ValueError(f"output must be a contiguous {out_dtype} tensor of shape [T, 7168]")
        if output.device != device:
            raise RuntimeError("output must live on the device of hidden_states")
    if T == 0:
        return output
    with torch.cuda.device(device):
        stream_ptr = torch.cuda.current_stream(device).cuda_stream
        ws = _workspace(device, T, E_local, stream_ptr)
        p = _problem(T, E_local, offset, scale, logits, bias, hs, hs_scale, w13, w13s, w2, w2s, output, topk_idx,
                     topk_w)
        _lib.check(_lib.load().b200moe_forward(C.byref(p), C.byref(ws.struct), stream_ptr), "b200moe_forward")
        if os.environ.get("B200MOE_CHECK_STATUS") == "1":
            check_status(device)
    return output


@torch.no_grad()
def kernel(
    routing_logits,
    routing_bias,
    hidden_states,
    hidden_states_scale,
    gemm1_weights,
    gemm1_weights_scale,
    gemm2_weights,
    gemm2_weights_scale,
    local_expert_offset,
    routed_scaling_factor,
    output=None,
):
    """Fused MoE layer; same arguments as the reference ``kernel`` (solution/python/kernel.py:71-83).

    routing_logits [T,256] f32 · routing_bias [256] bf16 · hidden_states [T,7168] e4m3 · hidden_states_scale [56,T] f32 ·
    gemm1_weights [E,4096,7168] e4m3 · gemm1_weights_scale [E,32,56] f32 · gemm2_weights [E,7168,2048] e4m3 ·
    gemm2_weights_scale [E,56,16] f32 · local_expert_offset, routed_scaling_factor: Python scalars or 0-d tensors ·
    output: optional bf16 [T,7168] destination.  Returns the output tensor.  E (local experts) is taken from the weight
    shape; the reference fixes it at 32.  Raises TypeError / ValueError on wrong dtypes or shapes and RuntimeError when
    the CUDA library is missing, an input is not on a CUDA device, or a launch fails.
    """
    if not torch.is_tensor(routing_logits) or routing_logits.dim() != 2:
        raise ValueError("routing_logits must be [T, 256]")
    T = int(routing_logits.shape[0])
    E_local, w13, w13s, w2, w2s = _check_weights(hidden_states, gemm1_weights, gemm1_weights_scale, gemm2_weights,
                                                 gemm2_weights_scale)
    logits = _require(routing_logits, "routing_logits", torch.float32, (T, E_GLOBAL))
    bias = _require(routing_bias.reshape(-1) if torch.is_tensor(routing_bias) else routing_bias, "routing_bias",
                    torch.bfloat16, (E_GLOBAL,))
    hs = _require(hidden_states, "hidden_states", _FP8, (T, H))
    hs_scale = _require(hidden_states_scale, "hidden_states_scale", torch.float32, (H_BLOCKS, T))
    offset = _host_scalar(local_expert_offset, int)
    scale = _host_scalar(routed_scaling_factor, float)
    return _run(T, E_local, offset, scale, logits, bias, hs, hs_scale, w13, w13s, w2, w2s, output, None, None)


class HostPipe:
    """Staging of the host-memory entry points (``kernel_host``, the expert-parallel shard's ``forward_host``): two
    copy streams and two sets of device buffers (router logits, e4m3 rows, output rows) plus two scale buffers, used in
    turn.  Which copy or layer call last touched a set is kept as an event ACROSS calls, so a call never waits for more
    than the buffers it is about to overwrite: with ``ready_event`` the copy-in of call k + 1 runs under the layer of
    call k and the copy-out of call k under the layer of call k + 1."""

    def __init__(self, device: torch.device, T: int, t_slice: int):
        self.device, self.T, self.t_slice = device, T, t_slice
        self.h2d, self.d2h = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.logits = [torch.empty((t_slice, E_GLOBAL), dtype=torch.float32, device=device) for _ in range(2)]
        self.hs = [torch.empty((t_slice, H), dtype=_FP8, device=device) for _ in range(2)]
        self.out = [torch.empty((t_slice, H), dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.scale = [torch.empty(H_BLOCKS * T, dtype=torch.float32, device=device) for _ in range(2)]
        self.done = [None, None]         # the layer has finished reading staging set k
        self.drained = [None, None]      # the copy-out has finished reading out[k]
        self.scale_free = [None, None]   # every layer call of the batch that used scale[j] has taken its slice
        self.runs = 0
        self.calls = 0

    @staticmethod
    def get(owner: dict, key, device: torch.device, T: int, t_slice: int) -> "HostPipe":
        """The pipe kept under ``owner[key]``, replaced by a larger one when the batch outgrows it (after the device
        has finished with the old buffers)."""
        pipe = owner.get(key)
        if pipe is None or pipe.t_slice < t_slice or pipe.T < T:
            if pipe is not None:
                torch.cuda.synchronize(device)
            pipe = HostPipe(device, T, t_slice)
            owner[key] = pipe
        return pipe

    def run(self, layer, logits, hs, hs_scale, output, slices: int, ready_event=None):
        """Queues the whole batch: ``layer(logits_dev, hs_dev, scale_dev, out_dev)`` is called once per run of tokens
        on the caller's current stream.  Without ``ready_event`` the caller's stream waits for the last copy-out;
        with it the event is recorded there instead and nothing waits."""
        T = int(logits.shape[0])
        t_slice = (T + slices - 1) // slices
        cur = torch.cuda.current_stream(self.device)
        h2d, d2h = self.h2d, self.d2h
        j = self.calls % 2
        self.calls += 1
        scale_dev = self.scale[j][:H_BLOCKS * T].view(H_BLOCKS, T)
        with torch.cuda.stream(h2d):
            if self.scale_free[j] is not None:
                h2d.wait_event(self.scale_free[j])
            scale_dev.copy_(hs_scale, non_blocking=True)
        last = None
        for i in range(slices):
            a, b = i * t_slice, min(T, (i + 1) * t_slice)
            n, k = b - a, self.runs % 2
            self.runs += 1
            with torch.cuda.stream(h2d):
                if self.done[k] is not None:
                    h2d.wait_event(self.done[k])
                self.logits[k][:n].copy_(logits[a:b], non_blocking=True)
                self.hs[k][:n].copy_(hs[a:b], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(h2d)
            cur.wait_event(arrived)
            if self.drained[k] is not None:
                cur.wait_event(self.drained[k])
            layer(self.logits[k][:n], self.hs[k][:n], scale_dev[:, a:b].contiguous() if slices > 1 else scale_dev,
                  self.out[k][:n])
            ev = torch.cuda.Event()
            ev.record(cur)
            self.done[k] = ev
            with torch.cuda.stream(d2h):
                d2h.wait_event(ev)
                output[a:b].copy_(self.out[k][:n], non_blocking=True)
                last = torch.cuda.Event()
                last.record(d2h)
                self.drained[k] = last
                if ready_event is not None and i == slices - 1:
                    ready_event.record(d2h)      # the caller's own event: it may re-record it whenever it likes
        self.scale_free[j] = self.done[(self.runs - 1) % 2]
        if ready_event is None:
            cur.wait_event(last)
        return output


_host_pipes: Dict[int, HostPipe] = {}


@torch.no_grad()
def kernel_host(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
                gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor, output=None,
                slices: Optional[int] = None, ready_event: Optional["torch.cuda.Event"] = None):
    """``kernel`` for activations that live in HOST memory: ``routing_logits``, ``hidden_states``,
    ``hidden_states_scale`` and ``output`` are pinned host tensors (``output=None`` allocates one), the bias and the
    expert weights are device tensors as in ``kernel``.  The tokens are cut into ``slices`` equal runs and pipelined
    over three streams, so the host-to-device copy of run i + 1 and the device-to-host copy of run i - 1 overlap the
    layer on run i; rows are independent, so the result equals one ``kernel`` call on all tokens bit for bit.
    Returns ``output`` after queueing everything.

    Without ``ready_event`` the caller's current stream waits for the last copy, so synchronising that stream (or the
    device) makes ``output`` valid; the default ``slices`` then balances the copies a call cannot hide against the
    cost of streaming the expert weights once per run.  With ``ready_event`` (a ``torch.cuda.Event``) the event is
    recorded after the last copy-out and NOTHING waits for it: wait for the event before reading ``output`` or
    rewriting the input tensors' memory.  Consecutive calls then overlap — the copy-in of the next batch runs under
    this batch's layer and this batch's copy-out under the next one's — and the default is one run per call.
    The reference has no host-memory entry point (its harness hands ``kernel`` device tensors)."""
    for name, t in (("routing_logits", routing_logits), ("hidden_states", hidden_states),
                    ("hidden_states_scale", hidden_states_scale)):
        if not torch.is_tensor(t) or t.is_cuda or (t.numel() > 0 and not t.is_pinned()):   # empty: nothing to pin
            raise RuntimeError(f"{name} must be a pinned host tensor")
    if routing_logits.dim() != 2:
        raise ValueError("routing_logits must be [T, 256]")
    T = int(routing_logits.shape[0])
    logits = _require(routing_logits, "routing_logits", torch.float32, (T, E_GLOBAL))
    hs = _require(hidden_states, "hidden_states", _FP8, (T, H))
    hs_scale = _require(hidden_states_scale, "hidden_states_scale", torch.float32, (H_BLOCKS, T))
    if output is None:
        output = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    elif (not torch.is_tensor(output) or output.is_cuda or not output.is_pinned() or output.dtype != torch.bfloat16
          or tuple(output.shape) != (T, H) or not output.is_contiguous()):
        raise ValueError("output must be a contiguous pinned host bf16 tensor of shape [T, 7168]")
    device = gemm1_weights.device
    _require_cuda(gemm1_weights=gemm1_weights)
    if T == 0:
        if ready_event is not None:
            ready_event.record(torch.cuda.current_stream(device))
        return output
    if slices is None and ready_event is not None:
        slices = 1
    if slices is None:
        # Every run streams the expert weights again (~E x 44 MB at ~5 TB/s) while the copies it can hide shrink with
        # the number of runs (22.7 KB per token over a ~55 GB/s host link): the sum is least near sqrt(copy / stream).
        # Measured at T = 16384 with 256 experts: 16.8 ms unsliced, 14.7 ms with 2 runs, 17.1 ms with 4.
        stream_s = gemm1_weights.shape[0] * 44.04e6 / 5e12
        copy_s = T * 22.7e3 / 55e9
        slices = max(1, min(8, int(round((copy_s / stream_s) ** 0.5)), T // 1024))
    if slices < 1 or slices > T:
        raise ValueError("slices must be in 1..T")

    def layer(logits_dev, hs_dev, scale_dev, out_dev):
        kernel(logits_dev, routing_bias, hs_dev, scale_dev, gemm1_weights, gemm1_weights_scale, gemm2_weights,
               gemm2_weights_scale, local_expert_offset, routed_scaling_factor, out_dev)

    with torch.cuda.device(device):
        pipe = HostPipe.get(_host_pipes, device.index, device, T, (T + slices - 1) // slices)
        return pipe.run(layer, logits, hs, hs_scale, output, slices, ready_event)


@torch.no_grad()
def quantize_activations(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 activations [T, 7168] -> (e4m3 [T, 7168], float32 scales [56, T]): the ``hidden_states`` /
    ``hidden_states_scale`` pair ``kernel`` takes, one scale per token per 128 columns (``b200moe_quantize_act``):
    s = max(amax * (1/448), 1e-12), q = e4m3(x * (1/s)).  The reference has no operator for this step; its profiling
    script builds the pair with torch by multiplying with 448 / amax (scripts/yjl_ncu.py:413-416)."""
    _require(x, "x", torch.bfloat16, (x.shape[0] if torch.is_tensor(x) and x.dim() == 2 else -1, H))
    _require_cuda(x=x)
    x = x.contiguous()
    T = x.shape[0]
    q = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((H // 128, T), dtype=torch.float32, device=x.device)
    if T == 0:
        return q, s
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().b200moe_quantize_act(x.data_ptr(), T, q.data_ptr(), s.data_ptr(),
                                                    torch.cuda.current_stream(x.device).cuda_stream),
                   "b200moe_quantize_act")
    return q, s


@torch.no_grad()
def kernel_from_topk(topk_idx, topk_weights, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
                     gemm2_weights, gemm2_weights_scale, local_expert_offset, output=None,
                     out_dtype=torch.bfloat16):
    """Same layer for tokens whose routing already ran (expert-parallel receiver): ``topk_idx`` [T,8] int32 global
    expert ids and ``topk_weights`` [T,8] f32 final weights replace logits, bias and scaling factor.  Only pairs whose
    expert lies in [offset, offset+E) contribute.  ``out_dtype=torch.float32`` returns the sums before the bfloat16
    rounding, which is how a shard's partial results travel back to the tokens' home ranks.  The reference has no such
    entry (single GPU only)."""
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("out_dtype must be torch.bfloat16 or torch.float32")
    if not torch.is_tensor(topk_idx) or topk_idx.dim() != 2:
        raise ValueError("topk_idx must be [T, 8]")
    T = int(topk_idx.shape[0])
    E_local, w13, w13s, w2, w2s = _check_weights(hidden_states, gemm1_weights, gemm1_weights_scale, gemm2_weights,
                                                 gemm2_weights_scale)
    idx = _require(topk_idx, "topk_idx", torch.int32, (T, TOP_K))
    w = _require(topk_weights, "topk_weights", torch.float32, (T, TOP_K))
    hs = _require(hidden_states, "hidden_states", _FP8, (T, H))
    hs_scale = _require(hidden_states_scale, "hidden_states_scale", torch.float32, (H_BLOCKS, T))
    offset = _host_scalar(local_expert_offset, int)
    return _run(T, E_local, offset, 1.0, None, None, hs, hs_scale, w13, w13s, w2, w2s, output, idx, w, out_dtype)


@torch.no_grad()
def kernel_from_records(records, gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale,
                        local_expert_offset, output=None, out_segments=None, plan=None, half_rows=False):
    """The layer over expert-parallel dispatch records read in place: ``records`` is uint8 [n, 7456] in the layout of
    ``b200moe_ep_dispatch`` (activations | 56 scales | 8 expert ids | 8 weights per row).  Returns float32 [n, 7168]
    partial rows (sum over THIS shard's experts), in record order.  With ``out_segments = (starts, bases)`` — row
    ranges ``starts[i]..starts[i+1]`` and raw float32 device addresses ``bases[i]`` (at most 8, possibly peer-GPU
    memory) — the rows are stored there instead and nothing is returned.  With ``plan`` (device address of a
    ``b200moe_ep_plan`` filled by ``b200moe_ep_exchange_counts``) ``records`` is the whole receive buffer (its row
    count is a capacity): how many leading rows are real and where their partial rows go is read on the device, so the
    host never learns the count; nothing is returned.  With ``half_rows`` the partial rows are written in the half
    form of ``b200moe_problem.partial_format`` (15232 bytes per row: eight float16 per scale byte) and the returned
    tensor is uint8 [n, 15232]; segment and plan destinations then have that row pitch.  No reference counterpart."""
    if not torch.is_tensor(records) or records.dim() != 2 or records.shape[1] != _lib.EP_RECORD_BYTES:
        raise ValueError(f"records must be uint8 [n, {_lib.EP_RECORD_BYTES}]")
    if records.dtype != torch.uint8 or not records.is_contiguous():
        raise TypeError("records must be a contiguous uint8 tensor")
    n = int(records.shape[0])
    E_local, w13, w13s, w2, w2s = _check_weights(None, gemm1_weights, gemm1_weights_scale, gemm2_weights,
                                                 gemm2_weights_scale)
    _require_cuda(records=records, gemm1_weights=w13, gemm1_weights_scale=w13s, gemm2_weights=w2,
                  gemm2_weights_scale=w2s)
    offset = _host_scalar(local_expert_offset, int)
    if offset < 0 or offset + E_local > E_GLOBAL:
        raise ValueError(f"local_expert_offset {offset} with {E_local} local experts exceeds {E_GLOBAL} experts")
    device = records.device
    if plan is not None:
        if out_segments is not None or output is not None:
            raise ValueError("plan excludes output and out_segments")
    elif out_segments is not None:
        starts, bases = out_segments
        if len(bases) > 8 or len(starts) != len(bases) + 1 or starts[0] != 0 or starts[-1] != n:
            raise ValueError("out_segments must cover rows 0..n with at most 8 segments")
        output = None
    elif output is None:
        output = (torch.empty((n, _lib.HALF_ROW_BYTES), dtype=torch.uint8, device=device) if half_rows
                  else torch.empty((n, H), dtype=torch.float32, device=device))
    elif half_rows:
        if (output.dtype != torch.uint8 or tuple(output.shape) != (n, _lib.HALF_ROW_BYTES)
                or not output.is_contiguous()):
            raise ValueError("output must be a contiguous uint8 tensor of shape [n, 15232]")
    elif output.dtype != torch.float32 or tuple(output.shape) != (n, H) or not output.is_contiguous():
        raise ValueError("output must be a contiguous float32 tensor of shape [n, 7168]")
    if n == 0:
        return output
    lib = _lib.load()
    with torch.cuda.device(device):
        stream_ptr = torch.cuda.current_stream(device).cuda_stream
        ws = _workspace(device, n, E_local, stream_ptr)
        p = _lib.Problem()
        _lib.check(lib.b200moe_ep_record_layout(records.data_ptr(), n, C.byref(p)), "b200moe_ep_record_layout")
        p.E_local, p.local_expert_offset, p.routed_scaling_factor = E_local, offset, 1.0
        p.gemm1_weights, p.gemm1_weights_scale = w13.data_ptr(), w13s.data_ptr()
        p.gemm2_weights, p.gemm2_weights_scale = w2.data_ptr(), w2s.data_ptr()
        p.partial_format = _lib.PARTIAL_HALF if half_rows else _lib.PARTIAL_F32
        if plan is not None:
            p.output, p.output_f32, p.plan = None, None, int(plan)
        elif out_segments is None:
            p.output, p.output_f32 = None, output.data_ptr()
        else:
            p.output, p.output_f32 = None, None
            p.out_seg_count = len(bases)
            for i, (s0, b) in enumerate(zip(starts, bases)):
                p.out_seg_start[i] = int(s0)
                p.out_seg_base[i] = int(b)
            p.out_seg_start[len(bases)] = int(starts[-1])
        _lib.check(lib.b200moe_forward(C.byref(p), C.byref(ws.struct), stream_ptr), "b200moe_forward")
    return output


@torch.no_grad()
def route(routing_logits, routing_bias, routed_scaling_factor, out=None):
    """Routing stage alone -> (topk_idx int32 [T,8], topk_weights float32 [T,8]); experts in descending biased score,
    ties to the lower id (reference: solution/python/pure_triton_impl.py:96-190).  Used by expert-parallel ranks, which
    route their own tokens before dispatch.  ``out`` = (idx, w) tensors to fill (their first T rows); needs no
    workspace (``b200moe_route_topk``)."""
    if not torch.is_tensor(routing_logits) or routing_logits.dim() != 2:
        raise ValueError("routing_logits must be [T, 256]")
    T = int(routing_logits.shape[0])
    logits = _require(routing_logits, "routing_logits", torch.float32, (T, E_GLOBAL))
    bias = _require(routing_bias.reshape(-1), "routing_bias", torch.bfloat16, (E_GLOBAL,))
    _require_cuda(routing_logits=logits, routing_bias=bias)
    device = logits.device
    if out is None:
        idx = torch.empty((T, TOP_K), dtype=torch.int32, device=device)
        w = torch.empty((T, TOP_K), dtype=torch.float32, device=device)
    else:
        idx, w = out
        if (idx.dtype != torch.int32 or w.dtype != torch.float32 or idx.shape[0] < T or w.shape[0] < T
                or tuple(idx.shape[1:]) != (TOP_K,) or tuple(w.shape[1:]) != (TOP_K,) or not idx.is_contiguous()
                or not w.is_contiguous() or idx.device != device or w.device != device):
            raise ValueError("out must be (int32 [>=T,8], float32 [>=T,8]) contiguous tensors on the logits' device")
        idx, w = idx[:T], w[:T]
    if T == 0:
        return idx, w
    with torch.cuda.device(device):
        _lib.check(_lib.load().b200moe_route_topk(logits.data_ptr(), bias.data_ptr(), T,
                                                  _host_scalar(routed_scaling_factor, float), idx.data_ptr(),
                                                  w.data_ptr(), torch.cuda.current_stream(device).cuda_stream),
                   "b200moe_route_topk")
    return idx, w


def check_status(device=None) -> None:
    """Synchronises the current stream and raises RuntimeError if any kernel since the last check recorded a failure
    (a bounded device-side wait that ran out).  The reference has no device-side waits and no such check."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = _devices.get(device.index)
    if st is None or st.active is None:
        return
    ws = st.carved[st.active]
    out = (C.c_int32 * 4)()
    with torch.cuda.device(device):
        rc = _lib.load().b200moe_read_status(C.byref(ws.struct), torch.cuda.current_stream(device).cuda_stream,
                                             C.byref(out))
    if rc == _lib.EDEVICE:
        st.active = None      # the next call re-runs b200moe_workspace_init: tile tickets may not be back at zero
        if st.mirror is not None:
            st.mirror.zero_()
        raise RuntimeError(f"device status word: code={out[0]} block={out[1]} role={out[2]} detail={out[3]}")
    _lib.check(rc, "b200moe_read_status")


def last_workspace(device=None) -> Optional[_Workspace]:
    """The workspace view used by the most recent call on ``device`` (tests read the sort metadata through it)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = _devices.get(device.index)
    if st is None or st.active is None:
        return None
    return st.carved[st.active]
