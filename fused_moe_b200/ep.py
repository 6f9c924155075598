"""Expert-parallel sharding of the 256 experts over G ranks (one process per GPU, torch.distributed).

The reference is single-GPU: its only hook for sharding is ``local_expert_offset``
(solution/python/pure_triton_impl.py:2141, masks at :248 and :505).  This module adds what a G-GPU deployment needs:

  rank r owns global experts [r*E_l, (r+1)*E_l), E_l = 256/G, and a slice of the tokens;
  1. every rank routes ITS tokens (all 256 logits are per token, the bias is replicated);
  2. dispatch: a token row (7168 e4m3 bytes + 56 scales + its 8 expert ids + 8 weights = 7456 bytes) goes once to
     every rank that owns at least one of its experts — group-limited routing bounds that by 4 ranks at G = 8;
  3. the receiver runs the layer on what arrived (``kernel_from_topk``: sort, gather, GEMM1+SwiGLU, GEMM2, reduce over
     ITS experts only), giving one partial row per received token, already weighted and summed over its experts;
  4. combine: fp32 partial rows return to the token's home rank, which adds them and rounds once to bf16.

Collectives go over NCCL (NVLink/NVSwitch); payloads land in local HBM before any kernel reads them.  Two classes share
the protocol: ``ExpertParallelMoE`` does the plumbing with torch ops around injected routing / expert callables, so it
also runs on CPU ranks (gloo) in the tests with the CPU oracle standing in; ``CudaExpertParallelMoE`` is the B200 shard,
where ranking, packing, the local experts and the final add are kernels of libb200moe.so.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

H = 7168
H_BLOCKS = 56
TOP_K = 8
E_GLOBAL = 256
ROW_BYTES = H + 4 * H_BLOCKS + 4 * TOP_K + 4 * TOP_K  # 7456, a multiple of 16


@dataclass
class DispatchPlan:
    """Who sends what: built on the home rank from its tokens' expert ids."""

    send_token: torch.Tensor      # [n_send] local token id of each outgoing row, grouped by destination rank
    send_splits: list             # rows per destination rank
    recv_splits: list             # rows per source rank


def plan_dispatch(topk_idx: torch.Tensor, world: int, group=None) -> DispatchPlan:
    """topk_idx [T,8] global expert ids -> rows to send, ordered by destination rank then token id.  The split sizes
    are exchanged with one small all_to_all and read back to the host (the collective needs them there)."""
    e_per_rank = E_GLOBAL // world
    T = topk_idx.shape[0]
    dest = topk_idx.long() // e_per_rank                                   # [T,8]
    hit = torch.zeros((T, world), dtype=torch.bool, device=topk_idx.device)
    hit.scatter_(1, dest, True)
    # nonzero of the transposed mask enumerates (rank, token) pairs rank-major with ascending token ids
    pairs = hit.t().nonzero(as_tuple=False)
    send_token = pairs[:, 1].contiguous()
    send_counts = hit.sum(dim=0).to(torch.int64)
    recv_counts = torch.empty_like(send_counts)
    if world > 1:
        dist.all_to_all_single(recv_counts, send_counts, group=group)
    else:
        recv_counts.copy_(send_counts)
    both = torch.stack([send_counts, recv_counts]).cpu()
    return DispatchPlan(send_token=send_token, send_splits=both[0].tolist(), recv_splits=both[1].tolist())


def pack_rows(tokens: torch.Tensor, hidden_states: torch.Tensor, hidden_states_scale: torch.Tensor,
              topk_idx: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
    """-> uint8 [n, 7456]: e4m3 row | 56 fp32 scales | 8 int32 expert ids | 8 fp32 weights, for the given tokens."""
    n = tokens.shape[0]
    buf = torch.empty((n, ROW_BYTES), dtype=torch.uint8, device=hidden_states.device)
    hs_u8 = hidden_states.view(torch.uint8)
    buf[:, :H] = hs_u8.index_select(0, tokens)
    scales = hidden_states_scale.t().index_select(0, tokens).contiguous()  # [n,56]
    buf[:, H:H + 224] = scales.view(torch.uint8).view(n, 224)
    buf[:, H + 224:H + 256] = topk_idx.to(torch.int32).index_select(0, tokens).contiguous().view(torch.uint8).view(n, 32)
    buf[:, H + 256:] = topk_w.index_select(0, tokens).contiguous().view(torch.uint8).view(n, 32)
    return buf


def unpack_rows(buf: torch.Tensor):
    """Inverse of pack_rows -> (hidden e4m3 [n,7168], scales [56,n] fp32, topk_idx [n,8] int32, topk_w [n,8] fp32)."""
    n = buf.shape[0]
    hs = buf[:, :H].contiguous().view(torch.float8_e4m3fn)
    scales = buf[:, H:H + 224].contiguous().view(torch.float32).view(n, H_BLOCKS).t().contiguous()
    idx = buf[:, H + 224:H + 256].contiguous().view(torch.int32).view(n, TOP_K)
    w = buf[:, H + 256:].contiguous().view(torch.float32).view(n, TOP_K)
    return hs, scales, idx, w


def _a2a(send: torch.Tensor, send_splits, recv_splits, world: int, group) -> torch.Tensor:
    recv = torch.empty((sum(recv_splits),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    if world > 1:
        dist.all_to_all_single(recv, send, output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
    else:
        recv.copy_(send)
    return recv


class ExpertParallelMoE:
    """One rank's shard of the layer.

    route_fn(logits [T,256], bias [256], scale) -> (topk_idx int32 [T,8], topk_w fp32 [T,8])
    expert_fn(topk_idx [n,8], topk_w [n,8], hidden e4m3 [n,7168], scales [56,n]) -> partial rows fp32 [n,7168]
              (sum over THIS rank's experts of weight * expert output; zeros where none is local).  Partials stay in
              fp32 until the home rank has added them: rounding each shard's share to bf16 first costs accuracy.
    """

    def __init__(self, route_fn: Callable, expert_fn: Callable, rank: int, world: int, group=None):
        if E_GLOBAL % world:
            raise ValueError(f"world size {world} does not divide {E_GLOBAL} experts")
        self.route_fn, self.expert_fn = route_fn, expert_fn
        self.rank, self.world, self.group = rank, world, group
        self.e_local = E_GLOBAL // world
        self.last_plan: Optional[DispatchPlan] = None
        self.last_recv = None  # (topk_idx, topk_w, hidden, scales) of the rows this rank received last

    @property
    def local_expert_offset(self) -> int:
        return self.rank * self.e_local

    @torch.no_grad()
    def forward(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, routed_scaling_factor,
                output: Optional[torch.Tensor] = None) -> torch.Tensor:
        T = routing_logits.shape[0]
        topk_idx, topk_w = self.route_fn(routing_logits, routing_bias, routed_scaling_factor)
        plan = plan_dispatch(topk_idx, self.world, self.group)
        self.last_plan = plan
        send = pack_rows(plan.send_token, hidden_states, hidden_states_scale, topk_idx, topk_w)
        recv = _a2a(send, plan.send_splits, plan.recv_splits, self.world, self.group)
        hs, scales, idx, w = unpack_rows(recv)
        self.last_recv = (idx, w, hs, scales)
        partial = self.expert_fn(idx, w, hs, scales)
        back = _a2a(partial, plan.recv_splits, plan.send_splits, self.world, self.group)
        acc = torch.zeros((T, H), dtype=torch.float32, device=hidden_states.device)
        acc.index_add_(0, plan.send_token, back.float())  # back is fp32 already on the CUDA path
        if output is None:
            return acc.to(torch.bfloat16)
        output.copy_(acc)
        return output


class CudaExpertParallelMoE:
    """One rank's shard on a B200, everything on the device done by libb200moe.so: routing, the stable ranking of
    (token, destination) pairs and record packing (``b200moe_ep_dispatch``), the local experts reading the received
    records in place (``kernel_from_records``) and the final add (``b200moe_ep_combine``).  torch.distributed only moves
    bytes: one all_gather of the G x G record counts (read back to the host, which NCCL needs for the split sizes) and
    one all_to_all_single per direction."""

    def __init__(self, weights: dict, rank: int, world: int, group=None, transport: str = "auto"):
        """transport: "peer" — records and partial rows are stored straight into the destination GPU's memory by the
        pack and reduce kernels (torch symmetric memory supplies the mapped buffers; up to 8 GPUs of one node), with a
        bounded flag barrier between phases and no payload collective; "nccl" — two all_to_all_single; "auto" — peer
        when it can be set up, else nccl."""
        if E_GLOBAL % world:
            raise ValueError(f"world size {world} does not divide {E_GLOBAL} experts")
        if transport not in ("auto", "peer", "nccl"):
            raise ValueError("transport must be 'auto', 'peer' or 'nccl'")
        self.weights, self.rank, self.world, self.group = weights, rank, world, group
        self.transport = "nccl" if (world == 1 or world > 8) else transport
        self._peer = None          # symmetric-memory state of the peer transport
        self._epoch = 0
        self.e_local = E_GLOBAL // world
        self.local_expert_offset = rank * self.e_local
        self._buf = {}
        self.last_records = None   # records this rank received in the last call (uint8 [n, 7456])
        self.last_splits = None    # (send_splits, recv_splits) of the last call
        self.profile = False       # True: record CUDA events around each phase, read them with phase_times()
        self._events = []

    def _mark(self, name):
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._events.append((name, ev))

    def phase_times(self):
        """us per phase of the last profiled call (synchronises)."""
        torch.cuda.synchronize()
        out = {}
        for (_, a), (name, b) in zip(self._events[:-1], self._events[1:]):
            out[name] = a.elapsed_time(b) * 1e3
        return out

    def _peer_setup(self, T: int, device):
        """Maps one slab per rank into every rank: [flags | receive records | returned partial rows].  Collective."""
        import ctypes as C
        import os
        from . import _lib
        if self._peer is not None and self._peer["T"] >= T:
            return self._peer
        # plain peer mappings only: no NVLink multicast object is bound to these buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        cap_recv = self.world * T                      # every token of every rank may come here
        cap_back = T * min(TOP_K, self.world)          # one returned row per (token, destination)
        off_recv = 256
        off_back = off_recv + (cap_recv * ROW_BYTES + 255) // 256 * 256
        total = off_back + cap_back * H * 4
        slab = symm_mem.empty(total, dtype=torch.uint8, device=device)
        slab[:256].zero_()
        group = self.group if self.group is not None else dist.group.WORLD
        hdl = symm_mem.rendezvous(slab, group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        peers = _lib.EpPeers()
        peers.world, peers.rank = self.world, self.rank
        for r in range(self.world):
            peers.flags[r] = ptrs[r]
            peers.recv_records[r] = ptrs[r] + off_recv
        status = torch.zeros(4, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)                 # flags are zero everywhere before the first epoch
        self._peer = dict(T=T, slab=slab, hdl=hdl, ptrs=ptrs, peers=peers, off_recv=off_recv, off_back=off_back,
                          cap_recv=cap_recv, cap_back=cap_back, status=status)
        return self._peer

    def check_status(self):
        """Raises if a bounded peer barrier ran out since the last check (synchronises)."""
        if self._peer is None:
            return
        st = self._peer["status"].cpu().tolist()
        if st[0] != 0:
            self._peer["status"].zero_()
            raise RuntimeError(f"expert-parallel barrier timed out: code={st[0]} rank={st[1]} waiting_for={st[2]} "
                               f"epoch={st[3]}")

    def _barrier(self, stream):
        import ctypes as C
        from . import _lib
        self._epoch += 1
        _lib.check(_lib.load().b200moe_ep_barrier(C.byref(self._peer["peers"]), self._epoch,
                                                  self._peer["status"].data_ptr(), stream), "b200moe_ep_barrier")

    def _buffers(self, T: int, device):
        import ctypes as C
        from . import _lib
        key = (T, device.index)
        b = self._buf.get(key)
        if b is None:
            n = C.c_size_t(0)
            _lib.check(_lib.load().b200moe_ep_scratch_bytes(T, self.world, C.byref(n)), "b200moe_ep_scratch_bytes")
            cap = T * min(TOP_K, self.world)
            b = dict(scratch=torch.empty(max(n.value, 256), dtype=torch.uint8, device=device), scratch_bytes=n.value,
                     send=torch.empty((max(cap, 1), ROW_BYTES), dtype=torch.uint8, device=device),
                     counts=torch.zeros(self.world, dtype=torch.int32, device=device),
                     slot_map=torch.empty((max(T, 1), TOP_K), dtype=torch.int32, device=device),
                     all_counts=torch.empty(self.world * self.world, dtype=torch.int32, device=device))
            self._buf = {key: b}
        return b

    @torch.no_grad()
    def forward(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, routed_scaling_factor,
                output: Optional[torch.Tensor] = None) -> torch.Tensor:
        import ctypes as C
        from . import _lib
        from . import kernel as K
        lib = _lib.load()
        T = routing_logits.shape[0]
        device = hidden_states.device
        if output is None:
            output = torch.empty((T, H), dtype=torch.bfloat16, device=device)
        self._events = []
        self._mark("start")
        idx, w = K.route(routing_logits, routing_bias, routed_scaling_factor)
        self._mark("route")
        if self.transport in ("auto", "peer"):
            try:
                self._peer_setup(T, device)
                self.transport = "peer"
            except Exception:
                if self.transport == "peer":
                    raise
                self.transport = "nccl"   # symmetric memory is not available here: fall back to the collective path
        if self.transport == "peer":
            return self._forward_peer(idx, w, hidden_states, hidden_states_scale, output, T, device)
        b = self._buffers(T, device)
        hs = hidden_states if hidden_states.is_contiguous() else hidden_states.contiguous()
        hss = hidden_states_scale if hidden_states_scale.is_contiguous() else hidden_states_scale.contiguous()
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            _lib.check(lib.b200moe_ep_dispatch(idx.data_ptr(), w.data_ptr(), hs.data_ptr(), hss.data_ptr(), T,
                                               self.world, b["scratch"].data_ptr(), b["scratch_bytes"],
                                               b["send"].data_ptr(), b["counts"].data_ptr(), b["slot_map"].data_ptr(),
                                               stream), "b200moe_ep_dispatch")
        self._mark("dispatch_kernels")
        if self.world > 1:
            dist.all_gather_into_tensor(b["all_counts"], b["counts"], group=self.group)
            m = b["all_counts"].cpu().view(self.world, self.world)
        else:
            m = b["counts"].cpu().view(1, 1)
        send_splits, recv_splits = m[self.rank].tolist(), m[:, self.rank].tolist()
        n_send, n_recv = sum(send_splits), sum(recv_splits)
        send = b["send"][:n_send]
        self._mark("counts_exchange_and_host_read")
        if self.world > 1:
            recv = torch.empty((n_recv, ROW_BYTES), dtype=torch.uint8, device=device)
            dist.all_to_all_single(recv, send, recv_splits, send_splits, group=self.group)
        else:
            recv = send
        self.last_records, self.last_splits = recv, (send_splits, recv_splits)
        self._mark("all_to_all_records")
        wts = self.weights
        part = K.kernel_from_records(recv, wts["gemm1_weights"], wts["gemm1_weights_scale"], wts["gemm2_weights"],
                                     wts["gemm2_weights_scale"], self.local_expert_offset)
        self._mark("local_experts")
        if self.world > 1:
            back = torch.empty((n_send, H), dtype=torch.float32, device=device)
            dist.all_to_all_single(back, part, send_splits, recv_splits, group=self.group)
        else:
            back = part
        self._mark("all_to_all_partials")
        if T > 0:
            with torch.cuda.device(device):
                stream = torch.cuda.current_stream(device).cuda_stream
                if n_send == 0:
                    output.zero_()
                else:
                    _lib.check(lib.b200moe_ep_combine(back.data_ptr(), b["slot_map"].data_ptr(), T, output.data_ptr(),
                                                      stream), "b200moe_ep_combine")
        self._mark("combine")
        return output


    def _forward_peer(self, idx, w, hidden_states, hidden_states_scale, output, T, device):
        import ctypes as C
        from . import _lib
        from . import kernel as K
        lib = _lib.load()
        pr = self._peer
        b = self._buffers(T, device)
        hs = hidden_states if hidden_states.is_contiguous() else hidden_states.contiguous()
        hss = hidden_states_scale if hidden_states_scale.is_contiguous() else hidden_states_scale.contiguous()
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            _lib.check(lib.b200moe_ep_rank(idx.data_ptr(), T, self.world, b["scratch"].data_ptr(), b["scratch_bytes"],
                                           b["counts"].data_ptr(), b["slot_map"].data_ptr(), stream),
                       "b200moe_ep_rank")
            self._mark("dispatch_kernels")
            dist.all_gather_into_tensor(b["all_counts"], b["counts"], group=self.group)
            m = b["all_counts"].cpu().view(self.world, self.world).tolist()   # m[s][d] = records s sends to d
            self._mark("counts_exchange_and_host_read")
            me = self.rank
            send_splits, recv_splits = m[me], [m[s_rank][me] for s_rank in range(self.world)]
            n_send, n_recv = sum(send_splits), sum(recv_splits)
            self.last_splits = (send_splits, recv_splits)
            # my segment in rank d's receive buffer starts after the segments of the ranks before me
            row0 = (C.c_int32 * self.world)(*[sum(m[s_rank][d] for s_rank in range(me)) for d in range(self.world)])
            _lib.check(lib.b200moe_ep_pack_peers(idx.data_ptr(), w.data_ptr(), hs.data_ptr(), hss.data_ptr(), T,
                                                 C.byref(pr["peers"]), row0, b["scratch"].data_ptr(),
                                                 b["scratch_bytes"], stream), "b200moe_ep_pack_peers")
            self._barrier(stream)
            self._mark("records_to_peers")
            recv = pr["slab"][pr["off_recv"]:pr["off_recv"] + n_recv * ROW_BYTES].view(n_recv, ROW_BYTES)
            self.last_records = recv
            # rows received from source s return to s's slab, after the rows s sent to the ranks before me
            starts, bases, acc = [0], [], 0
            for s_rank in range(self.world):
                acc += recv_splits[s_rank]
                starts.append(acc)
                bases.append(pr["ptrs"][s_rank] + pr["off_back"] + sum(m[s_rank][:me]) * H * 4)
            wts = self.weights
            K.kernel_from_records(recv, wts["gemm1_weights"], wts["gemm1_weights_scale"], wts["gemm2_weights"],
                                  wts["gemm2_weights_scale"], self.local_expert_offset, out_segments=(starts, bases))
            self._mark("local_experts_and_rows_to_peers")
            self._barrier(stream)
            self._mark("barrier")
            if output is None:
                output = torch.empty((T, H), dtype=torch.bfloat16, device=device)
            if T > 0:
                if n_send == 0:
                    output.zero_()
                else:
                    back_ptr = pr["ptrs"][me] + pr["off_back"]
                    _lib.check(lib.b200moe_ep_combine(back_ptr, b["slot_map"].data_ptr(), T, output.data_ptr(), stream),
                               "b200moe_ep_combine")
            self._mark("combine")
        return output


def make_cuda_shard(weights: dict, rank: int, world: int, group=None, transport: str = "auto") -> CudaExpertParallelMoE:
    """Shard backed by libb200moe.so: ``weights`` holds this rank's gemm1/gemm2 weights and scales (E_l experts)."""
    return CudaExpertParallelMoE(weights, rank, world, group, transport)
