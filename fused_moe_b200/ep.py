"""Expert-parallel sharding of the 256 experts over G ranks (one process per GPU, torch.distributed).

The reference is single-GPU: its only hook for sharding is ``local_expert_offset``
(solution/python/pure_triton_impl.py:2141, masks at :248 and :505).  This module adds what a G-GPU deployment needs:

  rank r owns global experts [r*E_l, (r+1)*E_l), E_l = 256/G, and a slice of the tokens;
  1. every rank routes ITS tokens (all 256 logits are per token, the bias is replicated);
  2. dispatch: a token row (7168 e4m3 bytes + 56 scales + its 8 expert ids + 8 weights = 7456 bytes) goes once to
     every rank that owns at least one of its experts — group-limited routing bounds that by 4 ranks at G = 8;
  3. the receiver runs the layer on what arrived (``kernel_from_topk``: sort, gather, GEMM1+SwiGLU, GEMM2, reduce over
     ITS experts only), giving one partial row per received token, already weighted and summed over its experts;
  4. combine: un-rounded partial rows (float32, or eight float16 per power-of-two scale byte) return to the token's
     home rank, which adds them and rounds once to bf16.

Payloads cross NVLink/NVSwitch either as plain peer stores from the pack and reduce kernels or as NCCL collectives;
either way they land in local HBM before any kernel reads them.  Two classes share
the protocol: ``ExpertParallelMoE`` does the plumbing with torch ops around injected routing / expert callables, so it
also runs on CPU ranks (gloo) in the tests with the CPU oracle standing in; ``CudaExpertParallelMoE`` is the B200 shard,
where ranking, packing, the local experts and the final add are kernels of libb200moe.so.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import os

# plain peer mappings only: no NVLink multicast object may ever be bound to the buffers of this module; the switch is
# read by torch's symmetric memory when it is first used, so it is set before anything can import that
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

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
    (token, destination) pairs, record packing, the local experts reading the received records in place and the final
    add.  Two transports:

    "peer" (default up to 8 GPUs of one node): one slab per rank — flags, count matrix, receive records, returned
    partial rows — is mapped into every rank (torch symmetric memory, plain peer mappings, no multicast).  A step is
    route -> rank -> count exchange + barrier -> pack (records stored straight into the destinations' slabs) -> barrier
    -> the layer on the received records, its last kernel storing each partial row straight into the home rank's
    slab -> barrier -> combine.  The counts never reach the host: ``b200moe_ep_exchange_counts`` leaves a plan in device
    memory that the following kernels read, so a step has NO host synchronisation and no collective call.

    "nccl": the records and the partial rows travel with two ``all_to_all_single``; the counts are all-gathered and read
    back to the host, which the collective needs for its split sizes.

    Capacity: the slab is sized at the first call for ``T_cap`` tokens per rank — the maximum over the ranks of the
    batch they bring to that call and of ``max_tokens_per_rank`` — so every rank may later bring any batch up to
    ``T_cap``; a larger batch raises ValueError on the rank that brings it (create the shard with a larger
    ``max_tokens_per_rank``).  The device re-checks the exchanged counts against the buffer sizes before anything is
    stored into a peer (status code 3)."""

    HDR_FLAGS, HDR_COUNTS, HDR_BYTES = 0, 256, 1024

    def __init__(self, weights: dict, rank: int, world: int, group=None, transport: str = "auto",
                 max_tokens_per_rank: Optional[int] = None, partial_rows: Optional[str] = None):
        if E_GLOBAL % world:
            raise ValueError(f"world size {world} does not divide {E_GLOBAL} experts")
        if transport not in ("auto", "peer", "nccl"):
            raise ValueError("transport must be 'auto', 'peer' or 'nccl'")
        if partial_rows not in (None, "float", "half"):
            raise ValueError("partial_rows must be 'float', 'half' or None")
        self.weights, self.rank, self.world, self.group = weights, rank, world, group
        # Form of the partial rows a shard returns to the tokens' home ranks: float32 (28672 bytes per row) or the
        # half form of b200moe_problem.partial_format (15232 bytes: eight float16 per power-of-two scale byte).  The
        # return is the larger of the two exchanges of a step and is bound by NVLink, so more than one rank defaults
        # to the half form (every rank must choose the same); a single rank sends nothing and keeps float32.
        self.half_rows = (partial_rows == "half") if partial_rows is not None else world > 1
        # more than 8 ranks span several nodes: collectives only; one rank needs no transport at all, "auto" then takes
        # the shorter collective-free nccl branch and an explicit "peer" runs the peer protocol on a local slab
        self.transport = "nccl" if (world > 8 or (world == 1 and transport == "auto")) else transport
        self.max_tokens_per_rank = max_tokens_per_rank
        self._peer = None          # symmetric-memory state of the peer transport
        self._epoch = 0
        self.e_local = E_GLOBAL // world
        self.local_expert_offset = rank * self.e_local
        self._buf = {}
        self._records = None       # nccl transport: records received in the last call
        self._splits = None
        self.profile = False       # True: record CUDA events around each phase, read them with phase_times()
        self._events = []

    # ------------------------------------------------------------------ bookkeeping
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

    def read_plan(self):
        """The device-side plan of the last peer-transport call as a ``_lib.EpPlan`` (synchronises; for tests, tools
        and statistics — the step itself never reads it on the host)."""
        from . import _lib
        if self._peer is None:
            return None
        torch.cuda.synchronize()
        raw = bytes(self._peer["plan"].cpu().numpy().tobytes())
        import ctypes as C
        return _lib.EpPlan.from_buffer_copy(raw[:C.sizeof(_lib.EpPlan)])

    @property
    def last_splits(self):
        """(records sent per destination rank, records received per source rank) of the last call (synchronises)."""
        if self.transport != "peer" or self._peer is None:
            return self._splits
        pl = self.read_plan()
        m = [[pl.matrix[s_rank * 8 + d] for d in range(self.world)] for s_rank in range(self.world)]
        return m[self.rank], [m[s_rank][self.rank] for s_rank in range(self.world)]

    @property
    def last_records(self):
        """The records this rank received in the last call, uint8 [n, 7456] (synchronises on the peer transport)."""
        if self.transport != "peer" or self._peer is None:
            return self._records
        n = self.read_plan().n_recv
        return self._peer["recv"][:n]

    # ------------------------------------------------------------------ set-up
    def _agree(self, value: int, op, device) -> int:
        t = torch.tensor([value], dtype=torch.int64, device=device)
        if self.world > 1:
            dist.all_reduce(t, op=op, group=self.group)
        return int(t.item())

    def _peer_setup(self, T: int, device):
        """First call only, collective: agrees on the capacity and on whether every rank can use peer memory, then maps
        one slab per rank into every rank: [flags | count matrix | receive records | returned partial rows]."""
        import os
        from . import _lib
        if self._peer is not None:
            if T > self._peer["T_cap"]:
                raise ValueError(f"{T} tokens exceed the {self._peer['T_cap']} per rank the expert-parallel buffers were "
                                 "sized for at the first call; create the shard with max_tokens_per_rank")
            return self._peer
        T_cap = self._agree(max(T, self.max_tokens_per_rank or 0, 1), dist.ReduceOp.MAX, device)
        # plain peer mappings only: no NVLink multicast object is bound to these buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        cap_recv = self.world * T_cap                      # every token of every rank may come here
        cap_back = T_cap * min(TOP_K, self.world)          # one returned row per (token, destination)
        off_recv = self.HDR_BYTES
        off_back = off_recv + (cap_recv * ROW_BYTES + 255) // 256 * 256
        back_row_bytes = _lib.HALF_ROW_BYTES if self.half_rows else H * 4
        total = off_back + cap_back * back_row_bytes
        slab, err, hdl = None, None, None
        if self.world == 1:
            slab = torch.empty(total, dtype=torch.uint8, device=device)   # the only "peer" is this rank itself
            slab[:self.HDR_BYTES].zero_()
            ptrs = [slab.data_ptr()]
        else:
            try:
                import torch.distributed._symmetric_memory as symm_mem
                slab = symm_mem.empty(total, dtype=torch.uint8, device=device)
            except Exception as exc:   # no symmetric memory on this build / device
                err = exc
            # every rank takes the same branch: the rendezvous below is collective
            if self._agree(0 if slab is None else 1, dist.ReduceOp.MIN, device) == 0:
                raise RuntimeError(f"peer transport unavailable on at least one rank ({err!r})")
            slab[:self.HDR_BYTES].zero_()
            group = self.group if self.group is not None else dist.group.WORLD
            hdl = symm_mem.rendezvous(slab, group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
        peers = _lib.EpPeers()
        peers.world, peers.rank, peers.cap_recv, peers.cap_back = self.world, self.rank, cap_recv, cap_back
        peers.back_row_bytes = back_row_bytes
        for r in range(self.world):
            peers.flags[r] = ptrs[r] + self.HDR_FLAGS
            peers.counts[r] = ptrs[r] + self.HDR_COUNTS
            peers.recv_records[r] = ptrs[r] + off_recv
            peers.back_rows[r] = ptrs[r] + off_back
        status = torch.zeros(4, dtype=torch.int32, device=device)
        plan = torch.zeros(512, dtype=torch.uint8, device=device)
        torch.cuda.synchronize(device)
        if self.world > 1:
            dist.barrier(group=self.group)             # flags are zero everywhere before the first epoch
        self._peer = dict(T_cap=T_cap, slab=slab, hdl=hdl, ptrs=ptrs, peers=peers, off_recv=off_recv, off_back=off_back,
                          cap_recv=cap_recv, cap_back=cap_back, status=status, plan=plan,
                          status_host=torch.zeros(4, dtype=torch.int32).pin_memory(),
                          recv=slab[off_recv:off_recv + cap_recv * ROW_BYTES].view(cap_recv, ROW_BYTES))
        self._peer["status_np"] = self._peer["status_host"].numpy()
        return self._peer

    def _choose_transport(self, T: int, device):
        """Settles "auto" at the first call, the same way on every rank."""
        if self.transport == "nccl" or self._peer is not None:
            return
        if self.transport == "peer":
            self._peer_setup(T, device)
            return
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
            have = 1
        except Exception:
            have = 0
        if self._agree(have, dist.ReduceOp.MIN, device) == 0:
            self.transport = "nccl"
            return
        try:
            self._peer_setup(T, device)
            self.transport = "peer"
        except RuntimeError:
            self.transport = "nccl"    # raised on every rank alike (the decision inside _peer_setup is collective)

    def check_status(self):
        """Raises if a bounded peer wait ran out or the exchanged counts did not fit since the last check
        (synchronises)."""
        if self._peer is None:
            return
        st = self._peer["status"].cpu().tolist()
        if st[0] != 0:
            self._peer["status"].zero_()
            self._peer["status_np"][:] = 0
            raise RuntimeError(self._status_text(st))

    @staticmethod
    def _status_text(st):
        if st[0] == 4:
            return (f"expert-parallel kernel refused a destination address: where={st[1]} row={st[2]} "
                    f"address bits={st[3]:#x}")
        if st[0] == 3:
            return (f"expert-parallel counts exceed the buffers: rank={st[1]} receive capacity={st[2]} "
                    f"return capacity={st[3]} (do all ranks pass batches within the agreed capacity?)")
        return f"expert-parallel barrier timed out: code={st[0]} rank={st[1]} waiting_for={st[2]} epoch={st[3]}"

    def _barrier(self, stream):
        import ctypes as C
        from . import _lib
        self._epoch += 1
        _lib.check(_lib.load().b200moe_ep_barrier(C.byref(self._peer["peers"]), self._epoch,
                                                  self._peer["status"].data_ptr(), stream), "b200moe_ep_barrier")

    def _buffers(self, T: int, device):
        """Rank-local buffers, sized once for the capacity (peer transport) or per batch size (nccl)."""
        import ctypes as C
        from . import _lib
        cap_T = self._peer["T_cap"] if self._peer is not None else T
        key = (cap_T, device.index)
        b = self._buf.get(key)
        if b is None:
            n = C.c_size_t(0)
            _lib.check(_lib.load().b200moe_ep_scratch_bytes(cap_T, self.world, C.byref(n)), "b200moe_ep_scratch_bytes")
            cap = cap_T * min(TOP_K, self.world)
            b = dict(scratch=torch.empty(max(n.value, 256), dtype=torch.uint8, device=device), scratch_bytes=n.value,
                     counts=torch.zeros(self.world, dtype=torch.int32, device=device),
                     slot_map=torch.empty((max(cap_T, 1), TOP_K), dtype=torch.int32, device=device),
                     idx=torch.empty((max(cap_T, 1), TOP_K), dtype=torch.int32, device=device),
                     w=torch.empty((max(cap_T, 1), TOP_K), dtype=torch.float32, device=device),
                     all_counts=torch.empty(self.world * self.world, dtype=torch.int32, device=device))
            if self._peer is None:
                b["send"] = torch.empty((max(cap, 1), ROW_BYTES), dtype=torch.uint8, device=device)
            self._buf = {key: b}
        return b

    # ------------------------------------------------------------------ the step
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
        self._choose_transport(T, device)
        if self.transport == "peer":
            self._peer_setup(T, device)    # capacity check only after the first call
            np_status = self._peer["status_np"]
            if np_status[0] != 0:          # copied at the end of an earlier call: no synchronisation here
                st = [int(x) for x in np_status]
                np_status[:] = 0
                self._peer["status"].zero_()
                raise RuntimeError(self._status_text(st) + "; the output of that call is invalid")
        b = self._buffers(T, device)
        self._events = []
        self._mark("start")
        idx, w = K.route(routing_logits, routing_bias, routed_scaling_factor, out=(b["idx"], b["w"]))
        self._mark("route")
        hs = hidden_states if hidden_states.is_contiguous() else hidden_states.contiguous()
        hss = hidden_states_scale if hidden_states_scale.is_contiguous() else hidden_states_scale.contiguous()
        if self.transport == "peer":
            return self._forward_peer(idx, w, hs, hss, output, T, device, b)
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
        self._records, self._splits = recv, (send_splits, recv_splits)
        self._mark("all_to_all_records")
        wts = self.weights
        part = K.kernel_from_records(recv, wts["gemm1_weights"], wts["gemm1_weights_scale"], wts["gemm2_weights"],
                                     wts["gemm2_weights_scale"], self.local_expert_offset, half_rows=self.half_rows)
        self._mark("local_experts")
        if self.world > 1:
            back = torch.empty((n_send,) + tuple(part.shape[1:]), dtype=part.dtype, device=device)
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
                    combine = lib.b200moe_ep_combine_half if self.half_rows else lib.b200moe_ep_combine
                    _lib.check(combine(back.data_ptr(), b["slot_map"].data_ptr(), T, output.data_ptr(), stream),
                               "b200moe_ep_combine")
        self._mark("combine")
        return output

    @torch.no_grad()
    def forward_host(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, routed_scaling_factor,
                     output: Optional[torch.Tensor] = None, slices: Optional[int] = None,
                     ready_event=None) -> torch.Tensor:
        """``forward`` for a rank whose tokens live in HOST memory: ``routing_logits``, ``hidden_states``,
        ``hidden_states_scale`` and ``output`` are pinned host tensors (``output=None`` allocates one); the bias is a
        device tensor.  The rank's tokens are cut into ``slices`` equal runs and every run is one complete
        expert-parallel step (so EVERY rank must pass the same ``slices``; default 2, or 1 with ``ready_event``, when
        the overlap comes from the neighbouring calls); the host-to-device copy of run i + 1 and the
        device-to-host copy of run i - 1 go over two side streams and overlap the step on run i.  Rows are independent,
        so the result equals one ``forward`` on all tokens.  Returns ``output`` after queueing everything: the caller's
        current stream waits for the last copy, unless ``ready_event`` is given — then that event is recorded after the
        last copy-out, nothing waits for it, and consecutive calls overlap their copies with each other's steps
        (see ``fused_moe_b200.kernel.kernel_host``)."""
        from . import kernel as K
        for name, t in (("routing_logits", routing_logits), ("hidden_states", hidden_states),
                        ("hidden_states_scale", hidden_states_scale)):
            if not torch.is_tensor(t) or t.is_cuda or (t.numel() > 0 and not t.is_pinned()):   # empty: nothing to pin
                raise RuntimeError(f"{name} must be a pinned host tensor")
        T = int(routing_logits.shape[0])
        device = routing_bias.device
        if output is None:
            output = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
        if slices is None:
            slices = 1 if (ready_event is not None or T < 2) else 2
        if slices < 1 or (T > 0 and slices > T):
            raise ValueError("slices must be in 1..T")
        if T == 0:
            if ready_event is not None:
                ready_event.record(torch.cuda.current_stream(device))
            return output

        def layer(logits_dev, hs_dev, scale_dev, out_dev):
            self.forward(logits_dev, routing_bias, hs_dev, scale_dev, routed_scaling_factor, out_dev)

        with torch.cuda.device(device):
            pipe = K.HostPipe.get(self.__dict__, "_host_pipe", device, T, (T + slices - 1) // slices)
            return pipe.run(layer, routing_logits, hidden_states, hidden_states_scale, output, slices, ready_event)

    def _forward_peer(self, idx, w, hs, hss, output, T, device, b):
        """Peer transport: nothing below waits for the device or calls a collective."""
        import ctypes as C
        from . import _lib
        from . import kernel as K
        lib = _lib.load()
        pr = self._peer
        peers = C.byref(pr["peers"])
        plan = pr["plan"].data_ptr()
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            _lib.check(lib.b200moe_ep_rank(idx.data_ptr(), T, self.world, b["scratch"].data_ptr(), b["scratch_bytes"],
                                           b["counts"].data_ptr(), b["slot_map"].data_ptr(), stream),
                       "b200moe_ep_rank")
            self._mark("rank_pairs")
            self._epoch += 1
            _lib.check(lib.b200moe_ep_exchange_counts(peers, b["counts"].data_ptr(), self._epoch, plan,
                                                      pr["status"].data_ptr(), stream), "b200moe_ep_exchange_counts")
            self._mark("count_exchange")
            _lib.check(lib.b200moe_ep_pack_peers_planned(idx.data_ptr(), w.data_ptr(), hs.data_ptr(), hss.data_ptr(),
                                                         T, peers, plan, b["scratch"].data_ptr(), b["scratch_bytes"],
                                                         pr["status"].data_ptr(), stream),
                       "b200moe_ep_pack_peers_planned")
            self._barrier(stream)
            self._mark("records_to_peers")
            wts = self.weights
            K.kernel_from_records(pr["recv"], wts["gemm1_weights"], wts["gemm1_weights_scale"], wts["gemm2_weights"],
                                  wts["gemm2_weights_scale"], self.local_expert_offset, plan=plan,
                                  half_rows=self.half_rows)
            self._mark("local_experts_and_rows_to_peers")
            self._barrier(stream)
            self._mark("barrier")
            if T > 0:
                back_ptr = pr["ptrs"][self.rank] + pr["off_back"]
                combine = lib.b200moe_ep_combine_half if self.half_rows else lib.b200moe_ep_combine
                _lib.check(combine(back_ptr, b["slot_map"].data_ptr(), T, output.data_ptr(), stream),
                           "b200moe_ep_combine")
            self._mark("combine")
            # the status word follows the step to pinned host memory; the next call looks at it before it starts
            pr["status_host"].copy_(pr["status"], non_blocking=True)
        return output


def make_cuda_shard(weights: dict, rank: int, world: int, group=None, transport: str = "auto",
                    max_tokens_per_rank: Optional[int] = None,
                    partial_rows: Optional[str] = None) -> CudaExpertParallelMoE:
    """Shard backed by libb200moe.so: ``weights`` holds this rank's gemm1/gemm2 weights and scales (E_l experts);
    ``partial_rows`` = "float" | "half" | None (half when world > 1) is the form in which partial rows return."""
    return CudaExpertParallelMoE(weights, rank, world, group, transport, max_tokens_per_rank, partial_rows)
