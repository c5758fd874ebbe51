"""Expert-parallel MoE layer: experts split evenly over ranks, tokens data-sharded, NCCL
all-to-all for dispatch and combine (torch.distributed is the plumbing; every compute step is a
C-ABI launch).  gem16 has no multi-GPU code; the protocol below is this library's.

Per layer, on every rank (T local tokens, R ranks, E experts, E/R local experts [r*E/R, (r+1)*E/R)):
  1. route the local tokens over all E experts (router replicated): ids, weights, counts,
     offsets and the stable permutation -- which orders assignments by expert, hence by owner rank;
  2. NVFP4-quantise the local tokens once and pack payload + scales + local expert id into one
     message row per assignment, in permutation order (1,600 B instead of 5,632 B of bf16);
  3. all-gather the per-expert counts (the only host read-back: the split sizes), all-to-all the
     packed rows;
  4. the owner sorts what it received by local expert with the same stable permutation kernel --
     arrival order is (source rank, expert, token, slot), so the result is (expert, global token,
     slot), exactly the single-GPU order -- scatters into the padded row space and runs the
     grouped gate_up GEMM, GELU requantisation and grouped down GEMM;
  5. expert outputs go back in arrival order through the reverse all-to-all, and each token's
     owner combines its topk contributions in slot order and adds its shared branch.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .lib import load
from .moe import MoeLayer, MoeWeights


def ep_splits(counts_all, rank: int, experts_per_rank: int):
    """Split sizes of the dispatch all-to-all from the gathered per-expert counts [R, E]:
    (rows this rank sends to each rank, rows it receives from each rank)."""
    ranks = counts_all.shape[0]
    per_owner = counts_all.reshape(ranks, ranks, experts_per_rank).sum(-1)   # [source, owner]
    return [int(v) for v in per_owner[rank]], [int(v) for v in per_owner[:, rank]]


class EpMoeLayer:
    """Buffers and launch sequence of one expert-parallel layer for `tokens` local tokens."""

    def __init__(self, weights: MoeWeights, tokens: int, topk: int, ga: float, ga_dn: float, ga_sh_dn: float,
                 group=None):
        self.lib = load()
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.w, self.tokens, self.topk = weights, tokens, topk
        self.ga, self.ga_dn = ga, ga_dn
        lib, dev, w, c = self.lib, weights.dev, weights, self.lib.cdll
        self.e_total, self.e_local = w.router_experts, w.experts
        assert self.e_local * self.world == self.e_total
        h, i, n = w.hidden, w.inter, tokens * topk
        # the local half (routing, shared branch, combine) reuses the single-GPU layer's buffers
        self.local = MoeLayer(weights, tokens, topk, ga, ga_dn, ga_sh_dn, allocate_experts=False)
        cap = n * self.world                      # worst case: every assignment of every rank lands here
        self.cap = cap
        u8 = dict(dtype=torch.uint8, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        self.xq = torch.empty((tokens, h // 2), **u8)
        self.xs = torch.empty((tokens, h // 16), **u8)
        # One dispatch message row per assignment: payload | block scales | local expert id | pad.
        self.msg_bytes = (h // 2 + h // 16 + 4 + 15) // 16 * 16
        self.send_msg = torch.zeros((n, self.msg_bytes), **u8)
        self.recv_msg = torch.empty((cap, self.msg_bytes), **u8)
        self.recv_eid = torch.empty((cap,), **i32)
        self.counts_all = torch.empty((self.world, self.e_total), **i32)
        self.rows_max = c.gemb_moe_padded_rows_max(cap, self.e_local, 1)
        self.l_counts = torch.empty((self.e_local,), **i32)
        self.l_offsets = torch.empty((self.e_local + 1,), **i32)
        self.l_perm = torch.empty((cap,), **i32)
        self.l_rows = torch.empty((cap,), **i32)
        self.l_plan = torch.zeros((c.gemb_moe_plan_ints(cap, self.e_local, 1),), **i32)
        self.l_ws = torch.empty((c.gemb_moe_permute_workspace_bytes(cap, self.e_local, 1),), **u8)
        self.a_packed = torch.zeros((self.rows_max, h // 2), **u8)
        self.a_scales = torch.zeros((c.gemb_interleaved_scale_bytes(self.rows_max, h),), **u8)
        self.gate_up = torch.empty((self.rows_max, 2 * i), dtype=torch.int16, device=dev)
        self.p_packed = torch.zeros((self.rows_max, i // 2), **u8)
        self.p_scales = torch.zeros((c.gemb_interleaved_scale_bytes(self.rows_max, i),), **u8)
        self.y = torch.empty((self.rows_max, h), dtype=torch.int16, device=dev)
        self.y_send = torch.empty((cap, h), dtype=torch.int16, device=dev)
        self.y_sorted = torch.empty((n, h), dtype=torch.int16, device=dev)
        self.inv_perm = torch.empty((n,), **i32)
        self.arange = torch.arange(n, **i32)
        self.side = torch.cuda.Stream(device=dev)     # shared branch runs beside the exchange
        self.last = {}

    def forward(self, x_bf16):
        lib, w, t, k, loc = self.lib, self.w, self.tokens, self.topk, self.local
        h, n = w.hidden, self.tokens * self.topk
        main = torch.cuda.current_stream()
        if w.shared is not None:
            # The shared dense branch depends only on x: run it on a side stream so it overlaps the
            # count exchange, both all-to-alls and the host read-back.
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                loc.shared_branch(x_bf16, self.side)
        # 1. routing of the local tokens over all experts
        lib.gemb_moe_router_logits(x_bf16, w.router_w, w.router_bias, loc.logits, t, h, self.e_total, None)
        lib.gemb_moe_route(loc.logits, None, loc.ids, loc.weights, None, t, self.e_total, k, None)
        lib.gemb_moe_permute(loc.ids, loc.counts, loc.offsets, loc.perm, loc.slot_rows, loc.plan, loc.workspace,
                             loc.workspace.numel(), t, self.e_total, k, None)
        # 2. quantise once, pack in permutation order
        lib.gemb_nvfp4_quantize(x_bf16, 1, self.xq, self.xs, t, h, self.ga, 0, 0, None)
        mb, sc_off, id_off = self.msg_bytes, h // 2, h // 2 + h // 16
        lib.gemb_moe_gather_rows(self.xq, self.send_msg, loc.perm, k, n, h // 2, h // 2, mb, None)
        lib.gemb_moe_gather_rows(self.xs, self.send_msg[:, sc_off:], loc.perm, k, n, h // 16, h // 16, mb, None)
        send_eid = (loc.ids.view(-1)[loc.perm.long()] % self.e_local).to(torch.int32)
        self.send_msg[:, id_off:id_off + 4] = send_eid.view(torch.uint8).view(n, 4)
        # 3. split sizes (host read-back of E*R integers), then the dispatch all-to-all
        dist.all_gather_into_tensor(self.counts_all.view(-1), loc.counts, group=self.group)
        send_splits, recv_splits = ep_splits(self.counts_all.cpu().numpy(), self.rank, self.e_local)
        n_recv = sum(recv_splits)
        dist.all_to_all_single(self.recv_msg[:n_recv], self.send_msg, recv_splits, send_splits, group=self.group)
        # 4. local experts
        if n_recv > 0:
            self.recv_eid[:n_recv] = self.recv_msg[:n_recv, id_off:id_off + 4].contiguous().view(torch.int32).view(-1)
            lib.gemb_moe_permute(self.recv_eid, self.l_counts, self.l_offsets, self.l_perm, self.l_rows, self.l_plan,
                                 self.l_ws, self.l_ws.numel(), n_recv, self.e_local, 1, None)
            lib.gemb_moe_scatter_quantized(self.recv_msg, self.recv_msg[:, sc_off:], self.l_rows, self.a_packed,
                                           self.a_scales, n_recv, h, mb, None)
            lib.gemb_moe_grouped_gemm_bf16(self.a_packed, self.a_scales, w.gu_packed, w.gu_scales, self.gate_up,
                                           self.l_plan, self.rows_max, self.e_local, 2 * w.inter, h, self.ga, w.gu_div, None)
            lib.gemb_moe_expert_gelu_quantize(self.gate_up, self.l_plan, self.p_packed, self.p_scales, self.rows_max,
                                              w.inter, self.ga_dn, None)
            lib.gemb_moe_grouped_gemm_bf16(self.p_packed, self.p_scales, w.dn_packed, w.dn_scales, self.y, self.l_plan,
                                           self.rows_max, self.e_local, h, w.inter, self.ga_dn, w.dn_div, None)
            lib.gemb_moe_gather_rows(self.y, self.y_send, self.l_rows, 1, n_recv, h * 2, h * 2, h * 2, None)
        # 5. reverse all-to-all, shared branch, slot-ordered combine on the token's owner
        dist.all_to_all_single(self.y_sorted.view(torch.uint8), self.y_send[:n_recv].view(torch.uint8), send_splits,
                               recv_splits, group=self.group)   # byte rows: 16-bit integers are not a NCCL type
        self.inv_perm[loc.perm.long()] = self.arange
        if w.shared is not None:
            main.wait_stream(self.side)
        shared = loc.s_out if w.shared is not None else None
        lib.gemb_moe_combine(self.y_sorted, self.inv_perm, loc.weights, shared, loc.out, t, h, k, None)
        self.last = {"n_recv": n_recv, "send_splits": send_splits, "recv_splits": recv_splits}
        return loc.out


class EpPullMoeLayer:
    """The same layer with the exchange done by this library's own kernels over peer memory
    (`csrc/ep.cu`): each rank leaves its quantised assignments in a buffer the others have mapped,
    the owners pull them straight into the grouped GEMM's padded row space, and each token's owner
    pulls its expert outputs back inside the combine.  All row positions are arithmetic on the
    all-gathered counts, so nothing is read back to the host and the launch sequence is fixed.

    Ordering between GPUs comes from two barriers per layer: one after the send buffer and the
    counts are written ("send buffers complete"), one after the expert GEMMs ("expert outputs
    complete").  With sync="flags" (default) they are the library's own flag barrier over peer memory
    and the counts are read from the peers' buffers; with sync="nccl" the first is the all-gather of
    the counts and the second a one-element all-reduce.  The barriers also make buffer reuse safe:
    a rank refills its send buffer only after the second barrier of the previous layer (every peer
    has pulled), and overwrites its expert outputs only after the first barrier of the next layer
    (every peer has combined)."""

    def __init__(self, weights: MoeWeights, tokens: int, topk: int, ga: float, ga_dn: float, ga_sh_dn: float,
                 group=None, how: str = "auto", emulate=None, sync: str = "flags"):
        """emulate=(rank, world): no process group; the caller runs every rank's stages in turn on one
        GPU and wires the buffer tables together with `connect` (single-GPU test of the protocol)."""
        from .peer import PeerBuffer, LocalBuffer
        self.lib = load()
        self.group = group
        self.emulated = emulate is not None
        self.rank, self.world = emulate if self.emulated else (dist.get_rank(group), dist.get_world_size(group))
        self.w, self.tokens, self.topk = weights, tokens, topk
        self.ga, self.ga_dn = ga, ga_dn
        lib, dev, w, c = self.lib, weights.dev, weights, self.lib.cdll
        self.e_total, self.e_local = w.router_experts, w.experts
        assert self.e_local * self.world == self.e_total
        h, i, n = w.hidden, w.inter, tokens * topk
        self.local = MoeLayer(weights, tokens, topk, ga, ga_dn, ga_sh_dn, allocate_experts=False)
        cap = n * self.world                      # worst case: every assignment of every rank lands here
        self.cap = cap
        u8 = dict(dtype=torch.uint8, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        self.xq = torch.empty((tokens, h // 2), **u8)
        self.xs = torch.empty((tokens, h // 16), **u8)
        self.msg_bytes = (h // 2 + h // 16 + 15) // 16 * 16   # payload | block scales | pad
        self.rows_max = c.gemb_moe_padded_rows_max(cap, self.e_local, 1)
        if self.emulated:
            self.send = LocalBuffer(n * self.msg_bytes, dev)
            self.y_peer = LocalBuffer(self.rows_max * h * 2, dev)
        else:
            self.send = PeerBuffer(n * self.msg_bytes, dev, group, how)
            self.y_peer = PeerBuffer(self.rows_max * h * 2, dev, group, how)
        self.send_msg = self.send.local.view(n, self.msg_bytes)
        self.y = self.y_peer.local.view(torch.int16).view(self.rows_max, h)
        self.counts_all = torch.zeros((self.world, self.e_total), **i32)
        segs = self.world * self.e_local
        self.l_plan = torch.zeros((c.gemb_moe_ep_plan_ints(cap, self.e_local),), **i32)
        self.recv_prefix = torch.zeros((segs + 1,), **i32)
        self.recv_src = torch.zeros((segs,), **i32)
        self.recv_dst = torch.zeros((segs,), **i32)
        self.row_base = torch.zeros((self.e_total,), **i32)
        self.a_packed = torch.zeros((self.rows_max, h // 2), **u8)
        self.a_scales = torch.zeros((c.gemb_interleaved_scale_bytes(self.rows_max, h),), **u8)
        self.gate_up = torch.empty((self.rows_max, 2 * i), dtype=torch.int16, device=dev)
        self.p_packed = torch.zeros((self.rows_max, i // 2), **u8)
        self.p_scales = torch.zeros((c.gemb_interleaved_scale_bytes(self.rows_max, i),), **u8)
        self.flag = torch.zeros((1,), device=dev)
        self.side = torch.cuda.Stream(device=dev)
        self.sync = "host" if self.emulated else sync
        if self.sync == "flags":
            # the per-expert counts where the peers can read them, and the barrier's flag words
            self.counts_peer = PeerBuffer(self.e_total * 4, dev, group, how)
            self.flags_peer = PeerBuffer(2 * 16 * 4, dev, group, how)
            self.local.counts = self.counts_peer.local.view(torch.int32)
            self.epochs = torch.zeros((2,), **i32)
            dist.barrier(group)   # every rank's flag words are zero before the first barrier kernel runs

    @staticmethod
    def connect(layers):
        """Emulation only: give every layer the addresses of all layers' send and output buffers."""
        for l in layers:
            l.send.set_table([m.send.local.data_ptr() for m in layers])
            l.y_peer.set_table([m.y_peer.local.data_ptr() for m in layers])

    def stage_send(self, x_bf16):
        """Steps 1-2: route the local tokens, quantise once, leave the message rows for the peers."""
        lib, w, t, k, loc = self.lib, self.w, self.tokens, self.topk, self.local
        h, n = w.hidden, self.tokens * self.topk
        main = torch.cuda.current_stream()   # every launch names the stream: the collectives are ordered on it
        if w.shared is not None:
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                loc.shared_branch(x_bf16, self.side)
        lib.gemb_moe_router_logits(x_bf16, w.router_w, w.router_bias, loc.logits, t, h, self.e_total, main)
        lib.gemb_moe_route(loc.logits, None, loc.ids, loc.weights, None, t, self.e_total, k, main)
        lib.gemb_moe_permute(loc.ids, loc.counts, loc.offsets, loc.perm, loc.slot_rows, loc.plan, loc.workspace,
                             loc.workspace.numel(), t, self.e_total, k, main)
        lib.gemb_nvfp4_quantize(x_bf16, 1, self.xq, self.xs, t, h, self.ga, 0, 0, main)
        mb = self.msg_bytes
        lib.gemb_moe_gather_rows(self.xq, self.send_msg, loc.perm, k, n, h // 2, h // 2, mb, main)
        lib.gemb_moe_gather_rows(self.xs, self.send_msg[:, h // 2:], loc.perm, k, n, h // 16, h // 16, mb, main)

    def stage_experts(self):
        """Steps 3-4 after the counts of all ranks are in `counts_all`: positions, pull, expert GEMMs."""
        lib, w = self.lib, self.w
        h, el, R = w.hidden, self.e_local, self.world
        main = torch.cuda.current_stream()
        lib.gemb_moe_ep_plan(self.counts_all, R, self.e_total, self.rank, self.l_plan, self.recv_prefix, self.recv_src,
                             self.recv_dst, self.row_base, self.rows_max, self.tokens * self.topk, main)
        lib.gemb_moe_ep_pull_dispatch(self.send.table, R, el, self.recv_prefix, self.recv_src, self.recv_dst,
                                      self.a_packed, self.a_scales, h, self.msg_bytes, self.tokens * self.topk,
                                      self.rows_max, main)
        lib.gemb_moe_grouped_gemm_bf16(self.a_packed, self.a_scales, w.gu_packed, w.gu_scales, self.gate_up,
                                       self.l_plan, self.rows_max, el, 2 * w.inter, h, self.ga, w.gu_div, main)
        lib.gemb_moe_expert_gelu_quantize(self.gate_up, self.l_plan, self.p_packed, self.p_scales, self.rows_max,
                                          w.inter, self.ga_dn, main)
        lib.gemb_moe_grouped_gemm_bf16(self.p_packed, self.p_scales, w.dn_packed, w.dn_scales, self.y, self.l_plan,
                                       self.rows_max, el, h, w.inter, self.ga_dn, w.dn_div, main)

    def stage_combine(self):
        """Step 5 after every rank's expert outputs are complete."""
        lib, w, loc = self.lib, self.w, self.local
        main = torch.cuda.current_stream()
        if w.shared is not None:
            main.wait_stream(self.side)
        shared = loc.s_out if w.shared is not None else None
        lib.gemb_moe_ep_pull_combine(self.y_peer.table, self.world, self.e_local, loc.ids, loc.slot_rows, self.row_base,
                                     loc.weights, shared, loc.out, self.tokens, w.hidden, self.topk, self.rows_max, main)
        return loc.out

    def forward(self, x_bf16):
        self.stage_send(x_bf16)
        if self.sync == "flags":
            lib, main = self.lib, torch.cuda.current_stream()
            lib.gemb_moe_ep_barrier(self.flags_peer.table, self.world, self.rank, 0, self.epochs, main)
            lib.gemb_moe_ep_gather_counts(self.counts_peer.table, self.world, self.e_total, self.counts_all, main)
            self.stage_experts()
            lib.gemb_moe_ep_barrier(self.flags_peer.table, self.world, self.rank, 1, self.epochs, main)
            return self.stage_combine()
        # counts of every rank -- and: every send buffer is complete
        dist.all_gather_into_tensor(self.counts_all.view(-1), self.local.counts, group=self.group)
        self.stage_experts()
        dist.all_reduce(self.flag, group=self.group)   # every expert output is complete
        return self.stage_combine()


class EpLayer:
    """One expert-parallel layer through gemb_moe_ep_layer_forward: the launch sequence, the flag
    barriers and the workspace plan live in the library (csrc/ep.cu); this class only owns the
    memory -- the four peer-mapped buffers (message rows out, expert rows back, counts, flags)
    and the local workspace -- and builds the descriptors.

    emulate=(rank, world): no process group; plain device buffers stand in for the peer-mapped
    ones and the caller walks all ranks through `stage(0..2)` on one GPU, wiring the address tables
    with `connect` and copying the counts on the host side (tests)."""

    def __init__(self, weights: MoeWeights, tokens: int, topk: int, ga: float, ga_dn: float, ga_sh_dn: float,
                 group=None, how: str = "auto", emulate=None, fused: bool = True):
        from .lib import MoeEpComm, MoeRecords
        from .peer import LocalBuffer, PeerBuffer
        self.lib = load()
        lib, dev, w, c = self.lib, weights.dev, weights, self.lib.cdll
        self.emulated = emulate is not None
        self.rank, self.world = emulate if self.emulated else (dist.get_rank(group), dist.get_world_size(group))
        self.w, self.tokens, self.topk, self.fused = weights, tokens, topk, fused
        self.ga, self.ga_dn, self.ga_sh_dn = ga, ga_dn, ga_sh_dn
        self.e_total, self.e_local = w.router_experts, w.experts
        assert self.e_local * self.world == self.e_total
        h, n = w.hidden, tokens * topk
        self.msg_bytes = c.gemb_moe_ep_message_row_bytes(h)
        make = (lambda nbytes: LocalBuffer(nbytes, dev)) if self.emulated else (lambda nbytes: PeerBuffer(nbytes, dev, group, how))
        # message rows in (one region of n rows per source rank), expert rows back
        self.send, self.recv = make(self.world * n * self.msg_bytes), make(n * h * 2)
        self.counts_peer, self.flags_peer = make(self.e_total * 4), make(2 * 16 * 4)
        self.epochs = torch.zeros((2,), dtype=torch.int32, device=dev)
        self.out = torch.empty((tokens, h), dtype=torch.int16, device=dev)
        self._desc = {}
        desc = self.descriptor()
        nbytes = c.gemb_moe_ep_layer_workspace_bytes(C.addressof(desc), tokens, self.world)
        if nbytes == 0:
            raise RuntimeError(lib.last_error())
        self.workspace = torch.full((nbytes + 256,), 255, dtype=torch.uint8, device=dev)
        self.base = (self.workspace.data_ptr() + 255) // 256 * 256
        rec = MoeRecords()
        lib.gemb_moe_ep_layer_records(desc, tokens, self.world, self.base, rec)
        self.rows_max = rec.padded_rows_max
        e, k = self.e_total, topk
        self.ids = self._view(rec.top_ids, torch.int32, tokens, k)
        self.weights = self._view(rec.top_weights, torch.float32, tokens, k)
        self.perm = self._view(rec.perm, torch.int32, n)
        self.offsets = self._view(rec.offsets, torch.int32, e + 1)
        self.counts_all = self._view(rec.counts_all, torch.int32, self.world, e)
        self.plan = self._view(rec.plan, torch.int32, c.gemb_moe_ep_plan_ints(n * self.world, self.e_local))
        self.counts = self.counts_peer.local.view(torch.int32)
        self.side = torch.cuda.Stream(device=dev)
        self.fork_event, self.join_event = torch.cuda.Event(), torch.cuda.Event()
        self.fork_event.record()
        self.join_event.record()
        self.comm = None
        if not self.emulated:
            self._make_comm()
            dist.barrier(group)   # every rank's flag words are zero before the first barrier kernel runs

    def _view(self, ptr, dtype, *shape):
        nbytes = torch.empty((), dtype=dtype).element_size()
        for d in shape:
            nbytes *= d
        off = ptr - self.workspace.data_ptr()
        return self.workspace[off:off + nbytes].view(dtype).view(*shape)

    def descriptor(self):
        key = (id(self.w), self.fused)
        if key not in self._desc:
            self._desc[key] = self.w.c_struct(self.topk, self.ga, self.ga_dn, self.ga_sh_dn, fused=self.fused)
        return self._desc[key]

    def _make_comm(self):
        from .lib import MoeEpComm
        m = MoeEpComm()
        m.ranks, m.rank = self.world, self.rank
        m.send_buffers_host, m.recv_buffers_host = C.addressof(self.send.table), C.addressof(self.recv.table)
        m.count_buffers_host, m.flag_arrays_host = C.addressof(self.counts_peer.table), C.addressof(self.flags_peer.table)
        m.local_epochs = self.epochs.data_ptr()
        self.comm = m

    @staticmethod
    def connect(layers):
        """Emulation only: give every layer the addresses of all layers' buffers."""
        for l in layers:
            for name in ("send", "recv", "counts_peer", "flags_peer"):
                getattr(l, name).set_table([getattr(m, name).local.data_ptr() for m in layers])
            l._make_comm()

    def stage(self, which, x_bf16=None, barriers=False):
        self.lib.gemb_moe_ep_layer_stage(self.descriptor(), self.comm, x_bf16, self.out, self.tokens, self.base,
                                         self.workspace.numel() - 256, which, 1 if barriers else 0,
                                         torch.cuda.current_stream())
        return self.out

    def forward(self, x_bf16):
        self.lib.gemb_moe_ep_layer_forward(self.descriptor(), self.comm, x_bf16, self.out, self.tokens, self.base,
                                           self.workspace.numel() - 256, torch.cuda.current_stream(), self.side,
                                           self.fork_event.cuda_event, self.join_event.cuda_event)
        return self.out
