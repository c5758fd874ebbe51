"""Tensor-parallel gated MLP over NCCL: gate/up split by output feature (column parallel, no
communication, the intermediate stays sharded), down split along K (row parallel, fp32 partial
sums all-reduced, rounded to bf16 once).  NVFP4 block scales run along K in groups of 16, so a K
split at a multiple of 64 keeps every block and its scale on one rank; the per-tensor divisors are
global.  gem16 has no multi-GPU code; this is the library's own sharding of its dense path."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .lib import load


class TpMlp:
    def __init__(self, dev, gate, up, down, tokens: int, ga: float, ga_dn: float, group=None, reduce: str = "auto"):
        """gate / up / down: (packed [rows, K/2] uint8, compact scales [rows, K/16] uint8, divisor) of the
        FULL matrices (identical on every rank); each rank keeps its shard."""
        self.lib = lib = load()
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        r, w = self.rank, self.world
        self.tokens, self.ga, self.ga_dn = tokens, ga, ga_dn
        inter, half_h = gate[0].shape
        self.hidden, self.inter = half_h * 2, inter
        assert inter % (64 * w) == 0
        self.i_local = il = inter // w
        c = lib.cdll

        def interleave(compact, rows, k):
            out = torch.zeros((c.gemb_interleaved_scale_bytes(rows, k),), dtype=torch.uint8, device=dev)
            lib.gemb_nvfp4_interleave_scales(compact.contiguous(), out, rows, k, None)
            return out

        def rows_shard(m):          # features [r*il, (r+1)*il)
            return m[0][r * il:(r + 1) * il].contiguous(), interleave(m[1][r * il:(r + 1) * il], il, self.hidden), m[2]

        self.gate, self.up = rows_shard(gate), rows_shard(up)
        # down [hidden, inter]: K slice [r*il, (r+1)*il) -> payload columns /2, scale columns /16
        dp = down[0][:, r * il // 2:(r + 1) * il // 2].contiguous()
        ds = interleave(down[1][:, r * il // 16:(r + 1) * il // 16], self.hidden, il)
        self.down = (dp, ds, down[2])
        u8 = dict(dtype=torch.uint8, device=dev)
        self.xq = torch.empty((tokens, half_h), **u8)
        self.xs = torch.zeros((c.gemb_interleaved_scale_bytes(tokens, self.hidden),), **u8)
        self.g = torch.empty((tokens, il), dtype=torch.int16, device=dev)
        self.u = torch.empty((tokens, il), dtype=torch.int16, device=dev)
        self.pq = torch.empty((tokens, il // 2), **u8)
        self.ps = torch.zeros((c.gemb_interleaved_scale_bytes(tokens, il),), **u8)
        # reduce = "peer": the library's reduce-scatter / all-gather over peer memory with its own flag
        # barrier; "nccl": all-reduce of the fp32 partials; "auto": peer when the buffers can be mapped.
        self.reduce = "nccl"
        self.partial = None
        if self.world > 1 and reduce in ("auto", "peer"):
            try:
                from .peer import PeerBuffer
                self.partial_peer = PeerBuffer(tokens * self.hidden * 4, dev, group)
                self.out_peer = PeerBuffer(tokens * self.hidden * 2, dev, group)
                self.flags_peer = PeerBuffer(2 * 16 * 4, dev, group)
                self.epochs = torch.zeros((2,), dtype=torch.int32, device=dev)
                self.partial = self.partial_peer.local.view(torch.float32).view(tokens, self.hidden)
                self.out = self.out_peer.local.view(torch.int16).view(tokens, self.hidden)
                self.reduce = "peer"
                dist.barrier(group)
            except Exception:
                if reduce == "peer":
                    raise
        if self.partial is None:
            self.partial = torch.empty((tokens, self.hidden), dtype=torch.float32, device=dev)

    def forward(self, x_bf16):
        lib, t, h, il = self.lib, self.tokens, self.hidden, self.i_local
        lib.gemb_nvfp4_quantize(x_bf16, 1, self.xq, self.xs, t, h, self.ga, 1, 0, None)
        lib.gemb_nvfp4_gemm_bf16(self.xq, self.xs, self.gate[0], self.gate[1], self.g, t, il, h, self.ga, self.gate[2], None)
        lib.gemb_nvfp4_gemm_bf16(self.xq, self.xs, self.up[0], self.up[1], self.u, t, il, h, self.ga, self.up[2], None)
        lib.gemb_nvfp4_gated_gelu_quantize(self.g, self.u, 1, self.pq, self.ps, t, il, self.ga_dn, 1, 0, None)
        lib.gemb_nvfp4_gemm_f32(self.pq, self.ps, self.down[0], self.down[1], self.partial, t, h, il, self.ga_dn,
                                self.down[2], None)
        if self.reduce == "peer":
            st, R, r = torch.cuda.current_stream(), self.world, self.rank
            lib.gemb_moe_ep_barrier(self.flags_peer.table, R, r, 0, self.epochs, st)     # every partial is complete
            lib.gemb_tp_reduce_rows(self.partial_peer.table, R, r, t, h, self.out, st)
            lib.gemb_moe_ep_barrier(self.flags_peer.table, R, r, 1, self.epochs, st)     # every slice is complete
            lib.gemb_tp_gather_rows(self.out_peer.table, R, r, t, h, self.out, st)
            return self.out.view(torch.bfloat16)
        if self.world > 1:
            dist.all_reduce(self.partial, group=self.group)
        return self.partial.to(torch.bfloat16)
