"""Test and benchmark harness around the MoE layer of the C ABI (torch only owns device memory).

`MoeLayer.forward` is one call of gemb_moe_layer_forward: the launch sequence, the workspace plan
and the fork / join of the shared branch live in the library (csrc/moe_layer.cu).  The stage
methods (`route`, `experts`, `shared_branch`, `combine`, `forward_stages`) issue the same
operator launches one by one from here, for stage timing and for tests that look at the
intermediate buffers; both ways give identical bytes.  Stage order:
docs/plans/gemma4-26b/specs/MOE_PREFILL_KERNEL_SPEC.md:34-47.
"""
from __future__ import annotations

import ctypes as C

import torch

from .lib import MoeLayerWeights, MoeRecords, Nvfp4Binding, load


class MoeWeights:
    """Device-resident NVFP4 expert weights in the layout the grouped GEMM consumes."""

    def __init__(self, lib, dev, router_w, router_bias, gu_packed, gu_scales, gu_div, dn_packed, dn_scales, dn_div,
                 shared=None, keep_compact=False):
        """keep_compact also keeps the row-major [rows, K/16] block scales as given (checkers
        that dequantise the weights themselves want them; the kernels use the interleaved copies)."""
        self.dev = dev
        if keep_compact:
            self.gu_compact, self.dn_compact = gu_scales, dn_scales
            self.shared_compact = None if shared is None else tuple(
                (p.cpu().numpy(), s.cpu().numpy(), float(d)) for p, s, d in shared)
        self.experts, self.two_inter, half_h = gu_packed.shape       # experts held on this device
        self.hidden, self.inter = half_h * 2, self.two_inter // 2
        self.router_w = torch.as_tensor(router_w, device=dev).contiguous()
        self.router_experts = self.router_w.shape[0]                # experts the router scores
        self.router_bias = None if router_bias is None else torch.as_tensor(router_bias, device=dev).contiguous()
        self.gu_packed = torch.as_tensor(gu_packed, device=dev).contiguous()
        self.dn_packed = torch.as_tensor(dn_packed, device=dev).contiguous()
        self.gu_div = torch.as_tensor(gu_div, device=dev, dtype=torch.float32).contiguous()
        self.dn_div = torch.as_tensor(dn_div, device=dev, dtype=torch.float32).contiguous()
        self.gu_scales = self._interleave(lib, gu_scales, self.two_inter, self.hidden)
        self.dn_scales = self._interleave(lib, dn_scales, self.hidden, self.inter)
        self.gu_fused, self.gu_fused_scales = self._fuse(lib, self.gu_packed, gu_scales, self.inter, self.hidden)
        self.shared = None
        if shared is not None:
            (sg_p, sg_s, sg_d), (sd_p, sd_s, sd_d) = shared
            self.shared = {
                "gu_packed": torch.as_tensor(sg_p, device=dev).contiguous(), "gu_div": float(sg_d),
                "gu_scales": self._interleave(lib, sg_s[None], sg_p.shape[0], self.hidden),
                "dn_packed": torch.as_tensor(sd_p, device=dev).contiguous(), "dn_div": float(sd_d),
                "dn_scales": self._interleave(lib, sd_s[None], self.hidden, sd_p.shape[1] * 2),
                "inter": sg_p.shape[0] // 2,
            }
            f, fs = self._fuse(lib, self.shared["gu_packed"][None], sg_s[None], sg_p.shape[0] // 2, self.hidden)
            self.shared["gu_fused"], self.shared["gu_fused_scales"] = f[0], fs[0]

    def c_struct(self, topk, ga, ga_dn, ga_sh_dn, fused=True, router_scale=None, router_eps=1e-6, per_expert_scale=None):
        """The gemb_moe_layer_weights descriptor of these weights (tensors stay owned by `self`)."""
        def ptr(t):
            return None if t is None else t.data_ptr()
        w = MoeLayerWeights()
        w.hidden, w.experts, w.topk, w.intermediate = self.hidden, self.router_experts, topk, self.inter
        w.router_weight, w.router_bias = ptr(self.router_w), ptr(self.router_bias)
        self._keep = (router_scale, per_expert_scale)
        w.router_input_scale, w.router_epsilon, w.per_expert_scale = ptr(router_scale), router_eps, ptr(per_expert_scale)
        w.gate_up = Nvfp4Binding(ptr(self.gu_packed), None, None, ga, 0.0, self.two_inter, self.hidden, ptr(self.gu_scales),
                                 ptr(self.gu_div), self.experts)
        w.down = Nvfp4Binding(ptr(self.dn_packed), None, None, ga_dn, 0.0, self.hidden, self.inter, ptr(self.dn_scales),
                              ptr(self.dn_div), self.experts)
        if fused:
            w.gate_up_fused, w.gate_up_fused_scales = ptr(self.gu_fused), ptr(self.gu_fused_scales)
        if self.shared is not None:
            s = self.shared
            w.shared_intermediate = s["inter"]
            w.shared_gate_up = Nvfp4Binding(ptr(s["gu_packed"]), None, None, ga, s["gu_div"], 2 * s["inter"], self.hidden,
                                            ptr(s["gu_scales"]), None, 0)
            w.shared_down = Nvfp4Binding(ptr(s["dn_packed"]), None, None, ga_sh_dn, s["dn_div"], self.hidden, s["inter"],
                                         ptr(s["dn_scales"]), None, 0)
            if fused:
                w.shared_gate_up_fused, w.shared_gate_up_fused_scales = ptr(s["gu_fused"]), ptr(s["gu_fused_scales"])
        return w

    def _fuse(self, lib, packed, compact, inter, k):
        """Per expert: gate rows [0, inter) and up rows [inter, 2*inter) -> the 32-feature
        interleaved layout the gated-epilogue GEMM consumes."""
        compact = torch.as_tensor(compact, device=self.dev).contiguous()
        n = packed.shape[0]
        out = torch.empty_like(packed)
        per = lib.cdll.gemb_interleaved_scale_bytes(2 * inter, k)
        out_s = torch.empty((n, per), dtype=torch.uint8, device=self.dev)
        for e in range(n):
            lib.gemb_nvfp4_pack_gate_up(packed[e, :inter], compact[e, :inter], packed[e, inter:], compact[e, inter:],
                                        out[e], out_s[e], inter, k, None)
        return out, out_s

    def _interleave(self, lib, compact, rows, k):
        compact = torch.as_tensor(compact, device=self.dev).contiguous()
        per = lib.cdll.gemb_interleaved_scale_bytes(rows, k)
        out = torch.empty((compact.shape[0], per), dtype=torch.uint8, device=self.dev)
        for e in range(compact.shape[0]):
            lib.gemb_nvfp4_interleave_scales(compact[e], out[e], rows, k, None)
        return out


class MoeLayer:
    """Preallocated buffers + the launch sequence for `tokens` tokens."""

    def __init__(self, weights: MoeWeights, tokens: int, topk: int, ga: float, ga_dn: float, ga_sh_dn: float = 1.0,
                 allocate_experts: bool = True, stages: bool = True):
        """stages=False skips the buffers only the stage methods use (forward() needs none of them)."""
        self.lib = load()
        self.side = None
        # gate/up GEMM + GELU + requantisation in one kernel: byte-identical, but with four epilogue
        # warps the extra arithmetic is not hidden yet, so the three-launch form is the default.
        self.fused = False
        self.w, self.tokens, self.topk = weights, tokens, topk
        self.ga, self.ga_dn, self.ga_sh_dn = ga, ga_dn, ga_sh_dn
        lib, dev, w = self.lib, weights.dev, weights
        e, h, i = w.router_experts, w.hidden, w.inter
        c = lib.cdll
        self.rows_max = c.gemb_moe_padded_rows_max(tokens, e, topk)
        i32 = dict(dtype=torch.int32, device=dev)
        u8 = dict(dtype=torch.uint8, device=dev)
        self.logits = torch.empty((tokens, e), device=dev)
        self.ids = torch.empty((tokens, topk), **i32)
        self.weights = torch.empty((tokens, topk), device=dev)
        self.counts = torch.empty((e,), **i32)
        self.offsets = torch.empty((e + 1,), **i32)
        self.perm = torch.empty((tokens * topk,), **i32)
        self.slot_rows = torch.empty((tokens * topk,), **i32)
        self.plan = torch.zeros((c.gemb_moe_plan_ints(tokens, e, topk),), **i32)
        self.workspace = torch.empty((c.gemb_moe_permute_workspace_bytes(tokens, e, topk),), **u8)
        if allocate_experts and stages:   # the expert-parallel layer owns its own (differently sized) expert buffers
            self.a_packed = torch.zeros((self.rows_max, h // 2), **u8)
            self.a_scales = torch.zeros((c.gemb_interleaved_scale_bytes(self.rows_max, h),), **u8)
            self.gate_up = torch.empty((self.rows_max, 2 * i), dtype=torch.int16, device=dev)
            self.p_packed = torch.zeros((self.rows_max, i // 2), **u8)
            self.p_scales = torch.zeros((c.gemb_interleaved_scale_bytes(self.rows_max, i),), **u8)
            self.y = torch.empty((self.rows_max, h), dtype=torch.int16, device=dev)
        self.out = torch.empty((tokens, h), dtype=torch.int16, device=dev)
        self.router_scale = self.per_expert_scale = None     # optional router tensors (bf16 [hidden], fp32 [experts])
        self.c_workspace = None
        if allocate_experts:
            # the library's own layer call: one workspace, records viewed in place
            desc = w.c_struct(topk, ga, ga_dn, ga_sh_dn, fused=False)
            nbytes = c.gemb_moe_layer_workspace_bytes(C.addressof(desc), tokens)
            if nbytes == 0:
                raise RuntimeError(lib.last_error())
            nbytes += tokens * h * 2 + 256        # room for the router's transformed input, should a test switch it on
            # filled with 0xFF: the layer must not depend on what the workspace held before
            self.c_workspace = torch.full((nbytes + 256,), 255, **u8)
            self.c_base = (self.c_workspace.data_ptr() + 255) // 256 * 256
            rec = MoeRecords()
            lib.gemb_moe_layer_records(desc, tokens, self.c_base, rec)

            view = self._ws_view
            self.logits = view(rec.logits, torch.float32, tokens, e)
            self.ids = view(rec.top_ids, torch.int32, tokens, topk)
            self.weights = view(rec.top_weights, torch.float32, tokens, topk)
            self.counts = view(rec.counts, torch.int32, e)
            self.offsets = view(rec.offsets, torch.int32, e + 1)
            self.perm = view(rec.perm, torch.int32, tokens * topk)
            self.slot_rows = view(rec.slot_rows, torch.int32, tokens * topk)
            self.plan = view(rec.plan, torch.int32, c.gemb_moe_plan_ints(tokens, e, topk))
            self.y = view(rec.expert_rows, torch.int16, self.rows_max, h)
            self.fork_event, self.join_event = torch.cuda.Event(), torch.cuda.Event()
            self._desc, self._y = {}, {}
        if w.shared is not None and stages:
            si = w.shared["inter"]
            self.s_packed = torch.empty((tokens, h // 2), **u8)
            self.s_scales = torch.zeros((c.gemb_interleaved_scale_bytes(tokens, h),), **u8)
            self.s_gate_up = torch.empty((tokens, 2 * si), dtype=torch.int16, device=dev)
            self.s_p_packed = torch.zeros((tokens, si // 2), **u8)
            self.s_p_scales = torch.zeros((c.gemb_interleaved_scale_bytes(tokens, si),), **u8)
            self.s_out = torch.empty((tokens, h), dtype=torch.int16, device=dev)

    def route(self, x_bf16, stream=None):
        lib, w, t = self.lib, self.w, self.tokens
        lib.gemb_moe_router_logits(x_bf16, w.router_w, w.router_bias, self.logits, t, w.hidden, w.experts, stream)
        lib.gemb_moe_route(self.logits, None, self.ids, self.weights, None, t, w.experts, self.topk, stream)
        lib.gemb_moe_permute(self.ids, self.counts, self.offsets, self.perm, self.slot_rows, self.plan, self.workspace,
                             self.workspace.numel(), t, w.experts, self.topk, stream)

    def experts(self, x_bf16, stream=None):
        lib, w, t = self.lib, self.w, self.tokens
        lib.gemb_moe_dispatch_quantize(x_bf16, self.slot_rows, self.a_packed, self.a_scales, t, w.hidden, self.topk,
                                       self.ga, stream)
        if self.fused:
            lib.gemb_moe_grouped_gemm_gated_quant(self.a_packed, self.a_scales, w.gu_fused, w.gu_fused_scales,
                                                  self.p_packed, self.p_scales, self.plan, self.rows_max, w.experts,
                                                  w.inter, w.hidden, self.ga, w.gu_div, self.ga_dn, stream)
            lib.gemb_moe_grouped_gemm_bf16(self.p_packed, self.p_scales, w.dn_packed, w.dn_scales, self.y, self.plan,
                                           self.rows_max, w.experts, w.hidden, w.inter, self.ga_dn, w.dn_div, stream)
            return
        lib.gemb_moe_grouped_gemm_bf16(self.a_packed, self.a_scales, w.gu_packed, w.gu_scales, self.gate_up, self.plan,
                                       self.rows_max, w.experts, 2 * w.inter, w.hidden, self.ga, w.gu_div, stream)
        lib.gemb_moe_expert_gelu_quantize(self.gate_up, self.plan, self.p_packed, self.p_scales, self.rows_max, w.inter,
                                          self.ga_dn, stream)
        lib.gemb_moe_grouped_gemm_bf16(self.p_packed, self.p_scales, w.dn_packed, w.dn_scales, self.y, self.plan,
                                       self.rows_max, w.experts, w.hidden, w.inter, self.ga_dn, w.dn_div, stream)

    def shared_branch(self, x_bf16, stream=None):
        lib, w, t, s = self.lib, self.w, self.tokens, self.w.shared
        lib.gemb_nvfp4_quantize(x_bf16, 1, self.s_packed, self.s_scales, t, w.hidden, self.ga, 1, 0, stream)
        if self.fused:
            lib.gemb_nvfp4_gemm_gated_quant(self.s_packed, self.s_scales, s["gu_fused"], s["gu_fused_scales"],
                                            self.s_p_packed, self.s_p_scales, t, s["inter"], w.hidden, self.ga,
                                            s["gu_div"], s["gu_div"], self.ga_sh_dn, stream)
            lib.gemb_nvfp4_gemm_bf16(self.s_p_packed, self.s_p_scales, s["dn_packed"], s["dn_scales"], self.s_out, t,
                                     w.hidden, s["inter"], self.ga_sh_dn, s["dn_div"], stream)
            return
        lib.gemb_nvfp4_gemm_bf16(self.s_packed, self.s_scales, s["gu_packed"], s["gu_scales"], self.s_gate_up, t,
                                 2 * s["inter"], w.hidden, self.ga, s["gu_div"], stream)
        lib.gemb_moe_expert_gelu_quantize(self.s_gate_up, None, self.s_p_packed, self.s_p_scales, t, s["inter"],
                                          self.ga_sh_dn, stream)
        lib.gemb_nvfp4_gemm_bf16(self.s_p_packed, self.s_p_scales, s["dn_packed"], s["dn_scales"], self.s_out, t,
                                 w.hidden, s["inter"], self.ga_sh_dn, s["dn_div"], stream)

    def combine(self, stream=None):
        shared = self.s_out if self.w.shared is not None else None
        self.lib.gemb_moe_combine(self.y, self.slot_rows, self.weights, shared, self.out, self.tokens, self.w.hidden,
                                  self.topk, stream)

    def forward(self, x_bf16, stream=None):
        """One gemb_moe_layer_forward call (shared branch forked onto a side stream)."""
        main = stream if stream is not None else torch.cuda.current_stream()
        if self.side is None:
            self.side = torch.cuda.Stream(device=self.w.dev)
            self.fork_event.record(main)     # creates the CUDA events behind the torch objects
            self.join_event.record(main)
        key = (id(self.w), self.fused, id(self.router_scale), id(self.per_expert_scale))
        if key not in self._desc:
            self._desc[key] = self.w.c_struct(self.topk, self.ga, self.ga_dn, self.ga_sh_dn, fused=self.fused,
                                              router_scale=self.router_scale, per_expert_scale=self.per_expert_scale)
            rec = MoeRecords()
            self.lib.gemb_moe_layer_records(self._desc[key], self.tokens, self.c_base, rec)
            self._y[key] = self._ws_view(rec.expert_rows, torch.int16, self.rows_max, self.w.hidden)
        self.y = self._y[key]    # the expert rows sit behind the optional buffers of the workspace
        self.lib.gemb_moe_layer_forward(self._desc[key], x_bf16, self.out, self.tokens, self.c_base,
                                        self.c_workspace.numel() - 256, main, self.side, self.fork_event.cuda_event,
                                        self.join_event.cuda_event)
        return self.out

    def _ws_view(self, ptr, dtype, *shape):
        n = torch.empty((), dtype=dtype).element_size()
        for d in shape:
            n *= d
        off = ptr - self.c_workspace.data_ptr()
        return self.c_workspace[off:off + n].view(dtype).view(*shape)

    def forward_stages(self, x_bf16, stream=None):
        """The same layer as separate launches from Python (stage timing, intermediate buffers)."""
        main = stream if stream is not None else torch.cuda.current_stream()
        if self.w.shared is not None:
            # The shared dense branch depends only on x: it runs on a side stream beside routing and
            # the expert GEMMs and joins before the combine (the fork/join is capturable).
            if self.side is None:
                self.side = torch.cuda.Stream(device=self.w.dev)
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                self.shared_branch(x_bf16, self.side)
        self.route(x_bf16, stream)
        self.experts(x_bf16, stream)
        if self.w.shared is not None:
            main.wait_stream(self.side)
        self.combine(stream)
        return self.out


def place_experts(bias, hidden, ranks, generator, topk=8, samples=8192, weight_std=0.02):
    """Load-time expert placement for expert parallelism: returns the router bias re-labelled so that rank r owns
    ids [r*E/R, (r+1)*E/R) (expert ids are labels; the router rows are exchangeable).  What is known before any
    token is routed is the popularity prior, and with top-k routing a hot expert saturates (it is picked by nearly
    every token and then holds as many rows as a whole rank's fair share at 8 ranks), so the expected load is
    estimated by routing a seeded calibration batch of random logits (the router weight's contribution is
    N(0, sigma^2) per expert) through the same top-k, and the experts go to the ranks greedily, heaviest first,
    each to the least loaded rank that still has a free slot.  Dealing the prior out in serpentine order left the
    fullest rank 31 % above the mean at 8 ranks; this leaves it 1-2 % above."""
    experts = bias.numel()
    sigma = weight_std * float(hidden) ** 0.5
    z = torch.randn((samples, experts), device=bias.device, generator=generator) * sigma + bias
    picked = torch.topk(z, topk, dim=1).indices.reshape(-1)
    load_est = torch.bincount(picked, minlength=experts).double().cpu()
    order = sorted(range(experts), key=lambda e: (-float(load_est[e]), e))
    per = experts // ranks
    new_bias = torch.empty_like(bias)
    fill, rank_load = [0] * ranks, [0.0] * ranks
    for src in order:
        r = min((r for r in range(ranks) if fill[r] < per), key=lambda r: (rank_load[r], r))
        new_bias[r * per + fill[r]] = bias[src]
        fill[r] += 1
        rank_load[r] += float(load_est[src])
    return new_bias


def synthetic_weights(dev, seed, hidden=2816, experts=128, inter=704, shared_inter=2112, zipf=True,
                      expert_range=None, placement_ranks=1, keep_compact=False):
    """Seeded synthetic 26B-A4B-like layer generated and quantised on the GPU: router fp32 ~ N(0, 0.02)
    with a Zipf(1.1) bias (-1.1 ln(rank) over a seeded permutation, zero mean), NVFP4 expert and
    shared weights ~ N(0, 0.02) with per-tensor divisor 6*448/amax.  expert_range=(lo, hi) keeps
    only those experts' weights (expert parallelism); the router always scores all of them."""
    lib = load()
    g = torch.Generator(device=dev)
    g.manual_seed(seed)

    def quant(rows, k):
        w = torch.randn((rows, k), device=dev, generator=g) * 0.02
        div = float(2688.0 / w.abs().max().item())
        packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=dev)
        scales = torch.empty((rows, k // 16), dtype=torch.uint8, device=dev)
        lib.gemb_nvfp4_quantize(w, 0, packed, scales, rows, k, div, 0, 0, None)
        return packed, scales, div

    router_w = torch.randn((experts, hidden), device=dev, generator=g) * 0.02
    bias = None
    if zipf:
        rank = torch.randperm(experts, device=dev, generator=g).double() + 1
        b = -1.1 * torch.log(rank)
        bias = (b - b.mean()).float()
        if placement_ranks > 1:
            bias = place_experts(bias, hidden, placement_ranks, g)
    # Every rank draws every expert (identical streams) and keeps its own range.
    lo, hi = expert_range if expert_range is not None else (0, experts)
    gu, dn = [], []
    for e in range(experts):
        a, b = quant(2 * inter, hidden), quant(hidden, inter)
        if lo <= e < hi:
            gu.append(a)
            dn.append(b)
    shared = None
    if shared_inter:
        shared = (quant(2 * shared_inter, hidden), quant(hidden, shared_inter))
    return MoeWeights(lib, dev, router_w, bias, torch.stack([x[0] for x in gu]), torch.stack([x[1] for x in gu]),
                      [x[2] for x in gu], torch.stack([x[0] for x in dn]), torch.stack([x[1] for x in dn]),
                      [x[2] for x in dn], shared, keep_compact=keep_compact)
