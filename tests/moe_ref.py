"""CPU restatement of one MoE layer out of the oracle's primitives (test infrastructure).

Follows docs/plans/gemma4-26b/specs/MOE_ROUTER_SPEC.md (router), MOE_PREFILL_KERNEL_SPEC.md:19-58
(assignments, stable permutation), tools/capture_gemma4_26b_goldens.py:232-240 (expert math with the
fused gate_up projection, gate first) with the bf16 / requantisation boundaries of
src/cuda/nvfp4/reference.cu:177-217, and MOE_SEMANTICS_SPEC.md:74-83 (slot-ordered fp32 combine).
"""
import numpy as np

from tests.util import bf16_bits, bf16_round, from_bf16_bits


def make_layer(orc, rng, hidden, experts, inter, shared_inter=0, zipf=True):
    """Seeded synthetic layer: router fp32 N(0, 0.02) + Zipf(1.1) bias, NVFP4 expert weights."""
    p = {"hidden": hidden, "experts": experts, "inter": inter}
    p["router_w"] = (rng.standard_normal((experts, hidden)) * 0.02).astype(np.float32)
    if zipf:
        rank = rng.permutation(experts) + 1
        bias = -1.1 * np.log(rank.astype(np.float64))
        p["router_bias"] = (bias - bias.mean()).astype(np.float32)
    else:
        p["router_bias"] = None

    def quant(w):
        g = float(np.float32(2688.0) / np.float32(np.abs(w).max()))
        packed, scales = orc.nvfp4_quantize(w, g)
        return packed, scales, g

    gu, dn = [], []
    for _ in range(experts):
        gu.append(quant((rng.standard_normal((2 * inter, hidden)) * 0.02).astype(np.float32)))
        dn.append(quant((rng.standard_normal((hidden, inter)) * 0.02).astype(np.float32)))
    p["gu_packed"] = np.stack([g[0] for g in gu]); p["gu_scales"] = np.stack([g[1] for g in gu])
    p["gu_div"] = np.array([g[2] for g in gu], np.float32)
    p["dn_packed"] = np.stack([d[0] for d in dn]); p["dn_scales"] = np.stack([d[1] for d in dn])
    p["dn_div"] = np.array([d[2] for d in dn], np.float32)
    if shared_inter:
        p["shared_inter"] = shared_inter
        p["sh_gu"] = quant((rng.standard_normal((2 * shared_inter, hidden)) * 0.02).astype(np.float32))
        p["sh_dn"] = quant((rng.standard_normal((hidden, shared_inter)) * 0.02).astype(np.float32))
    return p


def ffn_oracle(orc, xq, xs, ga, gu, dn, ga_dn, inter):
    """Gated FFN on already quantised rows: returns bf16-valued fp32 [rows, hidden]."""
    gate_up = orc.nvfp4_matmul(xq, xs, gu[0], gu[1], ga, gu[2])
    gate_up = bf16_round(gate_up.astype(np.float32))
    prod = orc.gated_gelu(gate_up[:, :inter], gate_up[:, inter:])
    pq, ps = orc.nvfp4_quantize(prod, ga_dn)
    y = orc.nvfp4_matmul(pq, ps, dn[0], dn[1], ga_dn, dn[2])
    return bf16_round(y.astype(np.float32)), gate_up, (pq, ps)


def moe_layer_oracle(orc, p, x_bf16_bits, topk, ga, ga_dn, ga_sh_dn=None):
    x = from_bf16_bits(x_bf16_bits)
    t, hidden = x.shape
    logits = orc.moe_router_logits(x_bf16_bits, p["router_w"], p["router_bias"])
    ids, weights = orc.moe_route(logits, topk)
    counts, offsets, perm = orc.moe_permute(ids, p["experts"])
    xq, xs = orc.nvfp4_quantize(x, ga)
    y_slots = np.zeros((t * topk, hidden), np.float32)
    for e in range(p["experts"]):
        sel = perm[offsets[e]:offsets[e + 1]]
        if sel.size == 0:
            continue
        tok = sel // topk
        y, _, _ = ffn_oracle(orc, xq[tok], xs[tok], ga, (p["gu_packed"][e], p["gu_scales"][e], float(p["gu_div"][e])),
                             (p["dn_packed"][e], p["dn_scales"][e], float(p["dn_div"][e])), ga_dn, p["inter"])
        y_slots[sel] = y
    shared = None
    if "sh_gu" in p:
        shared, _, _ = ffn_oracle(orc, xq, xs, ga, p["sh_gu"], p["sh_dn"], ga_sh_dn, p["shared_inter"])
    out = orc.moe_combine(bf16_bits(y_slots).reshape(t, topk, hidden), weights,
                          None if shared is None else bf16_bits(shared))
    return {"logits": logits, "ids": ids, "weights": weights, "counts": counts, "offsets": offsets, "perm": perm,
            "y_slots": y_slots, "shared": shared, "out": out}


def ep_plan_reference(counts_all, me):
    """Plain restatement of the position arithmetic (see the header comment of csrc/ep.cu)."""
    ranks, experts = counts_all.shape
    el = experts // ranks
    tot = counts_all.sum(0)
    pad = np.zeros(experts, np.int64)
    for d in range(ranks):
        po = 0
        for e in range(d * el, (d + 1) * el):
            pad[e] = po
            po += (tot[e] + 255) // 256 * 256
    my_pad = np.concatenate([[0], np.cumsum((counts_all[me] + 255) // 256 * 256)])[:-1]
    before_me = counts_all[:me].sum(0)
    row_base = pad + before_me - my_pad
    prefix, src, dst = [0], [], []
    for s in range(ranks):
        sorted_off = np.concatenate([[0], np.cumsum(counts_all[s])])
        for e in range(me * el, (me + 1) * el):
            src.append(sorted_off[e])
            dst.append(pad[e] + counts_all[:s, e].sum())
            prefix.append(prefix[-1] + counts_all[s, e])
    mine = slice(me * el, (me + 1) * el)
    padded_rows = int(((tot[mine] + 255) // 256 * 256).sum())
    return dict(row_base=row_base, prefix=np.array(prefix), src=np.array(src), dst=np.array(dst),
                pad_local=pad[mine], padded_rows=padded_rows)
