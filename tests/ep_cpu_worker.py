"""One gloo rank of the CPU expert-parallel protocol test (launched by tests/test_ep_cpu.py).

Follows gem16_b200/ep.py step for step with numpy + the CPU oracle instead of CUDA launches, and
checks that the rank's slice of the output is bit-identical to the single-process layer."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from gem16_b200.ep import ep_splits  # noqa: E402
from oracle import Oracle  # noqa: E402
from tests.moe_ref import ffn_oracle, make_layer, moe_layer_oracle  # noqa: E402
from tests.util import bf16_bits, from_bf16_bits  # noqa: E402


def a2a(send, send_splits, recv_splits):
    recv = torch.empty((sum(recv_splits),) + tuple(send.shape[1:]), dtype=send.dtype)
    dist.all_to_all_single(recv, send.contiguous(), recv_splits, send_splits)
    return recv


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    orc = Oracle()
    hidden, experts, inter, shared_inter, topk, tokens = 128, 32, 64, 64, 4, 22
    rng = np.random.default_rng(99)
    p = make_layer(orc, rng, hidden, experts, inter, shared_inter)
    x_all = bf16_bits(rng.standard_normal((tokens * world, hidden)).astype(np.float32))
    ga, ga_dn, ga_sh = 500.0, 300.0, 300.0
    ref = moe_layer_oracle(orc, p, x_all, topk, ga, ga_dn, ga_sh)
    x = x_all[rank * tokens:(rank + 1) * tokens]
    e_local = experts // world

    # 1. local routing over all experts
    logits = orc.moe_router_logits(x, p["router_w"], p["router_bias"])
    ids, weights = orc.moe_route(logits, topk)
    counts, offsets, perm = orc.moe_permute(ids, experts)
    assert np.array_equal(ids, ref["ids"][rank * tokens:(rank + 1) * tokens])
    # 2. quantise, pack in permutation order
    xq, xs = orc.nvfp4_quantize(from_bf16_bits(x), ga)
    tok = perm // topk
    send_payload, send_scales = torch.from_numpy(xq[tok]), torch.from_numpy(xs[tok])
    send_eid = torch.from_numpy((ids.reshape(-1)[perm] % e_local).astype(np.int32))
    # 3. counts, splits, dispatch
    gathered = [torch.empty(experts, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(counts))
    counts_all = torch.stack(gathered).numpy()
    send_splits, recv_splits = ep_splits(counts_all, rank, e_local)
    assert sum(send_splits) == tokens * topk
    r_payload = a2a(send_payload, send_splits, recv_splits).numpy()
    r_scales = a2a(send_scales, send_splits, recv_splits).numpy()
    r_eid = a2a(send_eid, send_splits, recv_splits).numpy()
    # 4. local experts in stable (expert, arrival) order
    n_recv = r_eid.shape[0]
    y_send = np.zeros((n_recv, hidden), np.uint16)
    if n_recv:
        _, l_off, l_perm = orc.moe_permute(r_eid.reshape(-1, 1), e_local)
        for e in range(e_local):
            sel = l_perm[l_off[e]:l_off[e + 1]]
            if sel.size == 0:
                continue
            g = rank * e_local + e
            y, _, _ = ffn_oracle(orc, r_payload[sel], r_scales[sel], ga,
                                 (p["gu_packed"][g], p["gu_scales"][g], float(p["gu_div"][g])),
                                 (p["dn_packed"][g], p["dn_scales"][g], float(p["dn_div"][g])), ga_dn, inter)
            y_send[sel] = bf16_bits(y)
    # 5. reverse all-to-all, shared branch, combine
    y_sorted = a2a(torch.from_numpy(y_send.view(np.uint8)), recv_splits, send_splits).numpy().view(np.uint16)
    inv = np.empty(tokens * topk, np.int64)
    inv[perm] = np.arange(tokens * topk)
    shared, _, _ = ffn_oracle(orc, xq, xs, ga, p["sh_gu"], p["sh_dn"], ga_sh, shared_inter)
    out = orc.moe_combine(y_sorted[inv].reshape(tokens, topk, hidden), weights, bf16_bits(shared))
    want = ref["out"][rank * tokens:(rank + 1) * tokens]
    assert np.array_equal(out, want), f"rank {rank}: expert-parallel output differs from the single-process layer"
    # global counts equal the single-process histogram
    assert np.array_equal(counts_all.sum(0), ref["counts"])
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
