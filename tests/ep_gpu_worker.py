"""One NCCL rank of the GPU expert-parallel test (launched by tests/test_ep_gpu.py with torchrun).
Every rank also runs the single-GPU layer on all tokens and requires its slice of the
expert-parallel output, ids, weights and global counts to be bit-identical."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from gem16_b200 import load  # noqa: E402
from gem16_b200.ep import EpLayer, EpMoeLayer, EpPullMoeLayer  # noqa: E402
from gem16_b200.moe import MoeLayer, synthetic_weights  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    lib = load()
    hidden, experts, inter, shared_inter, topk = 2816, 128, 704, 2112, 8
    tokens = int(sys.argv[1]) if len(sys.argv) > 1 else 96        # per rank
    e_local = experts // world
    full = synthetic_weights(dev, 7, hidden, experts, inter, shared_inter, placement_ranks=world)
    mine = synthetic_weights(dev, 7, hidden, experts, inter, shared_inter, expert_range=(rank * e_local, (rank + 1) * e_local),
                             placement_ranks=world)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    x_all = torch.randn((tokens * world, hidden), device=dev, generator=g).to(torch.bfloat16)
    ga = float(2688.0 / x_all.float().abs().max().item())
    ga_dn = ga_sh = 2688.0 / 8.0
    ref = MoeLayer(full, tokens * world, topk, ga, ga_dn, ga_sh)
    ref_out = ref.forward(x_all.view(torch.int16)).clone()
    ep = EpMoeLayer(mine, tokens, topk, ga, ga_dn, ga_sh)
    sl = slice(rank * tokens, (rank + 1) * tokens)
    for _ in range(2):     # twice: buffers are reused across layers
        out = ep.forward(x_all[sl].contiguous().view(torch.int16))
        torch.cuda.synchronize()
        lib.gemb_check_device_status()
        assert torch.equal(ep.local.ids, ref.ids[sl]), "expert ids differ"
        assert torch.equal(ep.local.weights, ref.weights[sl]), "routing weights differ"
        assert torch.equal(ep.counts_all.sum(0).to(torch.int32), ref.counts), "global counts differ"
        assert torch.equal(out, ref_out[sl]), "expert-parallel output differs from the single-GPU layer"
    # the same layer with the exchange done by the library's own kernels over peer memory, ordered
    # by the library's flag barrier and by NCCL collectives
    for sync in ("flags", "nccl"):
        pull = EpPullMoeLayer(mine, tokens, topk, ga, ga_dn, ga_sh, sync=sync)
        for _ in range(3):     # three times: send and output buffers are reused without a host sync in between
            out = pull.forward(x_all[sl].contiguous().view(torch.int16))
        torch.cuda.synchronize()
        lib.gemb_check_device_status()
        assert torch.equal(pull.counts_all.sum(0).to(torch.int32), ref.counts), f"global counts differ (peer path, {sync})"
        assert int(pull.recv_prefix[-1].item()) == ep.last["n_recv"], f"received row count differs (peer path, {sync})"
        assert torch.equal(out, ref_out[sl]), f"peer-memory expert-parallel output differs from the single-GPU layer ({sync})"
    # the library's own layer call (gemb_moe_ep_layer_forward): pack, fused barrier + positions, pull, grouped GEMMs
    # whose epilogue pushes every row to the token's owner, combine from the local receive buffer
    for fused in (True, False):
        layer = EpLayer(mine, tokens, topk, ga, ga_dn, ga_sh, fused=fused)
        ref.fused = fused
        want = ref.forward(x_all.view(torch.int16)).clone()
        for _ in range(4):     # every buffer is reused without a host sync in between
            out = layer.forward(x_all[sl].contiguous().view(torch.int16))
        torch.cuda.synchronize()
        lib.gemb_check_device_status()
        assert torch.equal(layer.ids, ref.ids[sl]) and torch.equal(layer.weights, ref.weights[sl]), "routing differs (library layer)"
        assert torch.equal(layer.counts_all.sum(0).to(torch.int32), ref.counts), "global counts differ (library layer)"
        assert torch.equal(out, want[sl]), f"library expert-parallel layer differs from the single-GPU layer (fused={fused})"
        if fused and tokens > 1024:
            # the two-half schedule of large batches (first half's push beside the second half's gate/up GEMM on
            # disjoint SMs), with the grouped GEMMs forced onto CTA pairs as a full-size batch would have them
            lib.gemb_set_tuning(5, 2)
            lib.gemb_set_tuning(10, 74)
            try:
                for _ in range(3):
                    out = layer.forward(x_all[sl].contiguous().view(torch.int16))
                torch.cuda.synchronize()
                lib.gemb_check_device_status()
                assert torch.equal(out, want[sl]), "two-half schedule differs from the single-GPU layer"
            finally:
                lib.gemb_set_tuning(10, 0)
                lib.gemb_set_tuning(5, 0)
    dist.barrier()
    print(f"rank {rank} ok n_recv={ep.last['n_recv']} peer={pull.send.how}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
