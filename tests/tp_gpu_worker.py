"""One NCCL rank of the tensor-parallel MLP test: the sharded result must match the unsharded
one within the GEMM gate (the sum over K is split, so 1-ulp bf16 flips are allowed)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from gem16_b200 import load  # noqa: E402
from gem16_b200.tp import TpMlp  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    lib = load()
    tokens, hidden, inter = 300, 3840, 15360
    g = torch.Generator(device=dev)
    g.manual_seed(3)

    def quant(rows, k):
        w = torch.randn((rows, k), device=dev, generator=g) * 0.02
        div = float(2688.0 / w.abs().max().item())
        p = torch.empty((rows, k // 2), dtype=torch.uint8, device=dev)
        s = torch.empty((rows, k // 16), dtype=torch.uint8, device=dev)
        lib.gemb_nvfp4_quantize(w, 0, p, s, rows, k, div, 0, 0, None)
        return p, s, div

    gate, up, down = quant(inter, hidden), quant(inter, hidden), quant(hidden, inter)
    x = torch.randn((tokens, hidden), device=dev, generator=g).to(torch.bfloat16).view(torch.int16)
    ga, ga_dn = 700.0, 2688.0 / 0.05
    mlp = TpMlp(dev, gate, up, down, tokens, ga, ga_dn, reduce="peer")
    sharded = mlp.forward(x).clone()
    again = mlp.forward(x)          # buffers and barrier epochs are reused
    assert torch.equal(sharded, again), "peer reduction is not repeatable"
    via_nccl = TpMlp(dev, gate, up, down, tokens, ga, ga_dn, reduce="nccl").forward(x)
    solo_group = dist.new_group([rank]) if False else None
    # unsharded reference on every rank: same class with a one-rank group
    groups = [dist.new_group([r]) for r in range(world)]
    full = TpMlp(dev, gate, up, down, tokens, ga, ga_dn, group=groups[rank]).forward(x)
    torch.cuda.synchronize()
    lib.gemb_check_device_status()
    for name, got in (("peer", sharded), ("nccl", via_nccl)):
        a, b = got.float(), full.float()
        rel = float((a - b).norm() / b.norm())
        mism = float((a != b).float().mean())
        assert rel <= 1e-3 and mism < 0.05, (name, rel, mism)
    # every rank holds the same bits after the gather
    mine = sharded.view(torch.int16).to(torch.int32).sum().reshape(1).double()
    both = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(both, mine)
    assert all(float(v) == float(both[0]) for v in both), "ranks disagree after the peer all-gather"
    dist.barrier()
    print(f"rank {rank} ok rel={rel:.2e} mismatch={mism:.4f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
