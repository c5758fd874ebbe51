"""One gloo rank of the CPU tensor-parallel MLP test: column-split gate/up, K-split down with an
all-reduce of the partial sums, checked against the unsharded oracle (launched by
tests/test_ep_cpu.py)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import Oracle  # noqa: E402
from tests.util import bf16_round  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    orc = Oracle()
    rng = np.random.default_rng(5)
    tokens, hidden, inter = 9, 128, 256
    x = bf16_round(rng.standard_normal((tokens, hidden)).astype(np.float32))
    ga, ga_dn = 600.0, 300.0

    def quant(rows, k):
        w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
        g = float(np.float32(2688.0) / np.abs(w).max())
        return orc.nvfp4_quantize(w, g) + (g,)

    gate, up, down = quant(inter, hidden), quant(inter, hidden), quant(hidden, inter)
    xq, xs = orc.nvfp4_quantize(x, ga)

    def mlp(rows_slice):
        g = bf16_round(orc.nvfp4_matmul(xq, xs, gate[0][rows_slice], gate[1][rows_slice], ga, gate[2]).astype(np.float32))
        u = bf16_round(orc.nvfp4_matmul(xq, xs, up[0][rows_slice], up[1][rows_slice], ga, up[2]).astype(np.float32))
        p = orc.gated_gelu(g, u)
        pq, ps = orc.nvfp4_quantize(p, ga_dn)      # block scales run along the local features only
        lo, hi = rows_slice.start, rows_slice.stop
        return orc.nvfp4_matmul(pq, ps, np.ascontiguousarray(down[0][:, lo // 2:hi // 2]),
                                np.ascontiguousarray(down[1][:, lo // 16:hi // 16]), ga_dn, down[2])

    il = inter // world
    partial = torch.from_numpy(mlp(slice(rank * il, (rank + 1) * il)))
    dist.all_reduce(partial)
    full = mlp(slice(0, inter))
    err = np.abs(partial.numpy() - full).max() / np.abs(full).max()
    assert err < 1e-12, err
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
