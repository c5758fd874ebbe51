"""World-size-2 gloo test of the expert-parallel protocol on CPU: split sizes, arrival order,
stable regrouping by local expert and the reverse path must reproduce the single-process MoE
layer bit for bit."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ep_splits():
    from gem16_b200.ep import ep_splits
    counts = np.arange(2 * 8).reshape(2, 8)            # 2 ranks, 8 experts, 4 per rank
    send, recv = ep_splits(counts, 0, 4)
    assert send == [0 + 1 + 2 + 3, 4 + 5 + 6 + 7] and recv == [6, 8 + 9 + 10 + 11]
    send, recv = ep_splits(counts, 1, 4)
    assert send == [38, 54] and recv == [22, 54]


def test_expert_parallel_protocol_two_ranks():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(ROOT, "tests", "ep_cpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


def test_tensor_parallel_mlp_two_ranks():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29633", os.path.join(ROOT, "tests", "tp_cpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


def test_peer_protocol_positions_reproduce_the_single_gpu_order():
    """The position arithmetic of the peer-memory protocol (csrc/ep.cu, restated in
    tests/moe_ref.ep_plan_reference) against a brute-force model: R ranks each sort their own
    assignments by expert; the rows an owner pulls, placed at recv_dst + j, must come out in the
    single-GPU order (expert, global token, slot), every expert starting on a multiple of 128 rows,
    and combine_row_base + the sender's local padded row must name the same row."""
    import numpy as np
    from tests.moe_ref import ep_plan_reference
    rng = np.random.default_rng(0)
    for ranks, experts, tokens, topk in [(2, 8, 37, 2), (4, 16, 50, 4), (8, 128, 9, 8)]:
        el = experts // ranks
        ids = rng.integers(0, experts, (ranks, tokens * topk))          # expert of assignment (token*topk + slot)
        ids[:, : experts // 2] = 0                                        # a hot expert and some empty ones
        counts = np.stack([np.bincount(ids[r], minlength=experts) for r in range(ranks)])
        order = [np.argsort(ids[r], kind="stable") for r in range(ranks)]  # each rank's send buffer
        # single-GPU order over all ranks' tokens: stable sort of (rank, assignment) by expert
        flat = [(int(ids[r, a]), r, int(a)) for r in range(ranks) for a in range(tokens * topk)]
        flat.sort(key=lambda x: x[0])
        for me in range(ranks):
            plan = ep_plan_reference(counts, me)
            mine = [x for x in flat if me * el <= x[0] < (me + 1) * el]
            want_row = {}
            pos_in_expert = {}
            for e, r, a in mine:
                k = pos_in_expert.get(e, 0)
                want_row[(r, a)] = int(plan["pad_local"][e - me * el]) + k
                pos_in_expert[e] = k + 1
            assert all(v % 256 == 0 for v in plan["pad_local"])
            got_row = {}
            for s_rank in range(ranks):
                for e_loc in range(el):
                    g = s_rank * el + e_loc
                    n = int(plan["prefix"][g + 1] - plan["prefix"][g])
                    for j in range(n):
                        a = int(order[s_rank][plan["src"][g] + j])
                        assert ids[s_rank, a] == me * el + e_loc
                        got_row[(s_rank, a)] = int(plan["dst"][g]) + j
            assert got_row == want_row
            assert plan["prefix"][-1] == len(mine) and plan["padded_rows"] >= len(mine)
        # the token owner's view: local padded row of an assignment -> row in the expert owner's output
        for me in range(ranks):
            plan = ep_plan_reference(counts, me)
            my_pad = np.concatenate([[0], np.cumsum((counts[me] + 255) // 256 * 256)])
            my_off = np.concatenate([[0], np.cumsum(counts[me])])
            for p, a in enumerate(order[me]):
                e = int(ids[me, a])
                slot_row = my_pad[e] + (p - my_off[e])                 # what gemb_moe_permute's slot_rows holds
                owner = e // el
                owner_plan = ep_plan_reference(counts, owner)
                g = me * el + (e - owner * el)
                want = int(owner_plan["dst"][g]) + (p - int(my_off[e]))
                assert int(plan["row_base"][e]) + slot_row == want


def test_expert_placement_balances_a_saturating_prior():
    """Load-time placement (gem16_b200.moe.place_experts): with a Zipf(1.1) prior and top-8 routing the hottest
    expert alone is worth a rank's fair share at 8 ranks; the greedy placement by a calibration estimate keeps the
    fullest rank within a few per cent of the mean on fresh tokens, is a permutation of the prior, and is
    reproducible from the seed (every rank must derive the same placement)."""
    import torch
    from gem16_b200.moe import place_experts
    experts, hidden, topk = 128, 2816, 8
    g = torch.Generator().manual_seed(5)
    rank = torch.randperm(experts, generator=g).double() + 1
    bias = (-1.1 * torch.log(rank))
    bias = (bias - bias.mean()).float()
    for ranks in (2, 4, 8):
        placed = place_experts(bias, hidden, ranks, torch.Generator().manual_seed(9))
        again = place_experts(bias, hidden, ranks, torch.Generator().manual_seed(9))
        assert torch.equal(placed, again)
        assert torch.equal(torch.sort(placed).values, torch.sort(bias).values)
        fresh = torch.randn((16384, experts), generator=torch.Generator().manual_seed(77)) * (0.02 * hidden ** 0.5) + placed
        counts = torch.bincount(torch.topk(fresh, topk, dim=1).indices.reshape(-1), minlength=experts).double()
        per_rank = counts.view(ranks, -1).sum(1)
        assert float(per_rank.max() / per_rank.mean()) < 1.05, (ranks, per_rank.tolist())
