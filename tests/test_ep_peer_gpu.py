"""The peer-memory expert-parallel protocol (csrc/ep.cu) on ONE GPU: the ranks are emulated by running
every rank's stages in turn, their "peer" buffers being ordinary buffers of the same device.  The
kernels, the position arithmetic and the launch sequence are the ones the multi-GPU layer uses; only
the two NCCL collectives are replaced by a host-side copy of the counts.  Result: bit-identical to the
single-GPU layer."""
import numpy as np
import pytest
import torch

from gem16_b200.ep import EpPullMoeLayer
from gem16_b200.moe import MoeLayer, synthetic_weights
from tests.moe_ref import ep_plan_reference

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ranks,tokens", [(2, 96), (4, 33), (8, 5)])
def test_emulated_ranks_match_single_gpu(lib, dev, ranks, tokens):
    hidden, experts, inter, shared_inter, topk = 2816, 128, 704, 2112, 8
    el = experts // ranks
    full = synthetic_weights(dev, 7, hidden, experts, inter, shared_inter, placement_ranks=ranks)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    x_all = torch.randn((tokens * ranks, hidden), device=dev, generator=g).to(torch.bfloat16)
    ga = float(2688.0 / x_all.float().abs().max().item())
    ga_dn = ga_sh = 2688.0 / 8.0
    ref = MoeLayer(full, tokens * ranks, topk, ga, ga_dn, ga_sh)
    ref_out = ref.forward(x_all.view(torch.int16)).clone()
    layers = []
    for r in range(ranks):
        mine = synthetic_weights(dev, 7, hidden, experts, inter, shared_inter, expert_range=(r * el, (r + 1) * el),
                                 placement_ranks=ranks)
        layers.append(EpPullMoeLayer(mine, tokens, topk, ga, ga_dn, ga_sh, emulate=(r, ranks)))
    EpPullMoeLayer.connect(layers)
    for rep in range(2):    # twice: every buffer is reused
        for r, l in enumerate(layers):
            l.stage_send(x_all[r * tokens:(r + 1) * tokens].contiguous().view(torch.int16))
        counts_all = torch.stack([l.local.counts for l in layers]).contiguous()
        for l in layers:
            l.counts_all.copy_(counts_all)
            l.stage_experts()
        outs = [l.stage_combine().clone() for l in layers]
        torch.cuda.synchronize()
        lib.gemb_check_device_status()
        c = counts_all.cpu().numpy().astype(np.int64)
        assert np.array_equal(c.sum(0), ref.counts.cpu().numpy())
        for r, l in enumerate(layers):
            want = ep_plan_reference(c, r)
            assert np.array_equal(l.row_base.cpu().numpy(), want["row_base"])
            assert np.array_equal(l.recv_prefix.cpu().numpy(), want["prefix"])
            assert np.array_equal(l.recv_src.cpu().numpy(), want["src"])
            assert np.array_equal(l.recv_dst.cpu().numpy(), want["dst"])
            plan = l.l_plan.cpu().numpy()
            assert plan[1] == want["padded_rows"] and plan[0] == want["padded_rows"] // 128
            assert np.array_equal(plan[2:2 + el], want["pad_local"])
            assert torch.equal(outs[r], ref_out[r * tokens:(r + 1) * tokens]), f"rank {r} output differs (pass {rep})"


@pytest.mark.parametrize("ranks,tokens,fused", [(2, 96, True), (2, 96, False), (4, 33, True), (8, 5, True), (8, 300, True)])
def test_library_ep_layer_emulated_ranks_match_single_gpu(lib, dev, ranks, tokens, fused):
    """gemb_moe_ep_layer_stage walked over all emulated ranks of one GPU (message rows with the
    assignment index pushed into the owner's buffer, positions from the counts, gather, grouped GEMMs whose epilogue stores each row
    into the token owner's receive buffer, combine from that buffer): output, ids, weights and
    counts bit-identical to the single-GPU layer, three passes over reused buffers."""
    from gem16_b200.ep import EpLayer
    hidden, experts, inter, shared_inter, topk = 2816, 128, 704, 2112, 8
    el = experts // ranks
    full = synthetic_weights(dev, 7, hidden, experts, inter, shared_inter, placement_ranks=ranks)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    ga_dn = ga_sh = 2688.0 / 8.0
    layers = []
    for r in range(ranks):
        mine = synthetic_weights(dev, 7, hidden, experts, inter, shared_inter, expert_range=(r * el, (r + 1) * el),
                                 placement_ranks=ranks)
        layers.append(EpLayer(mine, tokens, topk, 600.0, ga_dn, ga_sh, emulate=(r, ranks), fused=fused))
    EpLayer.connect(layers)
    ref = MoeLayer(full, tokens * ranks, topk, 600.0, ga_dn, ga_sh, stages=False)
    ref.fused = fused
    for rep in range(3):
        x_all = torch.randn((tokens * ranks, hidden), device=dev, generator=g).to(torch.bfloat16)
        ref_out = ref.forward(x_all.view(torch.int16)).clone()
        for r, l in enumerate(layers):
            l.stage(0, x_all[r * tokens:(r + 1) * tokens].contiguous().view(torch.int16))
        counts_all = torch.stack([l.counts for l in layers]).contiguous()
        for l in layers:
            l.counts_all.copy_(counts_all)
            l.stage(1)
        outs = [l.stage(2).clone() for l in layers]
        torch.cuda.synchronize()
        lib.gemb_check_device_status()
        assert torch.equal(counts_all.sum(0).to(torch.int32), ref.counts)
        for r, l in enumerate(layers):
            sl = slice(r * tokens, (r + 1) * tokens)
            assert torch.equal(l.ids, ref.ids[sl]) and torch.equal(l.weights, ref.weights[sl])
            assert torch.equal(outs[r], ref_out[sl]), f"rank {r} output differs (pass {rep})"


def test_ep_plan_rejects_bad_geometry(lib, dev):
    from gem16_b200.lib import GembError
    z = torch.zeros((64,), dtype=torch.int32, device=dev)
    with pytest.raises(GembError):
        lib.gemb_moe_ep_plan(z, 3, 128, 0, z, z, z, z, z, 128, 128, None)      # experts not a multiple of ranks
    with pytest.raises(GembError):
        lib.gemb_moe_ep_plan(z, 2, 128, 2, z, z, z, z, z, 128, 128, None)      # rank out of range
    with pytest.raises(GembError):
        lib.gemb_moe_ep_plan(None, 2, 128, 0, z, z, z, z, z, 128, 128, None)


def test_pull_dispatch_skips_rows_outside_the_buffers(lib, dev):
    """Positions that do not fit the buffers (counts that are not what the protocol promises) are
    skipped and reported through gemb_check_device_status(); nothing is read or written there."""
    import ctypes as C
    from gem16_b200.lib import GembError
    hidden, msg, send_rows, rows_max = 128, 80, 4, 128
    send = torch.full((send_rows, msg), 7, dtype=torch.uint8, device=dev)
    table = (C.c_uint64 * 1)(send.data_ptr())
    packed = torch.zeros((rows_max, hidden // 2), dtype=torch.uint8, device=dev)
    scales = torch.zeros((lib.cdll.gemb_interleaved_scale_bytes(rows_max, hidden),), dtype=torch.uint8, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    prefix = torch.tensor([0, 4], **i32)
    ok_src, ok_dst = torch.tensor([0], **i32), torch.tensor([0], **i32)
    lib.gemb_moe_ep_pull_dispatch(table, 1, 1, prefix, ok_src, ok_dst, packed, scales, hidden, msg, send_rows, rows_max, None)
    torch.cuda.synchronize()
    lib.gemb_check_device_status()
    assert int(packed[:4].min().item()) == 7 and int(packed[4:].max().item()) == 0
    packed.zero_()
    bad_src = torch.tensor([2], **i32)          # rows 2..5 of a 4-row send buffer
    lib.gemb_moe_ep_pull_dispatch(table, 1, 1, prefix, bad_src, ok_dst, packed, scales, hidden, msg, send_rows, rows_max, None)
    torch.cuda.synchronize()
    with pytest.raises(GembError):
        lib.gemb_check_device_status()
    assert int(packed[:2].min().item()) == 7 and int(packed[2:].max().item()) == 0   # in-range rows copied, the rest skipped
    lib.gemb_check_device_status()              # the record is cleared once read


def test_flag_barrier_and_count_gather_single_rank(lib, dev):
    """One rank: the barrier publishes and observes its own epoch (several times: the epoch lives on the
    device), and the count gather copies the rank's counts.  The multi-rank form runs in
    tests/test_ep_gpu.py, one rank per GPU."""
    import ctypes as C
    flags = torch.zeros((32,), dtype=torch.int32, device=dev)
    epochs = torch.zeros((2,), dtype=torch.int32, device=dev)
    table = (C.c_uint64 * 1)(flags.data_ptr())
    for _ in range(3):
        lib.gemb_moe_ep_barrier(table, 1, 0, 0, epochs, None)
    lib.gemb_moe_ep_barrier(table, 1, 0, 1, epochs, None)
    torch.cuda.synchronize()
    lib.gemb_check_device_status()
    assert epochs.tolist() == [3, 1] and int(flags[0]) == 3 and int(flags[16]) == 1
    counts = torch.arange(128, dtype=torch.int32, device=dev)
    out = torch.zeros((1, 128), dtype=torch.int32, device=dev)
    lib.gemb_moe_ep_gather_counts((C.c_uint64 * 1)(counts.data_ptr()), 1, 128, out, None)
    torch.cuda.synchronize()
    assert torch.equal(out[0], counts)
    from gem16_b200.lib import GembError
    with pytest.raises(GembError):
        lib.gemb_moe_ep_barrier(table, 1, 0, 2, epochs, None)      # only barriers 0 and 1 exist
    with pytest.raises(GembError):
        lib.gemb_moe_ep_barrier(table, 1, 1, 0, epochs, None)      # rank out of range


def test_flag_barrier_gives_up_and_reports(lib, dev):
    """The failure-detection path of the expert-parallel layer: a rank whose peer never reaches the barrier.
    Two ranks are declared, both flag arrays are buffers of this GPU, and only rank 0's barrier kernel
    ever runs, so the second slot of its array stays behind.  With the poll limit turned down to about a
    millisecond the kernel gives up, returns, and leaves code 5 for gemb_check_device_status (kInternal,
    reported once); the context stays usable and the next launch works.  Nothing here waits on
    another kernel: the flag is simply never written."""
    import ctypes as C
    from gem16_b200.lib import GembError
    mine = torch.zeros((32,), dtype=torch.int32, device=dev)
    theirs = torch.zeros((32,), dtype=torch.int32, device=dev)
    epochs = torch.zeros((2,), dtype=torch.int32, device=dev)
    table = (C.c_uint64 * 2)(mine.data_ptr(), theirs.data_ptr())
    lib.gemb_set_tuning(6, 2000)          # GEMB_TUNE_EP_BARRIER_SPINS: 2,000 polls of about 500 ns
    try:
        lib.gemb_moe_ep_barrier(table, 2, 0, 0, epochs, None)
        torch.cuda.synchronize()
        with pytest.raises(GembError) as err:
            lib.gemb_check_device_status()
        assert err.value.status_name == "kInternal" and "barrier" in str(err.value)
        lib.gemb_check_device_status()                       # the record is cleared once read
        # rank 0 did publish its epoch to both arrays before it gave up
        assert int(mine[0]) == 1 and int(theirs[0]) == 1 and int(mine[1]) == 0
        # once the peer's flag arrives (written here by the host), the same barrier passes
        mine[1] = 2
        lib.gemb_moe_ep_barrier(table, 2, 0, 0, epochs, None)
        torch.cuda.synchronize()
        lib.gemb_check_device_status()
        assert epochs.tolist() == [2, 0]
    finally:
        lib.gemb_set_tuning(6, 0)


def test_plan_with_impossible_counts_is_empty_and_recorded(lib, dev):
    """Counts that the protocol cannot produce (what a rank would read if it went on after a barrier gave
    up): more padded rows than the buffers hold, a negative count, more rows than a rank can send.  The plan
    kernel writes an empty plan and records code 6; the grouped GEMM then has no tile to run and the
    combine skips every row."""
    from gem16_b200.lib import GembError
    ranks, experts, el, cap, send_rows = 2, 8, 4, 1024, 256
    i32 = dict(dtype=torch.int32, device=dev)

    def plan_for(counts):
        plan = torch.full((lib.cdll.gemb_moe_ep_plan_ints(cap, el),), 77, **i32)
        prefix, src, dst = torch.full((ranks * el + 1,), 77, **i32), torch.full((ranks * el,), 77, **i32), torch.full((ranks * el,), 77, **i32)
        base = torch.full((experts,), 77, **i32)
        lib.gemb_moe_ep_plan(torch.tensor(counts, **i32), ranks, experts, 0, plan, prefix, src, dst, base, cap, send_rows, None)
        torch.cuda.synchronize()
        return plan.cpu().numpy(), prefix.cpu().numpy(), base.cpu().numpy()

    good = [[30, 30, 30, 30, 34, 34, 34, 34], [10, 20, 30, 40, 39, 39, 39, 39]]
    plan, prefix, base = plan_for(good)
    lib.gemb_check_device_status()
    assert plan[0] == 8 and plan[1] == 1024 and prefix[-1] == 220      # four experts, each padded to 256 rows
    for bad in ([[200, 200, 200, 200, 0, 0, 0, 0], [250, 250, 250, 250, 0, 0, 0, 0]],      # 4 x 512 padded rows > 1,024; 800 > 256 sent
                [[30, -1, 30, 30, 34, 34, 34, 34], good[1]],                                # a negative count
                [[64, 64, 64, 64, 1, 0, 0, 0], good[1]]):                                   # rank 0 would have sent 257 rows
        plan, prefix, base = plan_for(bad)
        with pytest.raises(GembError) as err:
            lib.gemb_check_device_status()
        assert err.value.status_name == "kInternal"
        assert plan[0] == 0 and plan[1] == 0 and not prefix.any() and (base < -cap).all()
