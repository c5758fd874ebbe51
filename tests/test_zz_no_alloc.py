"""GPU test of gemb_moe_permute_static, the permutation entry point for callers that cannot
allocate: hosts that own one load-time arena with no spare region, or code that runs where
cudaMalloc is forbidden.  It must give exactly the records gemb_moe_permute gives, also when it
is called twice in a row on different inputs (the built-in scratch keeps the previous call's
values and is never cleared).  Collected last so a failure here cannot hide another test."""
import numpy as np
import pytest
import torch

from gem16_b200.lib import GembError

pytestmark = pytest.mark.gpu


def routed_ids(tokens, experts, topk, seed):
    rng = np.random.default_rng(seed)
    logits = rng.standard_normal((tokens, experts)) + rng.standard_normal(experts) * 2
    return np.ascontiguousarray(np.argsort(-logits, axis=1, kind="stable")[:, :topk].astype(np.int32))


def run(lib, dev, ids, experts, static):
    t, k = ids.shape
    c = lib.cdll
    d_ids = torch.from_numpy(ids).to(dev)
    counts = torch.full((experts,), -1, dtype=torch.int32, device=dev)
    offsets = torch.full((experts + 1,), -1, dtype=torch.int32, device=dev)
    perm = torch.full((t * k,), -1, dtype=torch.int32, device=dev)
    rows = torch.full((t * k,), -1, dtype=torch.int32, device=dev)
    plan = torch.full((c.gemb_moe_plan_ints(t, experts, k),), -1, dtype=torch.int32, device=dev)
    if static:
        lib.gemb_moe_permute_static(d_ids, counts, offsets, perm, rows, plan, t, experts, k, None)
    else:
        ws = torch.empty((c.gemb_moe_permute_workspace_bytes(t, experts, k),), dtype=torch.uint8, device=dev)
        lib.gemb_moe_permute(d_ids, counts, offsets, perm, rows, plan, ws, ws.numel(), t, experts, k, None)
    torch.cuda.synchronize()
    tiles = int(plan[0].item())
    return [counts.cpu(), offsets.cpu(), perm.cpu(), rows.cpu(), plan[: 3 + experts + 2 * tiles + 1].cpu()]


def test_static_scratch_matches_workspace_variant_twice_in_a_row(lib, dev):
    # two back-to-back calls: a large problem first, then a smaller one that reuses (and must not
    # be disturbed by) the cells the first call left behind, then the large one again
    # (16 experts with top-1 is the sort an expert-parallel receiver does over its local experts)
    problems = [(4096, 128, 8, 1), (300, 64, 4, 2), (4096, 128, 8, 3), (16384, 128, 8, 4), (777, 16, 1, 5), (50, 3, 2, 6)]
    for tokens, experts, topk, seed in problems:
        ids = routed_ids(tokens, experts, topk, seed)
        got = run(lib, dev, ids, experts, static=True)
        want = run(lib, dev, ids, experts, static=False)
        for a, b in zip(got, want):
            assert torch.equal(a, b)
        assert int(got[0].sum()) == tokens * topk


def test_static_scratch_rejects_oversized_problems(lib, dev):
    p = torch.zeros((16,), dtype=torch.int32, device=dev)
    with pytest.raises(GembError) as e:
        lib.gemb_moe_permute_static(p, p, p, p, p, p, 16385, 128, 8, None)     # 131,080 assignments
    assert e.value.status_name == "kInvalidArgument" and "built-in scratch" in str(e.value)
