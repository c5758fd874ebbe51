"""CPU tests of the MoE restatement against the known-answer cases the gem16 plan lists
(docs/plans/gemma4-26b/specs/MOE_ROUTER_SPEC.md:59-63, MOE_PREFILL_KERNEL_SPEC.md:136-147,
specs/TEST_MATRIX.md:52-63).  The reference ships no executable MoE code: these KATs, derived
from the specifications, are what pins the restatement."""
import numpy as np
import pytest


def test_all_equal_logits_pick_lowest_ids(orc):
    ids, w = orc.moe_route(np.zeros((3, 128), np.float32), 8)
    assert ids.tolist() == [list(range(8))] * 3
    assert np.all(w == np.float32(0.125))


def test_ties_at_the_boundary_go_to_lower_id(orc):
    lg = np.full((1, 128), -5.0, np.float32)
    lg[0, [100, 90, 80, 70, 60, 50, 40]] = [7, 6, 5, 4, 3, 2, 1]      # ranks 0..6 distinct
    lg[0, [33, 17, 99]] = 0.5                                          # three-way tie for rank 7
    ids, w = orc.moe_route(lg, 8)
    assert ids[0].tolist() == [100, 90, 80, 70, 60, 50, 40, 17]
    assert abs(float(w.sum()) - 1.0) < 1e-6 and np.all(np.diff(w[0]) <= 0)


def test_one_dominant_expert(orc):
    lg = np.zeros((1, 128), np.float32)
    lg[0, 77] = 60.0
    ids, w = orc.moe_route(lg, 8)
    assert ids[0, 0] == 77 and ids[0, 1:].tolist() == list(range(7))
    assert w[0, 0] > 0.999999 and w[0, 1] < 1e-20


def test_per_expert_scale_applied_after_renormalisation(orc):
    rng = np.random.default_rng(0)
    lg = rng.standard_normal((5, 64)).astype(np.float32)
    scale = rng.uniform(0.5, 2.0, 64).astype(np.float32)
    ids, w = orc.moe_route(lg, 8)
    ids2, w2 = orc.moe_route(lg, 8, per_expert_scale=scale)
    assert np.array_equal(ids, ids2)
    assert np.array_equal(w2, w * scale[ids])            # one fp32 multiply, no second renorm


def test_probabilities_and_exp(orc):
    rng = np.random.default_rng(1)
    lg = (rng.standard_normal((16, 128)) * 3).astype(np.float32)
    ids, w, p = orc.moe_route(lg, 8, want_probs=True)
    ref = np.exp(lg.astype(np.float64) - lg.max(1, keepdims=True)); ref /= ref.sum(1, keepdims=True)
    assert np.abs(p - ref).max() < 1e-6 and np.abs(p.sum(1) - 1).max() < 1e-5
    order = np.argsort(-ref, axis=1, kind="stable")[:, :8]
    assert np.array_equal(ids, order)
    xs = np.linspace(-87, 0, 2001).astype(np.float32)
    got = np.array([orc.det_exp(float(v)) for v in xs])
    assert np.abs(got / np.exp(xs.astype(np.float64)) - 1).max() < 3e-7
    assert orc.det_exp(0.0) == 1.0 and orc.det_exp(-100.0) == 0.0


def test_invalid_router_inputs(orc):
    with pytest.raises(ValueError):
        orc.moe_route(np.zeros((1, 100), np.float32), 8)        # experts not a multiple of 32
    lg = np.zeros((1, 128), np.float32); lg[0, 3] = np.nan
    with pytest.raises(ValueError):
        orc.moe_route(lg, 8)
    with pytest.raises(ValueError):
        orc.moe_permute(np.array([[0, 200]], np.int32), 128)


@pytest.mark.parametrize("tokens", [1, 17, 511, 512, 1023])
def test_stable_permutation_round_trip(orc, tokens):
    # chunk sizes of docs/plans/gemma4-26b/milestones/M15_GROUPED_MOE_PREFILL.md:50-57
    rng = np.random.default_rng(tokens)
    lg = (rng.standard_normal((tokens, 128)) + rng.standard_normal(128) * 2).astype(np.float32)
    ids, _ = orc.moe_route(lg, 8)
    counts, offsets, perm = orc.moe_permute(ids, 128)
    flat = ids.reshape(-1)
    assert counts.sum() == tokens * 8 and np.array_equal(counts, np.bincount(flat, minlength=128))
    assert np.array_equal(offsets, np.concatenate([[0], np.cumsum(counts)]))
    assert np.array_equal(np.sort(perm), np.arange(tokens * 8))          # nothing lost or duplicated
    for e in range(128):
        seg = perm[offsets[e]:offsets[e + 1]]
        assert np.all(flat[seg] == e) and np.all(np.diff(seg) > 0)       # token asc, then slot asc
    for row in ids:
        assert len(set(row.tolist())) == 8                               # no duplicate selected id


def test_zero_hit_and_all_hit_experts(orc):
    ids = np.tile(np.arange(8, dtype=np.int32), (40, 1))                  # only experts 0..7 used
    counts, offsets, perm = orc.moe_permute(ids, 128)
    assert counts[:8].tolist() == [40] * 8 and not counts[8:].any()
    ids = (np.arange(128 * 8, dtype=np.int32).reshape(128, 8)) % 128      # every expert hit 8 times
    counts, _, _ = orc.moe_permute(ids, 128)
    assert counts.tolist() == [8] * 128


def test_combine_is_slot_ordered_fma(orc):
    from tests.util import bf16_bits, from_bf16_bits
    rng = np.random.default_rng(2)
    y = bf16_bits(rng.standard_normal((3, 8, 64)).astype(np.float32))
    w = rng.uniform(0, 0.3, (3, 8)).astype(np.float32)
    sh = bf16_bits(rng.standard_normal((3, 64)).astype(np.float32))
    out = from_bf16_bits(orc.moe_combine(y, w, sh))
    ref = (from_bf16_bits(y).astype(np.float64) * w[:, :, None]).sum(1) + from_bf16_bits(sh)
    assert np.abs(out - ref).max() < 0.02
    only = from_bf16_bits(orc.moe_combine(y, w, None))
    assert np.abs(only - (ref - from_bf16_bits(sh))).max() < 0.02


def test_layer_shared_only_and_expert_only(orc):
    # "shared-only and expert-only synthetic layers" (MOE_SEMANTICS_SPEC.md:124-134)
    from tests.moe_ref import make_layer, moe_layer_oracle
    from tests.util import bf16_bits, from_bf16_bits
    rng = np.random.default_rng(3)
    p = make_layer(orc, rng, hidden=128, experts=32, inter=64, shared_inter=64)
    x = bf16_bits(rng.standard_normal((9, 128)).astype(np.float32))
    full = moe_layer_oracle(orc, p, x, 4, 600.0, 3000.0, 3000.0)
    q = dict(p); q.pop("sh_gu"); q.pop("sh_dn")
    experts_only = moe_layer_oracle(orc, q, x, 4, 600.0, 3000.0)
    assert np.array_equal(full["ids"], experts_only["ids"])
    diff = from_bf16_bits(full["out"]) - from_bf16_bits(experts_only["out"])
    assert np.abs(diff - full["shared"]).max() < 0.02 * max(1.0, np.abs(full["shared"]).max())
