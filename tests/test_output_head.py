"""Output head (tied bf16 logits + soft cap + suppression + arg-max): CPU checks of the oracle's
selection rule, GPU parity of the fused kernel against the oracle."""
import numpy as np
import pytest
import torch


def select(logits, suppressed):
    """The reference's rule on given logits: larger value wins, ties to the lower id, suppressed ids never."""
    out = []
    for row in logits:
        masked = row.astype(np.float64).copy()
        masked[list(suppressed)] = -np.inf
        out.append(int(np.flatnonzero(masked == masked.max())[0]))
    return np.array(out, np.uint32)


def make_case(orc, rows, vocab, hidden, seed):
    rng = np.random.default_rng(seed)
    w = orc.to_bf16((rng.standard_normal((vocab, hidden)) * 0.05).astype(np.float32))
    h = (rng.standard_normal((rows, hidden)) * 2.0).astype(np.float32)
    return w, h


def test_oracle_selection_rule(orc):
    w, h = make_case(orc, 2, 512, 64, 1)
    w[7] = w[3]                                  # an exact tie between ids 3 and 7
    logits, sel = orc.output_head(w, h)
    assert logits.shape == (2, 512) and np.all(np.abs(logits) <= 30.0)
    assert np.array_equal(logits[:, 3], logits[:, 7])
    assert np.array_equal(sel, select(logits, []))
    top = int(sel[0])
    logits2, sel2 = orc.output_head(w, h, suppressed=[top])
    assert np.array_equal(logits, logits2) and sel2[0] != top
    assert np.array_equal(sel2, select(logits, [top]))
    # soft cap: a huge dot product saturates at +-30
    big = orc.to_bf16(np.full((1, 64), 50.0, np.float32))
    lg, _ = orc.output_head(big, np.full((1, 64), 50.0, np.float32))
    assert lg[0, 0] == np.float32(30.0)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,vocab,hidden,suppress", [(1, 4096 * 8 + 5, 3840, 0), (1, 1000, 64, 3), (3, 40000, 3840, 2),
                                                        (5, 9000, 2816, 1), (8, 4000, 512, 0)])
def test_output_head_matches_oracle(lib, dev, orc, rows, vocab, hidden, suppress):
    w, h = make_case(orc, rows, vocab, hidden, 10 * rows + suppress)
    want_logits, _ = orc.output_head(w, h)
    sup = list(np.argsort(-want_logits[0])[:suppress].astype(np.uint32))   # ban the best tokens of row 0
    blocks = lib.cdll.gemb_output_head_candidate_blocks()
    assert blocks == 4096
    wd = torch.from_numpy(w.view(np.int16)).to(dev)
    hd = torch.from_numpy(h).to(dev)
    sd = torch.tensor([int(s) for s in sup], dtype=torch.int32, device=dev) if sup else None
    cand = torch.full((rows, blocks, 2), -1, dtype=torch.int32, device=dev)
    logits = torch.full((rows, vocab), float("nan"), device=dev)
    selected = torch.full((rows,), -1, dtype=torch.int32, device=dev)
    lib.gemb_output_head_candidates(wd, hd, rows, sd, len(sup), None, cand, logits, vocab, hidden, None)
    lib.gemb_output_head_argmax(cand, rows, selected, None)
    torch.cuda.synchronize()
    got = logits.cpu().numpy()
    assert np.isfinite(got).all()
    # fp32 accumulation in a different order than binary64: tolerance on the capped logits
    assert np.abs(got - want_logits).max() <= 2e-5 * max(1.0, np.abs(want_logits).max()), np.abs(got - want_logits).max()
    # the selection itself is exact: the reference's rule applied to the kernel's own logits
    sel = selected.cpu().numpy().astype(np.uint32)
    assert np.array_equal(sel, select(got, sup))
    for s in sup:
        assert int(s) not in sel.tolist()
    # and it is the oracle's token whenever the oracle's top two are further apart than the tolerance
    _, want_sel = orc.output_head(w, h, suppressed=sup)
    for r in range(rows):
        masked = want_logits[r].astype(np.float64).copy()
        masked[[int(s) for s in sup]] = -np.inf
        top2 = np.sort(masked)[-2:]
        if top2[1] - top2[0] > 1e-4:
            assert sel[r] == want_sel[r]
    # same launch without the diagnostic logits and with the run-time suppression count
    cand2 = torch.full((rows, blocks, 2), -1, dtype=torch.int32, device=dev)
    dyn = torch.tensor([len(sup)], dtype=torch.int32, device=dev)
    pad = torch.cat([sd, torch.zeros(4, dtype=torch.int32, device=dev)]) if sup else torch.zeros(4, dtype=torch.int32, device=dev)
    lib.gemb_output_head_candidates(wd, hd, rows, pad, pad.numel(), dyn, cand2, None, vocab, hidden, None)
    torch.cuda.synchronize()
    assert torch.equal(cand, cand2)


@pytest.mark.gpu
def test_output_head_ties_and_validation(lib, dev, orc):
    from gem16_b200.lib import GembError
    w, h = make_case(orc, 1, 2048, 128, 3)
    w[1500] = w[20]
    w[20] = orc.to_bf16(np.full((128,), 3.0, np.float32) * np.sign(h[0]))   # a clear winner, twice
    w[1500] = w[20]
    wd, hd = torch.from_numpy(w.view(np.int16)).to(dev), torch.from_numpy(h).to(dev)
    cand = torch.zeros((1, 4096, 2), dtype=torch.int32, device=dev)
    sel = torch.zeros((1,), dtype=torch.int32, device=dev)
    lib.gemb_output_head_candidates(wd, hd, 1, None, 0, None, cand, None, 2048, 128, None)
    lib.gemb_output_head_argmax(cand, 1, sel, None)
    torch.cuda.synchronize()
    assert int(sel[0]) == 20                    # the lower id of the tie
    with pytest.raises(GembError):
        lib.gemb_output_head_candidates(wd, hd, 9, None, 0, None, cand, None, 2048, 128, None)     # too many rows
    with pytest.raises(GembError):
        lib.gemb_output_head_candidates(wd, hd, 1, None, 2, None, cand, None, 2048, 128, None)     # list without pointer
    with pytest.raises(GembError):
        lib.gemb_output_head_candidates(wd, hd, 1, None, 0, None, cand, None, 2048, 100, None)     # hidden % 8
    with pytest.raises(GembError):
        lib.gemb_output_head_argmax(None, 1, sel, None)
