"""bench.py's rule for comparing chosen experts end to end: a swap between experts whose reference logits are nearly
tied is accepted, anything else is a mismatch.  (CPU only: the rule is host code.)"""
import torch

import bench


def test_near_tie_swap_is_accepted_and_a_real_difference_is_not():
    logits = torch.zeros((3, 16))
    logits[0, :9] = torch.tensor([9.0, 8.0, 7.0, 6.0, 5.0, 4.0, 3.0, 2.0, 2.0 - 2.0e-4])   # 8th and 9th nearly tied
    logits[1, :9] = torch.tensor([9.0, 8.0, 7.0, 6.0, 5.0, 4.0, 3.0, 2.0, 1.9])             # a clear gap
    logits[2, :9] = torch.tensor([9.0, 8.0, 7.0, 6.0, 5.0, 4.0, 3.0, 2.0, 1.0])
    ref = logits.topk(8, -1).indices
    got = ref.clone()
    got[0, 7] = 8          # picks the 9th instead of the 8th: a near tie
    assert bench.ids_differ_beyond_ties(got, ref, logits) == []
    got[1, 7] = 8          # the same swap across a gap of 0.1
    assert bench.ids_differ_beyond_ties(got, ref, logits) == [1]
    got[1] = ref[1].flip(0)  # order inside the top 8 does not matter
    assert bench.ids_differ_beyond_ties(got, ref, logits) == []
    assert bench.ids_differ_beyond_ties(got, ref, logits, tie=1e-4) == [0]  # the op-level tolerance rejects it
