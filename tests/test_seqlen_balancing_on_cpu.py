import pytest
import torch

from verl_b200.utils.seqlen_balancing import (get_reverse_idx, get_seqlen_balanced_partitions, karmarkar_karp,
                                               rearrange_micro_batches, restore_dynamic_batch)


def test_partitions_cover_all_and_balance():
    torch.manual_seed(0)
    lens = torch.randint(10, 2000, (64,)).tolist()
    parts = get_seqlen_balanced_partitions(lens, 8, equal_size=True)
    assert sorted(i for p in parts for i in p) == list(range(64)) and all(len(p) == 8 for p in parts)
    sums = [sum(lens[i] for i in p) for p in parts]
    assert max(sums) - min(sums) < 0.05 * (sum(lens) / 8)


def test_karmarkar_karp_unequal_sizes():
    parts = karmarkar_karp([8, 7, 6, 5, 4], 2, equal_size=False)
    sums = sorted(sum([8, 7, 6, 5, 4][i] for i in p) for p in parts)
    assert sums == [14, 16] or sums == [15, 15]


def test_equal_size_requires_divisibility():
    with pytest.raises(AssertionError):
        karmarkar_karp([1, 2, 3], 2, equal_size=True)


def test_rearrange_micro_batches_respects_budget_and_restores_order():
    torch.manual_seed(1)
    lens = torch.randint(50, 500, (20,))
    parts = rearrange_micro_batches(lens, max_token_len=1200)
    assert sorted(i for p in parts for i in p) == list(range(20))
    assert all(sum(int(lens[i]) for i in p) <= 1200 for p in parts)
    data = torch.arange(20)
    cat = torch.cat([data[torch.tensor(p)] for p in parts])
    assert torch.equal(restore_dynamic_batch(cat, parts), data)


def test_reverse_idx():
    assert get_reverse_idx([2, 0, 1]) == [1, 2, 0]
