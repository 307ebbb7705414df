import torch

from lplb_b200 import eplb


def test_balanced_packing_equal_cardinality_and_lpt_quality():
    g = torch.Generator().manual_seed(0)
    w = torch.rand(3, 64, generator=g) ** 3
    pack, rank = eplb.balanced_packing(w, 8)
    for row in range(3):
        counts = torch.bincount(pack[row], minlength=8)
        assert counts.tolist() == [8] * 8
        for p in range(8):
            assert sorted(rank[row][pack[row] == p].tolist()) == list(range(8))
        loads = torch.zeros(8).scatter_add_(0, pack[row], w[row])
        # LPT with a cardinality cap stays close to the mean
        assert loads.max() / loads.mean() < 1.15


def test_balanced_packing_one_item_per_pack_is_identity():
    w = torch.rand(2, 8)
    pack, rank = eplb.balanced_packing(w, 8)
    assert torch.equal(pack, torch.arange(8).expand(2, 8))
    assert int(rank.sum()) == 0


def test_balanced_packing_small_case_by_hand():
    # heaviest first: 9->p0, 8->p1, 7->p1?  loads p0=9,p1=8 -> 7 goes to p1 (lighter) -> p1=15,
    # 1 -> p0 (only one with room).
    w = torch.tensor([[9.0, 8.0, 7.0, 1.0]])
    pack, rank = eplb.balanced_packing(w, 2)
    assert pack.tolist() == [[0, 1, 1, 0]]
    assert rank.tolist() == [[0, 0, 1, 1]]


def test_replicate_experts_identity_and_greedy():
    w = torch.tensor([[4.0, 1.0, 1.0]])
    phy2log, rank, cnt = eplb.replicate_experts(w, 3)
    assert phy2log.tolist() == [[0, 1, 2]] and cnt.tolist() == [[1, 1, 1]]
    phy2log, rank, cnt = eplb.replicate_experts(w, 5)
    # 4/1 is the largest -> replicate 0; then 4/2=2 > 1 -> replicate 0 again
    assert phy2log.tolist() == [[0, 1, 2, 0, 0]]
    assert rank.tolist() == [[0, 0, 0, 1, 2]]
    assert cnt.tolist() == [[3, 1, 1]]


def test_rebalance_is_a_permutation_without_replicas():
    g = torch.Generator().manual_seed(1)
    w = torch.rand(2, 256, generator=g)
    phy2log, log2phy, logcnt = eplb.rebalance_experts(w, 256, 4, 2, 32)
    assert phy2log.shape == (2, 256) and log2phy.shape == (2, 256, 1)
    for layer in range(2):
        assert sorted(phy2log[layer].tolist()) == list(range(256))
        assert torch.equal(phy2log[layer][log2phy[layer, :, 0]], torch.arange(256))
    assert int(logcnt.min()) == 1 and int(logcnt.max()) == 1
    # rank loads are closer than in natural order
    per_rank = w.gather(1, phy2log).reshape(2, 32, 8).sum(-1)
    natural = w.reshape(2, 32, 8).sum(-1)
    assert (per_rank.max(1).values / per_rank.mean(1)).max() < (natural.max(1).values / natural.mean(1)).max()


def test_rebalance_groups_stay_on_their_node():
    g = torch.Generator().manual_seed(2)
    w = torch.rand(1, 64, generator=g)
    phy2log, _, _ = eplb.rebalance_experts(w, 64, 8, 2, 8)  # 8 groups of 8 over 2 nodes of 4 GPUs
    node_of_phys = torch.arange(64) // 32
    group_of_log = phy2log[0] // 8
    for grp in range(8):
        nodes = node_of_phys[group_of_log == grp].unique()
        assert nodes.numel() == 1


def test_rebalance_with_replicas_and_global_policy():
    g = torch.Generator().manual_seed(3)
    w = torch.rand(1, 24, generator=g) + 0.1
    phy2log, log2phy, logcnt = eplb.rebalance_experts(w, 32, 3, 2, 8)  # 3 groups / 2 nodes -> global policy
    assert int(logcnt.sum()) == 32
    assert log2phy.shape[2] == int(logcnt.max())
    for e in range(24):
        slots = log2phy[0, e][log2phy[0, e] >= 0]
        assert slots.numel() == int(logcnt[0, e])
        assert bool((phy2log[0][slots] == e).all())
