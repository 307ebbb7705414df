import pytest
import torch

from lplb_b200 import Planner, topology
from lplb_b200.mapping import build_mapping


@pytest.mark.parametrize("with_history", [False, True])
@pytest.mark.parametrize(
    "r2o,n_group,ll,c",
    [(topology.cube(), 4, 8, 1), (topology.cube(), 4, 8, 2), (topology.ring(8), 4, 8, 1), (topology.torus(8, 4), 1, 8, 1)],
)
def test_mapping_invariants(r2o, n_group, ll, c, with_history):
    g, d = r2o.shape
    e = n_group * g * ll
    hist = None
    if with_history:
        hist = (torch.randn(e, generator=torch.Generator().manual_seed(5)) * 0.15 + 1).clamp_min(0).mul(2**20).long()
    m = build_mapping(r2o, n_group, ll, c, hist)
    pl = ll + c * d
    p2l = m.phy2log.reshape(n_group * g, pl).long()
    # the logical block is a permutation of all experts
    assert sorted(p2l[:, :ll].reshape(-1).tolist()) == list(range(e))
    # every replica slot mirrors the source rank's slot given by r2o
    for rank in range(n_group * g):
        grp, i = divmod(rank, g)
        for j in range(c):
            for dd in range(d):
                src_rank = grp * g + int(r2o[i, dd])
                assert p2l[rank, ll + j * d + dd] == p2l[src_rank, j * d + dd]
    assert int(m.logcnt.max()) == 2 and int(m.logcnt.min()) == 1
    assert int(m.logcnt.sum()) == n_group * g * pl
    # log2phy: original first, replica second, both hold the expert
    for ex in range(e):
        o, r = m.log2phy[ex].tolist()
        assert m.phy2log[o] == ex and o % pl < ll
        if r >= 0:
            assert m.phy2log[r] == ex and r % pl >= ll
            assert int(m.log2edge[ex]) == (o // pl) * d + (o % pl) % d
        else:
            assert int(m.log2edge[ex]) == -1
    if with_history:
        # heaviest first on every rank
        h = hist.double()[p2l[:, :ll]]
        assert bool((h[:, :-1] >= h[:, 1:]).all())


def test_planner_mapping_matches_reference_layout_without_history():
    p = Planner(topology.cube(), 256 + 2 * 32, 256, 32, device="cpu")
    phy2log, log2phy, logcnt = p.update_redundancy_mapping()
    assert phy2log.dtype == torch.int32 and phy2log.shape == (320,)
    per_rank = phy2log.reshape(32, 10)
    assert torch.equal(per_rank[:, :8].reshape(-1), torch.arange(256, dtype=torch.int32))
    # rank 0's replicas copy rank 3's slot 0 and rank 6's slot 1
    assert per_rank[0, 8] == per_rank[3, 0] and per_rank[0, 9] == per_rank[6, 1]
    assert log2phy.shape == (256, 2) and int(logcnt.max()) == 2


def test_state_dict_round_trip():
    p = Planner(topology.cube(), 80, 64, 8, device="cpu")
    hist = torch.arange(64).flip(0) * 100 + 7
    p.update_redundancy_mapping(hist)
    state = p.state_dict()
    q = Planner(topology.cube(), 80, 64, 8, device="cpu")
    q.load_state_dict(state)
    assert torch.equal(q.phy2log, p.phy2log) and torch.equal(q.mapping.log2edge, p.mapping.log2edge)
    with pytest.raises(ValueError):
        Planner(topology.ring(8), 72, 64, 8, device="cpu").load_state_dict(state)


def test_constructor_validation():
    with pytest.raises(ValueError):
        Planner(topology.cube(), 80, 64, None, device="cpu")
    with pytest.raises(ValueError):
        Planner(topology.cube(), 80, 64, 12, device="cpu")
    with pytest.raises(ValueError):
        Planner(topology.cube(), 72, 64, 8, device="cpu")  # 1 redundant per rank cannot fill 2 slots


def test_dump_lp_exposes_the_solver_inputs():
    from lplb_b200 import lp

    p = Planner(topology.cube(), 80, 64, 8, device="cpu")
    wl = torch.arange(64) * 3 + 5
    d = p.dump_lp(wl)
    assert d["M"].shape == (1, 8, 16) and d["A"][0].shape == (24, 42)
    assert torch.allclose(d["M"].sum(1), torch.zeros(1, 16, dtype=torch.float64))  # columns sum to zero
    _, t_opt = lp.solve_highs(d["bundle_loads"][0], d["fixed_loads"][0], topology.cube())
    assert abs(float(d["oracle_max_load"][0]) - t_opt) / t_opt < 1e-6


def test_default_cta_count_follows_the_batch_size():
    # one worker CTA per 384 indices beside the solver CTA, at least two CTAs, at most one per SM
    planner = Planner(topology.cube(), 256 + 16, 256, 8, device="cpu")
    sms = planner._default_sms()
    assert planner._default_ctas(0) == 2 and planner._default_ctas(1) == 2
    assert planner._default_ctas(384 * 3) == min(sms, 4)
    assert planner._default_ctas(384 * 3 + 1) == min(sms, 5)
    assert planner._default_ctas(10**9) == sms
