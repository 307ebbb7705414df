"""Property tests (hypothesis) of the CPU path: packing, and Planner.run end to end on random
topologies, shapes and routing, against the invariants every redirect has to keep."""

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from lplb_b200 import Planner, lp, topology
from lplb_b200.eplb import balanced_packing


@settings(max_examples=40, deadline=None, derandomize=True)
@given(
    layers=st.integers(1, 3),
    packs=st.integers(1, 8),
    per_pack=st.integers(1, 6),
    seed=st.integers(0, 2**31 - 1),
)
def test_balanced_packing_fills_every_pack_equally(layers, packs, per_pack, seed):
    n = packs * per_pack
    gen = torch.Generator().manual_seed(seed)
    weight = torch.rand(layers, n, generator=gen) ** 3  # skewed
    pack, rank = balanced_packing(weight, packs)
    assert pack.shape == rank.shape == (layers, n)
    for layer in range(layers):
        slots = (pack[layer] * per_pack + rank[layer]).tolist()
        assert sorted(slots) == list(range(n))  # every (pack, position) used exactly once
        loads = torch.zeros(packs).scatter_add_(0, pack[layer].long(), weight[layer])
        # greedy longest-first with a cardinality cap: never worse than the mean plus one item
        assert float(loads.max()) <= float(weight[layer].sum()) / packs + float(weight[layer].max()) + 1e-6


_TOPOLOGIES = st.sampled_from(
    [
        ("ring4", lambda: topology.ring(4)),
        ("ring8", lambda: topology.ring(8)),
        ("cube", topology.cube),
        ("torus2x3", lambda: topology.torus(2, 3)),
        ("torus2x4", lambda: topology.torus(2, 4)),
        ("hypercube", topology.hypercube),
    ]
)


@settings(max_examples=60, deadline=None, derandomize=True)
@given(
    topo=_TOPOLOGIES,
    ll=st.integers(2, 6),
    combined=st.integers(1, 2),
    n_group=st.integers(1, 2),
    tokens=st.integers(1, 400),
    topk=st.integers(1, 4),
    skew=st.floats(0.0, 2.0),
    with_history=st.booleans(),
    seed=st.integers(0, 2**31 - 1),
)
def test_cpu_run_keeps_the_redirect_invariants(topo, ll, combined, n_group, tokens, topk, skew, with_history, seed):
    r2o = topo[1]()
    g, d = r2o.shape
    if ll < combined * d:
        ll = combined * d
    ep = n_group * g
    e, pl = ep * ll, ll + combined * d
    topk = min(topk, e)
    gen = torch.Generator().manual_seed(seed)
    planner = Planner(r2o, ep * pl, e, ep, device="cpu", n_nodes=1)
    logits = torch.randn(tokens, e, generator=gen) + skew * torch.randn(e, generator=gen)
    idx = logits.topk(topk, dim=-1).indices
    idx[torch.rand(tokens, topk, generator=gen) < 0.05] = -1  # some dropped pairs
    if with_history:
        planner.update_redundancy_mapping(torch.bincount(idx[idx >= 0], minlength=e) + 1)
    avail = torch.zeros(1, dtype=torch.int64)
    out = planner.run(idx, avail, n_sms=4)

    assert out.shape == idx.shape and out.dtype == idx.dtype
    assert torch.equal(out == -1, idx == -1)
    valid = idx >= 0
    # every pair lands on a physical expert that holds its logical expert
    assert torch.equal(planner.phy2log.long()[out[valid]], idx[valid])
    # ... and only on the original or its replica
    l2p = planner.mapping.log2phy.long()
    orig, repl = l2p[idx[valid], 0], l2p[idx[valid], 1]
    assert bool(((out[valid] == orig) | (out[valid] == repl)).all())
    assert 0 <= int(avail) <= n_group
    if int(avail) == n_group and int(valid.sum()) > 0:
        # every LP converged: the realised maximum rank load is the LP optimum up to the
        # rounding of one token per replicated expert
        counts = torch.bincount(idx[valid], minlength=e)
        w, fixed = lp.bundle_loads(counts.double(), planner.phy2log, n_group, g, d, ll, combined)
        after = torch.bincount(out[valid] // pl, minlength=ep).reshape(n_group, g)
        for grp in range(n_group):
            _, t_opt = lp.solve_highs(w[grp], fixed[grp], r2o)
            assert float(after[grp].max()) <= t_opt * (1 + 1e-3) + combined * d + 1
