import torch

from lplb_b200 import Planner, topology
from lplb_b200.ops import reference as ref


def test_slice_bounds_cover_everything_once():
    for n, k in [(0, 4), (1, 4), (255, 3), (256, 3), (32768, 148), (65536, 100), (1000, 7)]:
        b = ref.slice_bounds(n, k)
        assert b[0] == 0 and b[-1] == n and all(x <= y for x, y in zip(b, b[1:]))
        assert all(x % 256 == 0 or x == n for x in b)


def test_count_reference_against_scatter_add():
    # reference tests/test_idx_processing.py:8-48 restated
    e = 256
    idx = torch.randint(-1, e, (4096, 8), generator=torch.Generator().manual_seed(42))
    counts, prefix = ref.count_reference(idx, e, 16)
    want = torch.zeros(e + 1, dtype=torch.long).scatter_add_(0, idx.view(-1) + 1, torch.ones(idx.numel(), dtype=torch.long))[1:]
    assert counts.shape == (e,) and int(counts.min()) >= 0
    assert int(counts.sum()) == int((idx != -1).sum())
    assert torch.equal(counts.long(), want)
    assert prefix.shape == (16, e) and torch.equal(prefix[-1], counts)
    assert bool((prefix[1:] >= prefix[:-1]).all())


def test_redirect_reference_exact_quotas():
    # reference tests/test_idx_processing.py:51-138 restated, with exact instead of 5e-2 quotas
    planner = Planner(topology.cube(), 256 + 2 * 32, 256, 32, device="cpu")
    g = torch.Generator().manual_seed(42)
    hist = (torch.randn(256, generator=g) * 0.15 + 1).clamp_min(0).mul(2**20).long()
    phy2log, log2phy, logcnt = planner.update_redundancy_mapping(hist)
    idx = torch.randint(-1, 256, (65536,), generator=g)
    o_weight = (torch.randn(4, 8, 2, generator=g) / 3 + 0.5).clamp(0, 1)
    out = planner.weighted_select_target(idx, o_weight, None, 16)
    assert out.shape == idx.shape and int(out.min()) >= -1 and int(out.max()) < 320
    assert torch.equal(out == -1, idx == -1)
    padded = torch.cat([torch.full((1, 2), -1, dtype=torch.int32), log2phy]).long()
    assert bool(((out == padded[idx + 1, 0]) | (out == padded[idx + 1, 1])).all())
    total = torch.bincount(idx[idx >= 0], minlength=256)
    kept = torch.bincount(idx[(idx >= 0) & (out == padded[idx + 1, 0])], minlength=256)
    quota = ref.quotas_reference(total, o_weight, planner.mapping.log2edge)
    assert torch.equal(kept, quota)
    edge = planner.mapping.log2edge.long()
    rep = edge >= 0
    err = (kept[rep].double() / total[rep].clamp_min(1) - o_weight.reshape(-1)[edge[rep]].double()).abs()
    assert float(err.max()) <= 0.5 / float(total[rep].min()) + 1e-6


def test_even_spread_is_even():
    # the picks for a quota are spread over the ordinals, not bunched at one end
    log2phy = torch.tensor([[0, 1]], dtype=torch.int32)
    log2edge = torch.tensor([0], dtype=torch.int32)
    idx = torch.zeros(1000, dtype=torch.int64)
    out = ref.redirect_reference(idx, torch.tensor([0.3]), log2phy, log2edge)
    kept = (out == 0).long()
    assert int(kept.sum()) == 300
    windows = kept.reshape(10, 100).sum(1)
    assert int(windows.min()) == 30 and int(windows.max()) == 30


def test_run_cpu_end_to_end_balances():
    planner = Planner(topology.cube(), 32 + 16, 32, 8, device="cpu")
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(4096, 32, generator=g) + torch.randn(32, generator=g) * 1.5
    idx = logits.topk(8, dim=-1).indices
    hist = torch.bincount(idx.reshape(-1), minlength=32)
    planner.update_redundancy_mapping(hist)
    avail = torch.zeros(1, dtype=torch.int64)
    out = planner.run(idx, avail, 8)
    assert int(avail) == 1
    before = torch.bincount(planner.mapping.log2phy[idx.reshape(-1), 0].long() // 6, minlength=8).double()
    after = torch.bincount(out.reshape(-1) // 6, minlength=8).double()
    assert float(after.max() / after.mean()) <= float(before.max() / before.mean()) + 1e-9
    assert float(after.max() / after.mean()) < 1.05
