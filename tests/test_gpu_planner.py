"""Single-GPU tests of the native planner kernels against plain PyTorch references.

Covers the reference's three test files (tests/test_solve.py, tests/test_idx_processing.py)
through the same public API, plus small bounds cases, the fused single-launch path and
the status block."""

import pytest
import torch

from lplb_b200 import Planner, lp, topology
from lplb_b200.ops import reference as ref
from tests.helpers import SOLVE_CONFIGS, balance_after, synthetic_loads

pytestmark = pytest.mark.gpu


def _planner(r2o, n_logical, ep_size, n_red, **kw):
    # most tests below compare launches bit for bit, so they solve every batch from scratch;
    # the warm-start default of the library has tests of its own
    kw.setdefault("warm_start", False)
    return Planner(r2o, n_logical + n_red * ep_size, n_logical, ep_size, device="cuda", **kw)


def _sms():
    return torch.cuda.get_device_properties(0).multi_processor_count


# ---------------------------------------------------------------- histogram
@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
def test_count_workload_matches_scatter_add(dtype):
    planner = _planner(topology.cube(), 256, 32, 2)
    torch.manual_seed(42)
    idx = torch.randint(-1, 256, (4096, 8), device="cuda").to(dtype)
    counts, by_sm = planner.count_workload(idx, _sms())
    assert counts.shape == (256,) and int(counts.min()) >= 0
    assert int(counts.sum()) == int((idx != -1).sum())
    want = torch.zeros(257, dtype=torch.long, device="cuda")
    want.scatter_add_(0, idx.view(-1).long() + 1, torch.ones(idx.numel(), dtype=torch.long, device="cuda"))
    assert torch.equal(counts.long(), want[1:])
    ref_counts, ref_prefix = ref.count_reference(idx.cpu(), 256, _sms())
    assert torch.equal(by_sm.cpu(), ref_prefix)


@pytest.mark.parametrize("n_tokens,n_sms", [(0, 3), (1, 1), (255, 2), (257, 3), (5000, 7), (70000, 148), (300, 200)])
def test_count_small_and_ragged_cases(n_tokens, n_sms):
    planner = _planner(topology.cube(), 16, 8, 2)
    idx = torch.randint(-1, 16, (n_tokens,), device="cuda", generator=torch.Generator("cuda").manual_seed(n_tokens))
    counts, by_sm = planner.count_workload(idx, n_sms)
    ref_counts, ref_prefix = ref.count_reference(idx.cpu(), 16, n_sms)
    assert torch.equal(counts.cpu(), ref_counts) and torch.equal(by_sm.cpu(), ref_prefix)
    # the kernel leaves its ticket at zero, so a second call gives the same answer
    counts2, _ = planner.count_workload(idx, n_sms)
    assert torch.equal(counts2, counts)


def test_out_of_range_indices_are_counted_not_trapped():
    planner = _planner(topology.cube(), 16, 8, 2)
    idx = torch.tensor([0, 1, 16, 99, -1, -7, 3], device="cuda")
    counts, _ = planner.count_workload(idx, 2)
    assert counts.tolist() == [1, 1, 0, 1] + [0] * 12
    st = planner.check_status(clear=True)
    assert st["error"] == "bad_index" and st["bad_indices"] == 3
    assert planner.check_status().ok


# ---------------------------------------------------------------- LP
@pytest.mark.parametrize("name,r2o,n_logical,ep_size,n_red,reorder,bound", SOLVE_CONFIGS)
def test_planner_solve_quality(name, r2o, n_logical, ep_size, n_red, reorder, bound):
    planner = _planner(r2o, n_logical, ep_size, n_red)
    history, current = synthetic_loads(n_logical, seed=41, device="cuda")
    phy2log, _, _ = planner.update_redundancy_mapping(history if reorder else None)
    avail = torch.zeros((), dtype=torch.int32, device="cuda")
    probs, normalised = planner.solve_probs(current, avail)
    assert int(avail) == planner.n_group
    assert probs.shape == (planner.n_group, planner.group_size, planner.num_redundants)
    assert probs.dtype == torch.float32 and float(probs.min()) >= 0 and float(probs.max()) <= 1
    assert torch.allclose(normalised.reshape(-1).cpu(), current.cpu().float() / float(current.max()))
    assert balance_after(planner, phy2log, current, probs) < bound
    # against the float64 oracle, group by group
    w, fixed = lp.bundle_loads(
        current.cpu().double(), phy2log.cpu(), planner.n_group, planner.group_size, planner.num_redundants,
        planner.n_local_logical_routed_experts, planner.combined_redundant_experts,
    )
    realised = lp.rank_loads(probs.cpu().double(), w, fixed, r2o).max(-1).values
    oracle = lp.solve_ipm(w, fixed, r2o, tol=1e-4)
    assert float((probs.cpu().double() - oracle.f).abs().max()) < 1e-4
    for grp in range(planner.n_group):
        _, t_opt = lp.solve_highs(w[grp], fixed[grp], r2o)
        assert (float(realised[grp]) - t_opt) / t_opt < 1e-3
    st = planner.check_status()
    assert st.ok and 1 <= st["lp_iters"] <= 12


def test_solver_sweep_against_oracle():
    # 512 Cube instances of the skewed shape: 128 experts, 16 per rank, Dirichlet(0.3)
    import numpy as np

    rng = np.random.default_rng(0)
    n_group = 64
    planner = _planner(topology.cube(), 128 * n_group, 8 * n_group, 2)
    worst = 0.0
    for _ in range(8):
        cnt = np.stack([
            -np.sort(-rng.multinomial(32768 * 8, rng.dirichlet(np.full(128, 0.3))).reshape(8, 16), axis=1)
            for _ in range(n_group)
        ])
        current = torch.from_numpy(cnt.reshape(-1)).int().cuda()
        avail = torch.zeros(1, dtype=torch.int64, device="cuda")
        probs, _ = planner.solve_probs(current, avail)
        assert int(avail) == n_group
        w = torch.from_numpy(cnt[:, :, :2].astype(np.float64))
        fixed = torch.from_numpy(cnt[:, :, 2:].sum(-1).astype(np.float64))
        realised = lp.rank_loads(probs.cpu().double(), w, fixed, topology.cube()).max(-1).values
        oracle = lp.solve_ipm(w, fixed, topology.cube(), tol=1e-7, max_iters=40)
        assert bool(oracle.converged.all())
        gap = (realised - oracle.t) / oracle.t
        worst = max(worst, float(gap.max()))
        assert float(gap.min()) > -1e-6
        for i in range(0, n_group, 16):  # spot-check the oracle itself against HiGHS
            _, t_opt = lp.solve_highs(w[i], fixed[i], topology.cube())
            assert abs(float(oracle.t[i]) - t_opt) / t_opt < 1e-6
    assert worst < 1e-3


def test_degenerate_loads_on_device():
    planner = _planner(topology.cube(), 64 * 4, 32, 2)
    current = torch.zeros(4, 8, 8, dtype=torch.int32)
    current[1, 0, 0] = 1000
    current[2, 3, 5] = 500
    current[3] = 9
    avail = torch.zeros((), dtype=torch.int32, device="cuda")
    probs, normalised = planner.solve_probs(current.cuda().reshape(-1), avail)
    assert int(avail) == 4 and not bool(torch.isnan(probs).any())
    assert torch.equal(probs[0].cpu(), torch.ones(8, 2))
    assert abs(float(probs[1, 0, 0]) - 0.5) < 1e-3
    # all-zero input: nothing to normalise, nothing to balance, still no NaN
    avail.zero_()
    probs, normalised = planner.solve_probs(torch.zeros(256, dtype=torch.int32, device="cuda"), avail)
    assert int(avail) == 4 and float(normalised.abs().max()) == 0 and float(probs.min()) == 1


def test_iteration_cap_reports_failure():
    planner = _planner(topology.cube(), 64, 8, 2, max_iters=1, tol=1e-9)
    _, current = synthetic_loads(64, seed=1, device="cuda")
    avail = torch.zeros((), dtype=torch.int32, device="cuda")
    probs, _ = planner.solve_probs(current, avail)
    assert int(avail) == 0
    st = planner.check_status(clear=True)
    assert st["error"] == "lp_not_converged" and st["lp_failures"] == 1
    assert float(probs.min()) >= 0 and float(probs.max()) <= 1


# ---------------------------------------------------------------- redirect
def _check_redirect(planner, idx, out, probs):
    m = planner.mapping
    e, p = planner.n_logical_routed_experts, planner.n_routed_experts
    idx_c, out_c = idx.reshape(-1).cpu().long(), out.reshape(-1).cpu().long()
    assert out.shape == idx.shape and out.dtype == idx.dtype
    assert int(out_c.min()) >= -1 and int(out_c.max()) < p
    assert torch.equal(out_c == -1, idx_c == -1)
    padded = torch.cat([torch.full((1, 2), -1, dtype=torch.int32), m.log2phy.cpu()]).long()
    orig, repl = padded[idx_c + 1, 0], padded[idx_c + 1, 1]
    assert bool(((out_c == orig) | (out_c == repl)).all())
    valid = idx_c >= 0
    total = torch.bincount(idx_c[valid], minlength=e)
    kept = torch.bincount(idx_c[valid & (out_c == orig)], minlength=e)
    quota = ref.quotas_reference(total, probs.cpu(), m.log2edge.cpu())
    assert torch.equal(kept, quota)


def test_weighted_select_target_exact_quotas():
    planner = _planner(topology.cube(), 256, 32, 2)
    torch.manual_seed(42)
    history = (torch.randn(256, device="cuda") * 0.15 + 1).clamp_min(0).mul(2**20).long()
    planner.update_redundancy_mapping(history)
    idx = torch.randint(-1, 256, (65536,), device="cuda")
    o_weight = (torch.randn(4, 8, 2, device="cuda") / 3 + 0.5).clamp(0, 1)
    _, by_sm = planner.count_workload(idx, _sms())
    out = planner.weighted_select_target(idx, o_weight, by_sm, _sms())
    _check_redirect(planner, idx, out, o_weight)
    # realised share vs requested share, the reference's 5e-2 criterion
    # (reference tests/test_idx_processing.py:132-138)
    m = planner.mapping
    rep = m.log2edge.cpu().long() >= 0
    idx_c, out_c = idx.cpu(), out.cpu()
    total = torch.bincount(idx_c[idx_c >= 0], minlength=256)[rep].double()
    kept = torch.bincount(idx_c[(idx_c >= 0) & (out_c == m.log2phy.cpu().long()[idx_c.clamp_min(0), 0])], minlength=256)[rep].double()
    want = o_weight.reshape(-1).cpu().double()[m.log2edge.cpu().long()[rep]]
    assert float((kept / total - want).abs().max()) < 5e-2


@pytest.mark.parametrize("n_tokens,n_sms,quota", [(1, 1, 0.5), (499 * 4, 3, 0.37), (1000, 5, 0.0), (1000, 5, 1.0), (70000, 148, 0.123)])
def test_redirect_degenerate_quotas(n_tokens, n_sms, quota):
    # includes totals that are multiples of 499, where the reference's hash degenerates
    planner = _planner(topology.cube(), 16, 8, 2)
    idx = torch.randint(0, 2, (n_tokens,), device="cuda") * 0  # every token picks expert 0
    probs = torch.full((1, 8, 2), quota, device="cuda")
    _, by_sm = planner.count_workload(idx, n_sms)
    out = planner.weighted_select_target(idx, probs, by_sm, n_sms)
    _check_redirect(planner, idx, out, probs)


# ---------------------------------------------------------------- fused run
@pytest.mark.parametrize("name,r2o,n_logical,ep_size,n_red", [
    ("cube", topology.cube(), 256, 8, 2),
    ("cube-ep32", topology.cube(), 256, 32, 2),
    ("ring", topology.ring(8), 64, 8, 1),
    ("hypercube", topology.hypercube(), 256, 16, 2),
    ("torus2x4", topology.torus(2, 4), 512, 8, 2),
    ("torus8x4-c2", topology.torus(8, 4), 256, 32, 4),
])
def test_fused_run_matches_staged_pipeline(name, r2o, n_logical, ep_size, n_red):
    planner = _planner(r2o, n_logical, ep_size, n_red)
    gen = torch.Generator("cuda").manual_seed(5)
    for step, n_sms in enumerate([_sms(), 13, 1, _sms()]):
        bias = torch.randn(n_logical, device="cuda", generator=gen)
        logits = torch.randn(2048, n_logical, device="cuda", generator=gen) + bias
        idx = logits.topk(8, dim=-1).indices
        if step == 1:
            planner.update_redundancy_mapping(torch.bincount(idx.reshape(-1), minlength=n_logical))
            idx[::7, 3] = -1
        avail = torch.zeros((), dtype=torch.int32, device="cuda")
        out = planner.run(idx, avail, n_sms)
        assert int(avail) == planner.n_group
        probs = planner.last_probs.clone()
        _check_redirect(planner, idx, out, probs)
        avail2 = torch.zeros((), dtype=torch.int32, device="cuda")
        counts, _ = planner.count_workload(idx, n_sms)
        staged_probs, _ = planner.solve_probs(counts, avail2)
        assert torch.equal(staged_probs, probs)  # same arithmetic on the same counts
        assert planner.check_status().ok
    assert planner.check_status()["calls"] == 4


def test_fused_run_balances_real_routing():
    planner = _planner(topology.cube(), 256, 8, 2)
    gen = torch.Generator("cuda").manual_seed(0)
    bias = torch.randn(256, device="cuda", generator=gen)
    logits = (torch.randn(4096, 256, device="cuda", generator=gen) + bias).bfloat16()
    idx = logits.topk(8, dim=-1).indices
    # placement from an older batch with the same bias, so that it is good but not perfect
    old = (torch.randn(4096, 256, device="cuda", generator=gen) + bias).bfloat16().topk(8, dim=-1).indices
    planner.update_redundancy_mapping(torch.bincount(old.reshape(-1), minlength=256))
    avail = torch.zeros(1, dtype=torch.int64, device="cuda")
    out = planner.run(idx, avail)
    assert int(avail) == 1
    pl = planner.n_local_routed_experts
    before = torch.bincount(planner.mapping.log2phy[idx.reshape(-1), 0].long() // pl, minlength=8).double()
    after = torch.bincount(out.reshape(-1) // pl, minlength=8).double()
    assert float(after.max()) <= float(before.max()) + 2
    # the realised max load is the LP optimum up to rounding of quotas
    counts = torch.bincount(idx.reshape(-1), minlength=256)
    w, fixed = lp.bundle_loads(counts.cpu().double(), planner.phy2log.cpu(), 1, 8, 2, 32, 1)
    _, t_opt = lp.solve_highs(w[0], fixed[0], topology.cube())
    assert float(after.max()) <= t_opt * (1 + 1e-3) + 16


def test_run_replays_from_a_cuda_graph():
    """One capture, many replays: the launch number lives on the device, so a replayed launch
    is indistinguishable from an eager one.  Each replay must redirect the batch that is in
    the static input buffer at that time, with the quotas of that batch's own LP."""
    planner = _planner(topology.cube(), 256, 8, 2)
    gen = torch.Generator("cuda").manual_seed(3)
    bias = torch.randn(256, device="cuda", generator=gen)
    batches = [
        (torch.randn(2048, 256, device="cuda", generator=gen) + bias).bfloat16().topk(8, dim=-1).indices
        for _ in range(4)
    ]
    planner.update_redundancy_mapping(torch.bincount(batches[0].reshape(-1), minlength=256))
    idx_static = batches[0].clone()
    out_static = torch.empty_like(idx_static)
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # first launch outside the capture (attribute and occupancy queries)
        planner.run(idx_static, avail, out=out_static)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        planner.run(idx_static, avail, out=out_static)
    calls_before = planner.check_status()["calls"]
    avail.zero_()
    for batch in batches:
        idx_static.copy_(batch)
        graph.replay()
        torch.cuda.synchronize()
        _check_redirect(planner, batch, out_static, planner.last_probs.clone())
    status = planner.check_status()
    assert status.ok and status["calls"] == calls_before + len(batches)
    assert int(avail) == len(batches)
    # and an eager launch after the replays continues the same launch numbering
    out = planner.run(batches[1], avail)
    _check_redirect(planner, batches[1], out, planner.last_probs.clone())
    assert planner.check_status()["calls"] == calls_before + len(batches) + 1
    # a new placement is copied into the tables the captured launch already points at
    old_phy2log = planner.phy2log.clone()
    skewed = torch.bincount(batches[2].reshape(-1), minlength=256) * torch.arange(1, 257, device="cuda")
    planner.update_redundancy_mapping(skewed)
    assert not torch.equal(old_phy2log, planner.phy2log)
    idx_static.copy_(batches[3])
    graph.replay()
    torch.cuda.synchronize()
    _check_redirect(planner, batches[3], out_static, planner.last_probs.clone())
    assert planner.check_status().ok


def test_run_reads_and_writes_pinned_host_memory():
    planner = _planner(topology.cube(), 256, 8, 2)
    gen = torch.Generator("cuda").manual_seed(3)
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    for n_tokens, n_sms in ((4096, _sms()), (300, 5), (40000, 16)):  # the last one exceeds the register-kept part
        idx = (torch.randn(n_tokens, 256, device="cuda", generator=gen)).topk(8, dim=-1).indices
        idx[::11, 2] = -1
        host_idx = idx.cpu().pin_memory()
        host_out = torch.empty_like(host_idx).pin_memory()
        got = planner.run(host_idx, avail, n_sms, out=host_out)
        torch.cuda.synchronize()
        assert got.data_ptr() == host_out.data_ptr() and not got.is_cuda
        _check_redirect(planner, idx, host_out.cuda(), planner.last_probs)
        # same shares and quotas as the all-device call
        dev_out = planner.run(idx, avail, n_sms)
        assert torch.equal(torch.bincount(dev_out.reshape(-1) + 1, minlength=273).cpu(),
                           torch.bincount(host_out.reshape(-1) + 1, minlength=273))
        # device result written into a caller-provided device buffer
        buf = torch.empty_like(idx)
        assert planner.run(idx, avail, n_sms, out=buf).data_ptr() == buf.data_ptr()
    cached = planner.run(host_idx, avail)
    torch.cuda.synchronize()
    assert cached.is_pinned() and cached.shape == host_idx.shape
    assert planner.check_status().ok


def test_warm_start_cuts_iterations_and_keeps_the_optimum():
    planner = _planner(topology.cube(), 256, 8, 2, warm_start=True)
    cold = _planner(topology.cube(), 256, 8, 2)
    gen = torch.Generator("cuda").manual_seed(9)
    bias = torch.randn(256, device="cuda", generator=gen)

    def batch():
        return (torch.randn(8192, 256, device="cuda", generator=gen) + bias).bfloat16().topk(8, dim=-1).indices

    hist = torch.bincount(batch().reshape(-1), minlength=256)
    planner.update_redundancy_mapping(hist)
    cold.update_redundancy_mapping(hist)
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    iters = []
    for step in range(8):
        if step == 5:
            bias = torch.randn(256, device="cuda", generator=gen)  # the routing distribution moves
        idx = batch()
        out = planner.run(idx, avail)
        _check_redirect(planner, idx, out, planner.last_probs)
        st = planner.check_status(clear=True)
        assert st.ok
        cold.run(idx, avail)
        iters.append((st["lp_iters"], cold.check_status(clear=True)["lp_iters"]))
        counts = torch.bincount(idx.reshape(-1), minlength=256)
        w, fixed = lp.bundle_loads(counts.cpu().double(), planner.phy2log.cpu(), 1, 8, 2, 32, 1)
        realised = float(lp.rank_loads(planner.last_probs.cpu().double(), w, fixed, topology.cube()).max())
        _, t_opt = lp.solve_highs(w[0], fixed[0], topology.cube())
        assert (realised - t_opt) / t_opt < 1e-3
        # the staged kernels share the state: same anchor, same answer
        local, _ = planner.count_workload(idx, _sms())
        staged_probs, _ = planner.solve_probs(local, avail)
        assert torch.allclose(staged_probs, planner.last_probs, atol=1e-6)
    assert iters[0][0] == iters[0][1]  # first solve is cold
    assert all(w <= c for w, c in iters)
    assert iters[2][0] < iters[2][1] and iters[3][0] < iters[3][1]  # steady state: fewer iterations
    assert iters[5][0] == iters[5][1]  # the guard sent the shifted batch down the cold path
    planner.invalidate_warm_start()
    planner.run(batch(), avail)
    assert planner.check_status()["lp_iters"] >= iters[0][0] - 1


# ---------------------------------------------------------------- exchange on one GPU
def test_exchange_loopback_sums_prefilled_peer():
    planner = _planner(topology.cube(), 64, 8, 2)
    eng = planner._engine
    eng.open_exchange_loopback(2, 0)
    peer = torch.arange(64, dtype=torch.int32) * 3
    mine = torch.randint(0, 100, (64,), dtype=torch.int32, device="cuda")
    for _ in range(3):  # both parities
        eng.debug_fill_slot(1, peer, eng.completed_launches() + 1)  # "rank 1 has published for the next launch"
        got = eng.all_reduce_counts(mine)
        assert torch.equal(got.cpu(), mine.cpu() + peer)
    idx = torch.randint(0, 64, (4096, 4), device="cuda")
    avail = torch.zeros((), dtype=torch.int32, device="cuda")
    eng.debug_fill_slot(1, peer, eng.completed_launches() + 1)
    out = eng.run_fused(idx, avail, 16, True)
    counts = torch.bincount(idx.reshape(-1), minlength=64).int()
    ws = eng.workspace()
    glob = ws[8 + 2 * 64 : 8 + 3 * 64]
    assert torch.equal(glob.cpu(), counts.cpu() + peer)
    assert planner.check_status().ok
    _check_redirect(planner, idx, out, eng.last_probs())


def test_groups_beyond_a_warp_run_the_fused_single_launch_without_a_host_sync():
    # torus(8, 8): one LP group of 64 ranks, solved by the thread-block solver inside the fused
    # kernel; the whole step is one launch and the host never waits for the device
    planner = _planner(topology.torus(8, 8), 512, 64, 2)
    assert planner._native_solver is True and planner._engine.solver() == "block"
    gen = torch.Generator("cuda").manual_seed(2)
    idx = (torch.randn(4096, 512, device="cuda", generator=gen) + torch.randn(512, device="cuda", generator=gen)).topk(8, dim=-1).indices
    planner.update_redundancy_mapping(torch.bincount(idx.reshape(-1), minlength=512))
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    planner.run(idx, avail)  # first call: attribute and occupancy queries
    calls = planner.check_status()["calls"]
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")  # any host synchronisation raises from here on
    try:
        out = planner.run(idx, avail)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    probs = planner.last_probs.clone()
    assert int(avail) == 2 and probs.shape == (1, 64, 2)
    assert planner.check_status()["calls"] == calls + 1
    _check_redirect(planner, idx, out, probs)
    counts, _ = planner.count_workload(idx, _sms())
    w, fixed = lp.bundle_loads(counts.cpu().double(), planner.phy2log.cpu(), 1, 64, 2, 8, 1)
    realised = float(lp.rank_loads(probs.cpu().double(), w, fixed, topology.torus(8, 8)).max())
    _, t_opt = lp.solve_highs(w[0], fixed[0], topology.torus(8, 8))
    assert (realised - t_opt) / t_opt < 1e-3
    st = planner.check_status()
    assert st.ok and 0 <= st["lp_gap"] <= 1e-4 and st["lp_iters"] <= 12


@pytest.mark.parametrize("name,r2o,ll", [
    ("cube", topology.cube(), 8),
    ("ring5", topology.ring(5), 4),
    ("hypercube", topology.hypercube(), 8),
    ("torus8x4", topology.torus(8, 4), 8),
    ("ring100", topology.ring(100), 2),
    ("circulant12x3", topology.circulant(12, (1, 2, 5)), 6),
    ("circulant10x5", topology.circulant(10, (1, 2, 3, 4, 5)), 8),
    ("circulant128x4", topology.circulant(128, (1, 2, 64, 127)), 8),
])
def test_block_solver_reaches_the_optimum_for_any_group_shape(name, r2o, ll):
    """The thread-block solver on group sizes that are not multiples of 8 or 32, on every
    instantiated replica count and on the padded one (5 replicas run as 8), warm and cold."""
    g, d = r2o.shape
    planner = _planner(r2o, g * ll, g, d, solver="block", warm_start=True)
    assert planner._engine.solver() == "block"
    gen = torch.Generator().manual_seed(11)
    base = (torch.rand(g * ll, generator=gen) + 0.5) * 4000
    iters = []
    for step in range(3):
        counts = (base * (1 + 0.03 * torch.randn(g * ll, generator=gen))).clamp_min(0).int().cuda()
        avail = torch.zeros(1, dtype=torch.int32, device="cuda")
        probs, _ = planner.solve_probs(counts, avail)
        assert int(avail) == 1 and float(probs.min()) >= 0 and float(probs.max()) <= 1
        w, fixed = lp.bundle_loads(counts.cpu().double(), planner.phy2log.cpu(), 1, g, d, ll, 1)
        realised = float(lp.rank_loads(probs.cpu().double(), w, fixed, r2o).max())
        _, t_opt = lp.solve_highs(w[0], fixed[0], r2o)
        assert -1e-6 < (realised - t_opt) / t_opt < 1e-3, (name, step, realised, t_opt)
        st = planner.check_status(clear=True)
        assert st.ok and st["lp_gap"] <= 1e-4
        iters.append(st["lp_iters"])
    assert iters[1] <= iters[0] and iters[2] <= iters[0]  # later batches start from the saved iterate


def test_block_and_warp_solver_agree():
    gen = torch.Generator().manual_seed(4)
    for r2o, ll, n_group in ((topology.cube(), 8, 3), (topology.hypercube(), 4, 2), (topology.torus(8, 4), 4, 1)):
        g, d = r2o.shape
        e = g * ll * n_group
        warp = _planner(r2o, e, g * n_group, d, solver="warp")
        block = _planner(r2o, e, g * n_group, d, solver="block")
        assert (warp._engine.solver(), block._engine.solver()) == ("warp", "block")
        counts = (torch.rand(e, generator=gen) * 5000).int().cuda()
        a1 = torch.zeros(1, dtype=torch.int32, device="cuda")
        a2 = torch.zeros(1, dtype=torch.int32, device="cuda")
        p1, n1 = warp.solve_probs(counts, a1)
        p2, n2 = block.solve_probs(counts, a2)
        assert int(a1) == int(a2) == n_group and torch.equal(n1, n2)
        assert float((p1 - p2).abs().max()) < 2e-4  # same method, different elimination order
        assert warp.check_status()["lp_iters"] == block.check_status()["lp_iters"]
        # and inside the fused kernel (`run` would give several block-solver groups a launch of
        # their own, so the engine is called directly)
        idx = torch.randint(-1, e, (3000, 4), device="cuda")
        warp.run(idx, a1)
        o2 = block._engine.run_fused(idx, a2, _sms(), False, None)
        _check_redirect(block, idx, o2, block._engine.last_probs().clone())
        assert float((warp.last_probs - block._engine.last_probs()).abs().max()) < 2e-4
        o3 = block.run(idx, a2)
        _check_redirect(block, idx, o3, block.last_probs.clone())
        assert float((warp.last_probs - block.last_probs).abs().max()) < 2e-4


def test_several_wide_groups_are_solved_side_by_side():
    # hypercube with ep_size 64: four LP groups of 16 ranks.  `run` leaves the single launch so
    # that every group gets a CTA of its own; result and status are as for any other call.
    planner = _planner(topology.hypercube(), 256, 64, 2)
    assert planner._engine.solver() == "block" and planner.n_group == 4
    gen = torch.Generator("cuda").manual_seed(8)
    idx = (torch.randn(4096, 256, device="cuda", generator=gen) + torch.randn(256, device="cuda", generator=gen)).topk(8, dim=-1).indices
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = planner.run(idx, avail)
    assert int(avail) == 4
    counts, _ = planner.count_workload(idx, _sms())
    probs, _ = planner.solve_probs(counts, torch.zeros(1, dtype=torch.int32, device="cuda"))
    _check_redirect(planner, idx, out, probs)
    assert planner.check_status().ok


def test_odd_number_of_experts_keeps_the_tables_aligned():
    # 9 ranks x 3 logical experts = 27: the int2 table of the redirect phase must not depend on
    # the parity of the expert count
    r2o = topology.torus(3, 3)
    planner = _planner(r2o, 27, 9, 2)
    idx = torch.randint(-1, 27, (5000, 2), device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = planner.run(idx, avail, 7)
    assert int(avail) == 1
    _check_redirect(planner, idx, out, planner.last_probs.clone())
    counts, by_sm = planner.count_workload(idx, 5)
    probs, _ = planner.solve_probs(counts, avail)
    staged = planner.weighted_select_target(idx, probs, by_sm, 5)
    _check_redirect(planner, idx, staged, probs)
    # the exchange pushes single words instead of pairs when the count is odd
    eng = planner._engine
    eng.open_exchange_loopback(2, 0)
    peer = torch.arange(27, dtype=torch.int32) * 7
    eng.debug_fill_slot(1, peer, eng.completed_launches() + 1)
    mine = torch.randint(0, 100, (27,), dtype=torch.int32, device="cuda")
    assert torch.equal(eng.all_reduce_counts(mine).cpu(), mine.cpu() + peer)
    assert planner.check_status().ok


def test_library_default_is_warm_started_and_status_can_be_polled():
    planner = Planner(topology.cube(), 272, 256, 8, device="cuda")
    assert planner.warm_start is True
    gen = torch.Generator("cuda").manual_seed(21)
    bias = torch.randn(256, device="cuda", generator=gen)
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    iters, seen = [], None
    for step in range(4):
        idx = (torch.randn(8192, 256, device="cuda", generator=gen) + bias).bfloat16().topk(8, dim=-1).indices
        out = planner.run(idx, avail)
        _check_redirect(planner, idx, out, planner.last_probs.clone())
        polled = planner.poll_status()  # never blocks; lags by a call or two
        seen = polled or seen
        iters.append(planner.check_status()["lp_iters"])
    assert min(iters[1:]) < iters[0], iters
    torch.cuda.synchronize()
    last = planner.poll_status()
    assert last is not None and last.ok and last["calls"] >= 3
    assert planner.check_status()["calls"] == 4


def test_two_level_exchange_on_one_gpu():
    # 4 ranks in 2 nodes of 2, this GPU plays rank 0: level 0 needs rank 1 (same node), level 1
    # needs the node sum published by rank 2 (same position in the other node)
    planner = _planner(topology.cube(), 64, 8, 2)
    eng = planner._engine
    eng.open_exchange_loopback(4, 0)
    eng.set_exchange_nodes(2)
    neighbour = torch.arange(64, dtype=torch.int32) + 1
    other_node = torch.arange(64, dtype=torch.int32) * 5 + 2
    mine = torch.randint(0, 100, (64,), dtype=torch.int32, device="cuda")
    for _ in range(3):
        epoch = eng.completed_launches() + 1
        eng.debug_fill_slot(1, neighbour, epoch, 0)
        eng.debug_fill_slot(2, other_node, epoch, 1)
        got = eng.all_reduce_counts(mine)
        assert torch.equal(got.cpu(), mine.cpu() + neighbour + other_node)
    # the other node never answers: reported, its share replaced by this node's sum
    planner2 = _planner(topology.cube(), 64, 8, 2, peer_timeout_us=300.0)
    eng2 = planner2._engine
    eng2.open_exchange_loopback(4, 0)
    eng2.set_exchange_nodes(2)
    eng2.debug_fill_slot(1, neighbour, 1, 0)
    got = eng2.all_reduce_counts(mine)
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), 2 * (mine.cpu() + neighbour))
    st = planner2.check_status(clear=True)
    assert st["error"] == "peer_timeout" and st["detail"] == 0b100
    # the other node answers, but marks its sum as degraded (bit 31 of the first word: one of
    # its ranks was late and replaced): the sum is used as it is and the report is passed on
    marked = other_node.clone()
    marked[0] |= -(1 << 31)
    epoch = eng2.completed_launches() + 1
    eng2.debug_fill_slot(1, neighbour, epoch, 0)
    eng2.debug_fill_slot(2, marked, epoch, 1)
    got = eng2.all_reduce_counts(mine)
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), mine.cpu() + neighbour + other_node)
    st = planner2.check_status(clear=True)
    assert st["error"] == "peer_timeout" and st["detail"] == 0b100 and st["timeouts"] == 1


def test_exchange_wait_runs_out_and_falls_back():
    # a flag that nothing sets: the wait must end by itself, report, and still route
    planner = _planner(topology.cube(), 64, 8, 2, peer_timeout_us=300.0)
    eng = planner._engine
    eng.open_exchange_loopback(2, 0)
    idx = torch.randint(0, 64, (4096, 4), device="cuda")
    avail = torch.zeros((), dtype=torch.int32, device="cuda")
    out = eng.run_fused(idx, avail, 8, True)
    torch.cuda.synchronize()
    st = planner.check_status(clear=True)
    assert st["error"] == "peer_timeout" and st["phase"] == "exchange" and st["detail"] == 0b10 and st["timeouts"] == 1
    assert int(avail) == 1
    _check_redirect(planner, idx, out, eng.last_probs())
    # fallback used this rank's counts for the absent peer: shares equal the local solve
    local = Planner(topology.cube(), 80, 64, 8, device="cuda")
    a2 = torch.zeros((), dtype=torch.int32, device="cuda")
    local.run(idx, a2, 8)
    assert torch.allclose(local.last_probs, eng.last_probs(), atol=1e-6)
    # the context is still healthy
    assert int(torch.ones(4, device="cuda").sum()) == 4


# ---------------------------------------------------------------- timing helpers
def test_timing_helpers_report_the_solve_kernel():
    from lplb_b200.utils.timing import bench_kineto, time_cuda

    planner = _planner(topology.cube(), 64, 8, 2)
    _, current = synthetic_loads(64, seed=1, device="cuda")
    avail = torch.zeros((), dtype=torch.int32, device="cuda")
    seconds = bench_kineto(lambda: planner.solve_probs(current, avail), "solve_kernel", 20)
    assert 1e-6 < seconds < 1e-3
    stats = time_cuda(lambda: planner.solve_probs(current, avail), iters=20, warmup=3)
    assert stats["min"] <= stats["p50"] <= stats["max"] and stats["p50"] < 1e3
