"""Run by tests/test_gpu_bounds_build.py in a child process with LPLB_B200_DEBUG_BOUNDS=1: the
small planner and MoE cases on the bounds-checking build of the extension.

Every data-dependent index of the planner and MoE support kernels is range-checked in that
build; a clean run must leave the violation counters at zero.  One case then feeds the engine
a topology table with an entry one past the last rank: the check has to record it (code,
phase, source line, index, limit) and skip the access, and the step still completes."""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, _native, topology  # noqa: E402
from lplb_b200.models.moe import MoELayer  # noqa: E402


def main():
    assert _native.BOUNDS_CHECK and _native.load().__name__.endswith("_bounds")
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(0)
    avail = torch.zeros(1, dtype=torch.int32, device=dev)
    # clean runs: fused and staged steps on both solvers, odd expert counts, ragged slices, loopback exchange
    for r2o, ll, n_tokens, n_sms in (
        (topology.cube(), 4, 1000, 7), (topology.ring(5), 3, 257, 3), (topology.hypercube(), 2, 4096, 148),
        (topology.torus(3, 3), 3, 5000, 16), (topology.torus(8, 4), 2, 300, 5),
    ):
        g, d = r2o.shape
        planner = Planner(r2o, g * (ll + d), g * ll, g, device=dev)
        idx = torch.randint(-1, g * ll, (n_tokens, 2), device=dev, generator=gen)
        for _ in range(2):
            out = planner.run(idx, avail, n_sms)
        counts, by_sm = planner.count_workload(idx, n_sms)
        probs, _ = planner.solve_probs(counts, avail)
        planner.weighted_select_target(idx, probs, by_sm, n_sms)
        st = planner.check_status()
        assert st.ok and "bounds_skipped" not in st, st
        assert int(out.max()) < g * (ll + d)
    planner = Planner(topology.cube(), 80, 64, 8, device=dev)
    eng = planner._engine
    eng.open_exchange_loopback(2, 0)
    eng.debug_fill_slot(1, torch.arange(64, dtype=torch.int32), eng.completed_launches() + 1)
    eng.run_fused(torch.randint(0, 64, (2048, 4), device=dev), avail, 16, True)
    assert planner.check_status().ok
    # MoE layer: plan, schedule, dispatch, combine under the checks (unfused and fused dispatch)
    small = Planner(topology.cube(), 16 + 16, 16, 8, device=dev)
    layer = MoELayer(small, 256, 128, 2, max_tokens=256)
    x = torch.randn(200, 256, device=dev, generator=gen).bfloat16()
    w, ids = torch.softmax(torch.randn(200, 16, device=dev, generator=gen), -1).topk(2, dim=-1)
    for fused in (False, True):
        layer.fuse_dispatch = fused
        y = layer.forward(x, ids, w, avail, "lplb")
        torch.cuda.synchronize(dev)
        assert layer.check() == 0, layer.engine.status().tolist()
        ref = layer.reference_forward(x, ids, w).float()
        assert float((y.float() - ref).abs().max() / ref.abs().max()) < 2e-2

    # a table entry one past the last rank: recorded, skipped, and the step still completes
    bad = Planner(topology.hypercube(), 16 * 6, 16 * 4, 16, device=dev)
    r2o = topology.hypercube().clone()
    r2o[3, 1] = 16
    bad._engine.set_topology(r2o.to(dev), bad.o2r)
    idx = torch.randint(0, 64, (512, 2), device=dev, generator=gen)
    out = bad.run(idx, avail)
    torch.cuda.synchronize(dev)
    st = bad.check_status()
    assert st["error"] == "index_out_of_bounds" and st["phase"] == "solve", st
    assert st["bounds_index"] == 16 and st["bounds_limit"] == 16 and st["bounds_skipped"] >= 1 and st["bounds_line"] > 0, st
    assert int(out.min()) >= 0 and int(out.max()) < 16 * 6
    assert int(torch.ones(4, device=dev).sum()) == 4  # the context is healthy
    print("BOUNDS_BUILD_OK")


if __name__ == "__main__":
    main()
