"""Worker run by tests/test_multigpu.py under torch.distributed.run (one rank per GPU).

Checks the in-kernel NVLink statistics exchange against ``torch.distributed.all_reduce``,
that every rank computes identical shares, and that a rank which skips a step makes the
others' bounded wait run out, report, and recover after a collective reset.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, cube, hypercube, lp  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD

    # cold solves here: the steps below compare shares bit for bit with a second planner
    planner = Planner(cube(), 256 + 16, 256, 8, group, device=dev, comm="p2p", peer_timeout_us=2e5, warm_start=False)
    assert planner.comm == "p2p" and planner.deep_ep_initialized

    # 1. stand-alone exchange is bitwise equal to NCCL's all-reduce, many times in a row
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    for step in range(20):
        mine = torch.randint(0, 5000, (256,), device=dev, generator=gen, dtype=torch.int32)
        want = mine.clone()
        dist.all_reduce(want, group=group)
        got = planner._engine.all_reduce_counts(mine)
        assert torch.equal(got, want), f"rank {rank} step {step}: exchange differs from all_reduce"

    # 2. fused run: global statistics, identical shares on every rank, balanced result
    bias = torch.randn(256, device=dev, generator=torch.Generator(device=dev).manual_seed(7))
    hist = None
    for step in range(12):
        logits = torch.randn(4096, 256, device=dev, generator=gen) + bias
        idx = logits.bfloat16().topk(8, dim=-1).indices
        counts = torch.bincount(idx.reshape(-1), minlength=256)
        dist.all_reduce(counts, group=group)
        if step == 2:
            planner.update_redundancy_mapping(counts)  # same on every rank
        avail = torch.zeros(1, dtype=torch.int32, device=dev)
        out = planner.run(idx, avail, 148 if step % 2 else 37)
        assert int(avail) == 1
        ws = planner._engine.workspace()
        assert torch.equal(ws[8 + 2 * 256 : 8 + 3 * 256].long(), counts), f"rank {rank}: global counts differ"
        probs = planner.last_probs.clone()
        gathered = [torch.empty_like(probs) for _ in range(world)]
        dist.all_gather(gathered, probs, group=group)
        assert all(torch.equal(g, probs) for g in gathered), "shares differ between ranks"
        pl = planner.n_local_routed_experts
        load = torch.bincount(out.reshape(-1) // pl, minlength=8).double()
        dist.all_reduce(load, group=group)
        w, fixed = lp.bundle_loads(counts.cpu().double(), planner.phy2log.cpu(), 1, 8, 2, 32, 1)
        _, t_opt = lp.solve_highs(w[0], fixed[0], cube())
        assert float(load.max()) <= t_opt * (1 + 1e-3) + 8 * world, (float(load.max()), t_opt)
        assert planner.check_status().ok
    hist = counts

    # 2a. four LP groups (ep_size 32 on the Cube) and four redundant experts per rank (two per
    # topology slot), statistics from the `world` real ranks over the in-kernel exchange
    keep_alive = []
    # and two groups of 16 ranks (thread-block solver): `run` gives each group a CTA of its own,
    # so it counts, exchanges (stand-alone exchange kernel over the same peer slots), solves and
    # redirects in separate launches
    for name, r2o, ep_size, n_red in (("four groups", cube(), 32, 2), ("two experts per slot", cube(), 8, 4),
                                      ("two wide groups", hypercube(), 32, 2)):
        multi = Planner(r2o, 256 + n_red * ep_size, 256, ep_size, group, device=dev, comm="p2p", warm_start=False)
        one_launch = not (multi.n_group > 1 and multi._engine.solver() == "block")
        for step in range(4):
            logits = torch.randn(2048, 256, device=dev, generator=gen) + bias
            idx = logits.bfloat16().topk(8, dim=-1).indices
            counts = torch.bincount(idx.reshape(-1), minlength=256)
            dist.all_reduce(counts, group=group)
            if step == 1:
                multi.update_redundancy_mapping(counts)
            avail = torch.zeros(1, dtype=torch.int32, device=dev)
            multi.run(idx, avail, 148 if step % 2 else 20)
            assert int(avail) == multi.n_group, name
            if one_launch:
                ws = multi._engine.workspace()
                assert torch.equal(ws[8 + 2 * 256 : 8 + 3 * 256].long(), counts), f"rank {rank}: {name}: global counts differ"
            probs = multi.last_probs.clone()
            gathered = [torch.empty_like(probs) for _ in range(world)]
            dist.all_gather(gathered, probs, group=group)
            assert all(torch.equal(g, probs) for g in gathered), f"{name}: shares differ between ranks"
            assert multi.check_status().ok
        keep_alive.append(multi)  # peers stay mapped until every rank is done

    # 3. a rank skips one step: the others' wait runs out, they report it and still route
    dist.barrier(group=group)
    torch.cuda.synchronize(dev)
    logits = torch.randn(1024, 256, device=dev, generator=gen) + bias
    idx = logits.topk(8, dim=-1).indices
    avail = torch.zeros(1, dtype=torch.int32, device=dev)
    if rank != world - 1:
        out = planner.run(idx, avail)
        torch.cuda.synchronize(dev)
        st = planner.check_status(clear=True)
        assert st["error"] == "peer_timeout" and st["detail"] == 1 << (world - 1), st
        assert int(avail) == 1 and int(out.min()) >= 0
    # the absence is learnt on the host; everybody resets the exchange before the next launch
    planner.reset_exchange()
    for step in range(4):
        logits = torch.randn(1024, 256, device=dev, generator=gen) + bias
        idx = logits.topk(8, dim=-1).indices
        counts = torch.bincount(idx.reshape(-1), minlength=256)
        dist.all_reduce(counts, group=group)
        avail.zero_()
        planner.run(idx, avail)
        ws = planner._engine.workspace()
        assert torch.equal(ws[8 + 2 * 256 : 8 + 3 * 256].long(), counts)
        assert planner.check_status().ok

    # 4. the NCCL pipeline gives the same shares as the fused kernel
    staged = Planner(cube(), 256 + 16, 256, 8, group, device=dev, comm="nccl", warm_start=False)
    staged.load_state_dict(planner.state_dict())
    avail.zero_()
    out_f = planner.run(idx, avail)
    local_counts, by_sm = staged.count_workload(idx, 148)
    probs_s, _ = staged.solve_probs(local_counts, avail)
    assert torch.equal(probs_s, planner.last_probs)

    # 4a. two-level schedule (nodes of world/2 ranks) is bitwise equal to the all-reduce as well
    if world >= 4:
        two = Planner(cube(), 256 + 16, 256, 8, group, device=dev, comm="p2p", exchange_node_size=world // 2,
                      warm_start=False)
        for step in range(10):
            mine = torch.randint(0, 5000, (256,), device=dev, generator=gen, dtype=torch.int32)
            want = mine.clone()
            dist.all_reduce(want, group=group)
            assert torch.equal(two._engine.all_reduce_counts(mine), want), f"rank {rank}: two-level exchange differs"
        idx = (torch.randn(2048, 256, device=dev, generator=gen) + bias).topk(8, dim=-1).indices
        counts = torch.bincount(idx.reshape(-1), minlength=256)
        dist.all_reduce(counts, group=group)
        avail.zero_()
        two.run(idx, avail)
        assert torch.equal(two._engine.workspace()[8 + 2 * 256 : 8 + 3 * 256].long(), counts)
        assert two.check_status().ok

    # 4b. warm-started solves stay identical on every rank (same history, same arithmetic)
    warm = Planner(cube(), 256 + 16, 256, 8, group, device=dev, comm="p2p", peer_timeout_us=2e5)
    assert warm.warm_start  # the library default
    warm.load_state_dict(planner.state_dict())
    warm_iters = []
    for step in range(6):
        logits = torch.randn(4096, 256, device=dev, generator=gen) + bias
        idx = logits.bfloat16().topk(8, dim=-1).indices
        avail.zero_()
        warm.run(idx, avail)
        probs = warm.last_probs.clone()
        gathered = [torch.empty_like(probs) for _ in range(world)]
        dist.all_gather(gathered, probs, group=group)
        assert all(torch.equal(g, probs) for g in gathered), "warm-started shares differ between ranks"
        st = warm.check_status(clear=True)
        assert st.ok and int(avail) == 1
        warm_iters.append(st["lp_iters"])
    assert min(warm_iters[1:]) < warm_iters[0], warm_iters
    # 4c. a step whose exchange times out must not leave a saved iterate behind: the ranks that
    # saw the timeout drop theirs inside the kernel, and after the collective reset every rank
    # starts cold again, so the shares agree without anybody having to remember to invalidate
    dist.barrier(group=group)
    torch.cuda.synchronize(dev)
    idx = (torch.randn(1024, 256, device=dev, generator=gen) + bias).topk(8, dim=-1).indices
    if rank != world - 1:
        avail.zero_()
        warm.run(idx, avail)
        torch.cuda.synchronize(dev)
        st = warm.check_status(clear=True)
        assert st["error"] == "peer_timeout", st
        assert int(warm._engine.warm_start_valid().sum()) == 0, "a timed-out step left a warm-start state behind"
    warm.reset_exchange()
    for step in range(3):
        idx = (torch.randn(4096, 256, device=dev, generator=gen) + bias).bfloat16().topk(8, dim=-1).indices
        avail.zero_()
        warm.run(idx, avail)
        probs = warm.last_probs.clone()
        gathered = [torch.empty_like(probs) for _ in range(world)]
        dist.all_gather(gathered, probs, group=group)
        assert all(torch.equal(g, probs) for g in gathered), "shares differ between ranks after a timeout and a reset"
        assert warm.check_status(clear=True).ok

    # 5. expert-parallel MoE layer over the same ranks: dispatch and combine cross NVLink
    from lplb_b200 import ring
    from lplb_b200.models.moe import MoELayer

    r2o = cube() if world == 8 else ring(world)
    red = r2o.shape[1]
    n_logical = 4 * world
    mp = Planner(r2o, n_logical + red * world, n_logical, world, group, device=dev, comm="p2p", warm_start=False)
    layer = MoELayer(mp, 512, 256, 4, max_tokens=512, group=group, capacity_factor=4.0)
    layer.engine.set_timeout_us(2e5)
    single = Planner(r2o, n_logical + red * world, n_logical, world, device=dev)  # reference weights only
    ref_layer = MoELayer(single, 512, 256, 4, max_tokens=512)
    for step in range(4):
        g2 = torch.Generator(device=dev).manual_seed(1000 * step + rank)
        tokens = 300 + 17 * rank
        x = torch.randn(tokens, 512, device=dev, generator=g2).bfloat16()
        logits = torch.randn(tokens, n_logical, device=dev, generator=g2) + torch.linspace(-1, 1, n_logical, device=dev)
        w, idx = torch.softmax(logits, -1).topk(4, dim=-1)
        if step == 1:
            hist = torch.bincount(idx.reshape(-1), minlength=n_logical)
            dist.all_reduce(hist, group=group)
            mp.update_redundancy_mapping(hist)
            layer.place_weights()
        if step == 3:
            layer.reset()  # collective: flags, counters and launch numbers start over on every rank
        avail.zero_()
        layer.fuse_dispatch = step >= 2  # later steps send the rows from inside the first GEMM
        layer.send_ctas = 16 if step >= 3 else 0  # and the last ones from CTAs that run no tiles
        out = layer.forward(x, idx, w, avail, "lplb" if step % 2 == 0 else "static")
        torch.cuda.synchronize(dev)
        assert layer.check() == 0, layer.engine.status().tolist()
        ref = ref_layer.reference_forward(x, idx, w).float()
        err = float((out.float() - ref).abs().max() / ref.abs().max())
        assert err < 2e-2, f"rank {rank} step {step}: MoE output differs from the reference by {err}"

    dist.barrier(group=group)
    torch.cuda.synchronize(dev)
    if rank == 0:
        print("DIST_WORKER_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
