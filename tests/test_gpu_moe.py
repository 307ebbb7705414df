"""Single-GPU tests of the benchmark MoE layer kernels against plain PyTorch fp32 references."""

import pytest
import torch

from lplb_b200 import Planner, cube, ring
from lplb_b200.models.moe import MoELayer, interleave_gate_up

pytestmark = pytest.mark.gpu


def _layer(hidden, inter, n_logical, topk, max_tokens, r2o=None, red=2):
    r2o = cube() if r2o is None else r2o
    planner = Planner(r2o, n_logical + red * 8, n_logical, 8, device="cuda", warm_start=False)
    layer = MoELayer(planner, hidden, inter, topk, max_tokens=max_tokens)
    layer.engine.set_timeout_us(1e5)  # a mis-programmed pipeline ends in 0.1 s, with an error code
    return planner, layer


def _inputs(tokens, hidden, n_logical, topk, seed=0):
    g = torch.Generator("cuda").manual_seed(seed)
    x = torch.randn(tokens, hidden, device="cuda", generator=g).bfloat16()
    logits = torch.randn(tokens, n_logical, device="cuda", generator=g)
    w, idx = torch.softmax(logits, -1).topk(topk, dim=-1)
    return x, idx, w


def test_interleave_layout():
    gate = torch.arange(256).float().unsqueeze(1).expand(256, 4)
    up = gate + 1000
    w = interleave_gate_up(gate, up)
    assert w.shape == (512, 4)
    assert w[:128, 0].tolist() == list(range(128)) and w[128:256, 0].tolist() == [1000 + i for i in range(128)]
    assert w[256, 0] == 128 and w[384, 0] == 1128


def test_dispatch_places_every_pair_in_its_experts_rows():
    planner, layer = _layer(512, 256, 32, 4, 1024)
    x, idx, w = _inputs(1000, 512, 32, 4)
    idx[::13, 1] = -1
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    phys = layer.route(idx, avail, "lplb")
    layer.forward_physical(x, phys, w, upto=2)
    torch.cuda.synchronize()
    assert layer.check() == 0
    nl = layer.n_local
    plan = layer.engine.plan().cpu()
    rows, start = plan[:nl].long(), plan[nl : 2 * nl].long()
    valid = phys >= 0
    assert torch.equal(rows, torch.bincount(phys[valid], minlength=nl).cpu())
    assert torch.equal(start, rows.cumsum(0) - rows)
    total = int(rows.sum())
    meta = layer.engine.recv_meta()[:total].long()
    assert int((meta >> 20).max()) == 0  # source rank 0
    slot = meta & 0xFFFFF  # return slot of every received row
    assert sorted(slot.tolist()) == list(range(total))  # a permutation of the return slots
    pair_slot = layer.engine.pair_slot()[: phys.numel()].long()
    assert torch.equal(pair_slot >= 0, valid.reshape(-1))
    pair_of_slot = torch.empty(total, dtype=torch.long, device="cuda")
    pair_of_slot[pair_slot[pair_slot >= 0]] = (pair_slot >= 0).nonzero().reshape(-1)
    pair = pair_of_slot[slot]  # the (token, k) pair behind every received row
    # rows of one expert return to consecutive slots
    for s0, n in zip(start.tolist(), rows.tolist()):
        if n:
            assert slot[s0 : s0 + n].tolist() == list(range(int(slot[s0]), int(slot[s0]) + n))
    assert torch.equal(layer.engine.recv_x()[:total], x[pair // 4])
    owner = torch.repeat_interleave(torch.arange(nl), rows).cuda()
    assert torch.equal(phys.reshape(-1)[pair], owner)


@pytest.mark.parametrize("hidden,inter,tokens,topk", [(512, 256, 1000, 4), (1024, 128, 77, 2), (256, 384, 2048, 8)])
def test_layer_matches_fp32_reference(hidden, inter, tokens, topk):
    planner, layer = _layer(hidden, inter, 32, topk, 2048)
    x, idx, w = _inputs(tokens, hidden, 32, topk, seed=tokens)
    planner.update_redundancy_mapping(torch.bincount(idx.reshape(-1), minlength=32))
    layer.place_weights()
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = layer.reference_forward(x, idx, w).float()
    # fuse: 0 = stand-alone dispatch, 1 = rows sent by extra warps of the first GEMM kernel,
    # 2 = rows sent by 16 CTAs of that kernel that run no tiles
    for policy, fuse in (("lplb", 0), ("static", 0), ("lplb", 1), ("static", 1), ("lplb", 2), ("static", 2), ("lplb", 0)):
        layer.fuse_dispatch = fuse > 0
        layer.send_ctas = 16 if fuse == 2 else 0
        out = layer.forward(x, idx, w, avail, policy)
        torch.cuda.synchronize()
        assert layer.check() == 0
        err = (out.float() - ref).abs().max() / ref.abs().max()
        assert float(err) < 2e-2, (policy, fuse, float(err))
    layer.fuse_dispatch, layer.send_ctas = False, 0
    # the first GEMM alone, row by row, against silu(x Wg^T) * (x Wu^T)
    phys = layer.route(idx, avail, "lplb")
    layer.forward_physical(x, phys, w, upto=3)
    torch.cuda.synchronize()
    plan = layer.engine.plan().cpu()
    nl = layer.n_local
    for slot in range(nl):
        n, s0 = int(plan[slot]), int(plan[nl + slot])
        if n == 0:
            continue
        gate, up, _ = layer.logical_weights(int(planner.phy2log[slot]))
        xin = layer.engine.recv_x()[s0 : s0 + n].float()
        want = torch.nn.functional.silu(xin @ gate.float().T) * (xin @ up.float().T)
        got = layer.engine.act()[s0 : s0 + n].float()
        assert float((got - want).abs().max() / want.abs().max().clamp_min(1e-6)) < 1e-2


def test_repeated_calls_and_replaced_placement():
    planner, layer = _layer(256, 128, 16, 2, 512, r2o=ring(8), red=1)
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = []
    for step in range(5):
        x, idx, w = _inputs(300 + 40 * step, 256, 16, 2, seed=step)
        if step == 3:
            planner.update_redundancy_mapping(torch.bincount(idx.reshape(-1), minlength=16))
            with pytest.raises(RuntimeError):
                layer.forward(x, idx, w, avail)
            layer.place_weights()
        out = layer.forward(x, idx, w, avail)
        ref = layer.reference_forward(x, idx, w).float()
        assert float((out.float() - ref).abs().max() / ref.abs().max()) < 2e-2
        outs.append(out)
    assert layer.check() == 0 and int(layer.engine.epoch()) >= 5


def test_reset_restarts_the_launch_numbering_and_the_layer_keeps_working():
    planner, layer = _layer(256, 128, 16, 2, 512, r2o=ring(8), red=1)
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in range(6):
        layer.fuse_dispatch = step % 2 == 1  # the fused dispatch keeps cumulative arrival counters
        x, idx, w = _inputs(200 + 30 * step, 256, 16, 2, seed=10 + step)
        if step == 3:
            layer.reset()
            assert int(layer.engine.epoch()) == 0 and layer.engine.status().abs().sum().item() == 0
        out = layer.forward(x, idx, w, avail)
        ref = layer.reference_forward(x, idx, w).float()
        assert float((out.float() - ref).abs().max() / ref.abs().max()) < 2e-2
    assert layer.check() == 0 and int(layer.engine.epoch()) == 3


MOE_OVERFLOW = 13  # kMoeOverflow in csrc/moe_gemm.cuh


def _per_row_error(out, ref):
    """Largest error of a row relative to that row's norm: a wrong tile on a row with few or
    small contributions shows up here even when the tensor-wide maximum hides it."""
    num = (out.float() - ref.float()).norm(dim=1)
    den = ref.float().norm(dim=1).clamp_min(1e-3 * float(ref.float().norm(dim=1).mean()))
    return float((num / den).max())


@pytest.mark.parametrize("mode", ["unfused", "fused-warps", "fused-ctas"])
def test_layer_at_the_benchmark_shape_row_by_row(mode):
    """hidden 7168, SwiGLU 2048: 112 K-blocks in the first GEMM and 32 in the second, 16 and 56
    N-tiles, so the pipeline stages and barrier phases wrap dozens of times per tile.  Four
    logical experts (plus replicas) with a few hundred rows each; checked per row."""
    r2o = ring(2)
    planner = Planner(r2o, 4 + 2, 4, 2, device="cuda", warm_start=False)
    layer = MoELayer(planner, 7168, 2048, 2, max_tokens=640, weight_scale=7168**-0.5)
    layer.engine.set_timeout_us(2e5)
    g = torch.Generator("cuda").manual_seed(5)
    x = torch.randn(600, 7168, device="cuda", generator=g).bfloat16()
    logits = torch.randn(600, 4, device="cuda", generator=g) + torch.tensor([1.0, 0.0, -1.0, 0.5], device="cuda")
    w, idx = torch.softmax(logits, -1).topk(2, dim=-1)
    idx[::17, 1] = -1  # some tokens use one expert only
    planner.update_redundancy_mapping(torch.bincount(idx[idx >= 0].reshape(-1), minlength=4))
    layer.place_weights()
    layer.fuse_dispatch = mode != "unfused"
    layer.send_ctas = 16 if mode == "fused-ctas" else 0
    avail = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = layer.reference_forward(x, idx, w)
    for policy in ("lplb", "static"):
        out = layer.forward(x, idx, w, avail, policy)
        torch.cuda.synchronize()
        assert layer.check() == 0, layer.engine.status().tolist()
        assert _per_row_error(out, ref) < 1e-2, (mode, policy)
    # the first GEMM's rows on their own (SwiGLU epilogue), per row as well
    phys = layer.route(idx, avail, "lplb")
    layer.forward_physical(x, phys, w, upto=3)
    torch.cuda.synchronize()
    plan, nl = layer.engine.plan().cpu(), layer.n_local
    for slot in range(nl):
        n, s0 = int(plan[slot]), int(plan[nl + slot])
        if n == 0:
            continue
        gate, up, _ = layer.logical_weights(int(planner.phy2log[slot]))
        xin = layer.engine.recv_x()[s0 : s0 + n].float()
        want = torch.nn.functional.silu(xin @ gate.float().T) * (xin @ up.float().T)
        assert _per_row_error(layer.engine.act()[s0 : s0 + n], want) < 1e-2, (mode, slot)


@pytest.mark.parametrize("fused", [False, True])
def test_receive_buffer_overflow_drops_pairs_and_reports(fused):
    """A receive buffer smaller than the routed pairs: the senders drop what does not fit, the
    status block says so, the kept pairs give exactly what they give without the overflow,
    the dropped ones contribute nothing, and nothing is written past the buffer."""
    planner = Planner(cube(), 32 + 16, 32, 8, device="cuda", warm_start=False)
    layer = MoELayer(planner, 256, 128, 4, max_tokens=256, capacity_rows=384)  # 1024 pairs arrive
    assert layer.capacity == 384
    layer.engine.set_timeout_us(1e5)
    layer.fuse_dispatch = fused
    with pytest.raises(RuntimeError):  # more tokens than the layer was built for: refused on the host
        big = _inputs(257, 256, 32, 4)
        layer.forward_physical(big[0], big[1], big[2])
    x, idx, w = _inputs(256, 256, 32, 4)
    phys = layer.route(idx, torch.zeros(1, dtype=torch.int32, device="cuda"), "static")
    out = layer.forward_physical(x, phys, w)
    torch.cuda.synchronize()
    assert layer.check() == MOE_OVERFLOW
    slots = layer.engine.pair_slot()[: phys.numel()].reshape(phys.shape)
    kept = slots >= 0
    assert int(kept.sum()) == 384  # exactly the capacity was used, the rest dropped
    rows = layer.engine.plan()[: layer.n_local].long()
    assert int(rows.sum()) == 384
    meta = layer.engine.recv_meta()[:384].long()
    assert sorted((meta & 0xFFFFF).tolist()) == sorted(slots[kept].tolist())  # every kept row has its return slot
    assert bool(torch.isfinite(out.float()).all())
    ref = layer.reference_forward(x, torch.where(kept, idx, torch.full_like(idx, -1)), w)
    scale = float(ref.float().abs().max())
    assert float((out.float() - ref.float()).abs().max()) < 2e-2 * scale
    untouched = ~kept.any(dim=1)  # tokens that lost every pair come back as zeros
    if bool(untouched.any()):
        assert float(out[untouched].float().abs().max()) == 0.0
    # the layer recovers once the status is cleared and the batch fits
    layer.reset()
    small = _inputs(64, 256, 32, 4, seed=3)
    phys = layer.route(small[1], torch.zeros(1, dtype=torch.int32, device="cuda"), "static")
    out = layer.forward_physical(small[0], phys, small[2])
    torch.cuda.synchronize()
    assert layer.check() == 0
    ref = layer.reference_forward(*small).float()
    assert float((out.float() - ref).abs().max() / ref.abs().max()) < 2e-2
