"""Run the CUDA solver's device code on the CPU through the lock-step warp emulation
(csrc/host_sim.h) and compare it with the float64 oracle."""

import ctypes
import shutil
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from lplb_b200 import lp, topology

CSRC = Path(__file__).resolve().parents[1] / "lplb_b200" / "csrc"


@pytest.fixture(scope="module")
def sim(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    so = tmp_path_factory.mktemp("sim") / "libsim.so"
    subprocess.run(
        ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", str(CSRC / "sim_solver.cpp"), "-o", str(so)],
        check=True,
    )
    return ctypes.CDLL(str(so))


def _solve(lib, r2o, w, fixed, max_iters=24, tol=1e-4):
    g, d = r2o.shape
    nb = w.shape[0]
    r = np.ascontiguousarray(r2o.numpy().astype(np.int32))
    o = np.ascontiguousarray(topology.invert_r2o(r2o).numpy().astype(np.int32))
    wa = np.ascontiguousarray(w.numpy().astype(np.float64))
    fa = np.ascontiguousarray(fixed.numpy().astype(np.float64))
    f = np.zeros((nb, g, d))
    iters = np.zeros(nb, np.int32)
    conv = np.zeros(nb, np.int32)
    ptr = lambda a: ctypes.c_void_p(a.ctypes.data)  # noqa: E731
    rc = lib.lplb_sim_solve(g, d, ptr(r), ptr(o), nb, ptr(wa), ptr(fa), max_iters, ctypes.c_double(tol), ptr(f), ptr(iters), ptr(conv))
    assert rc == 0
    return torch.from_numpy(f), iters, conv


@pytest.mark.parametrize("name,nb", [("cube", 9), ("ring8", 6), ("hypercube", 3), ("ring5", 5), ("torus2x4", 4)])
def test_device_solver_matches_oracle(sim, name, nb):
    r2o = topology.by_name(name)
    g, d = r2o.shape
    gen = torch.Generator().manual_seed(7)
    cnt = ((torch.randn(nb, g, 8, generator=gen, dtype=torch.float64) * 0.3 + 1).clamp_min(0) * 4096).floor()
    w, fixed = cnt[:, :, :d].contiguous(), cnt[:, :, d:].sum(-1)
    if nb > 2:  # an empty group sharing a warp with live ones
        w[2], fixed[2] = 0, 0
    f, iters, conv = _solve(sim, r2o, w, fixed)
    assert conv.all() and bool(((f >= 0) & (f <= 1)).all())
    for i in range(nb):
        if float(w[i].sum() + fixed[i].sum()) == 0:
            assert torch.equal(f[i], torch.ones(g, d, dtype=torch.float64)) and iters[i] == 0
            continue
        _, t_opt = lp.solve_highs(w[i], fixed[i], r2o)
        mine = float(lp.rank_loads(f[i], w[i], fixed[i], r2o).max())
        assert -1e-9 < (mine - t_opt) / t_opt < 1e-3
        assert 1 <= iters[i] <= 12


def test_device_solver_follows_the_torch_restatement(sim):
    r2o = topology.cube()
    gen = torch.Generator().manual_seed(3)
    cnt = ((torch.randn(8, 8, 8, generator=gen, dtype=torch.float64) * 0.3 + 1).clamp_min(0) * 4096).floor()
    w, fixed = cnt[:, :, :2].contiguous(), cnt[:, :, 2:].sum(-1)
    f, iters, _ = _solve(sim, r2o, w, fixed)
    ref = lp.solve_ipm(w, fixed, r2o, tol=1e-4)
    assert iters.tolist() == ref.iters.tolist()
    assert float((f - ref.f).abs().max()) < 1e-5


def test_iteration_cap_is_reported(sim):
    r2o = topology.cube()
    w = torch.rand(2, 8, 2, dtype=torch.float64, generator=torch.Generator().manual_seed(1)) * 1000
    fixed = torch.rand(2, 8, dtype=torch.float64, generator=torch.Generator().manual_seed(2)) * 1000
    f, iters, conv = _solve(sim, r2o, w, fixed, max_iters=1, tol=1e-9)
    assert not conv.any() and iters.tolist() == [1, 1]
    assert bool(((f >= 0) & (f <= 1)).all())
