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


def test_warm_start_on_device_code_matches_the_torch_restatement(sim):
    """A stream of similar batches, then a shifted one: the anchor logic of the device code
    (run under warp emulation) takes the same decisions and iterations as lp.solve_ipm."""
    r2o = topology.cube()
    g, d = r2o.shape
    gen = torch.Generator().manual_seed(11)
    mean = (torch.rand(g, 8, generator=gen, dtype=torch.float64) + 0.5) * 4096
    anchor_c = np.zeros((1, g, 4 * d + 3))
    valid_c = np.zeros(1, np.int32)
    anchor_t = None
    r = np.ascontiguousarray(r2o.numpy().astype(np.int32))
    o = np.ascontiguousarray(topology.invert_r2o(r2o).numpy().astype(np.int32))
    ptr = lambda a: ctypes.c_void_p(a.ctypes.data)  # noqa: E731
    seen = []
    for step in range(5):
        if step == 3:
            mean = mean.flip(0) * torch.linspace(0.3, 2.0, 8, dtype=torch.float64)  # the distribution moves
        cnt = (mean * (1 + 0.02 * torch.randn(g, 8, generator=gen, dtype=torch.float64))).floor().unsqueeze(0)
        w, fixed = cnt[:, :, :d].contiguous(), cnt[:, :, d:].sum(-1)
        ref = lp.solve_ipm(w, fixed, r2o, tol=1e-4, warm_start=True, anchor=anchor_t)
        anchor_t = ref.anchor
        wa, fa = np.ascontiguousarray(w.numpy()), np.ascontiguousarray(fixed.numpy())
        f = np.zeros((1, g, d))
        iters, conv = np.zeros(1, np.int32), np.zeros(1, np.int32)
        rc = sim.lplb_sim_solve_warm(g, d, ptr(r), ptr(o), 1, ptr(wa), ptr(fa), 24, ctypes.c_double(1e-4), ptr(f),
                                     ptr(iters), ptr(conv), ptr(anchor_c), ptr(valid_c), ctypes.c_double(0.05),
                                     ctypes.c_double(1e-3))
        assert rc == 0 and conv[0] == 1
        assert int(iters[0]) == int(ref.iters[0])
        assert float((torch.from_numpy(f) - ref.f).abs().max()) < 1e-5
        _, t_opt = lp.solve_highs(w[0], fixed[0], r2o)
        assert (float(lp.rank_loads(torch.from_numpy(f[0]), w[0], fixed[0], r2o).max()) - t_opt) / t_opt < 1e-3
        seen.append((bool(ref.warm[0]), int(iters[0])))
    assert [s[0] for s in seen] == [False, True, True, False, True]  # cold, warm, warm, guard trips, warm
    assert seen[1][1] < seen[0][1] and seen[2][1] < seen[0][1]


# ---------------------------------------------------------------- thread-block solver
def _solve_block(lib, r2o, w, fixed, max_iters=24, tol=1e-4, anchor=None, valid=None, guard=0.1):
    g, d = r2o.shape
    nb = w.shape[0]
    r = np.ascontiguousarray(r2o.numpy().astype(np.int32))
    o = np.ascontiguousarray(topology.invert_r2o(r2o).numpy().astype(np.int32))
    wa = np.ascontiguousarray(w.numpy().astype(np.float64))
    fa = np.ascontiguousarray(fixed.numpy().astype(np.float64))
    f = np.zeros((nb, g, d))
    iters = np.zeros(nb, np.int32)
    conv = np.zeros(nb, np.int32)
    ptr = lambda a: None if a is None else ctypes.c_void_p(a.ctypes.data)  # noqa: E731
    rc = lib.lplb_sim_solve_block(g, d, ptr(r), ptr(o), nb, ptr(wa), ptr(fa), max_iters, ctypes.c_double(tol), ptr(f),
                                  ptr(iters), ptr(conv), ptr(anchor), ptr(valid), ctypes.c_double(guard),
                                  ctypes.c_double(1e-3))
    assert rc == 0
    return torch.from_numpy(f), iters, conv


@pytest.mark.parametrize("name,nb", [
    ("cube", 2), ("ring5", 2), ("hypercube", 2), ("torus8x4", 2), ("torus8x8", 1), ("ring41", 1),
    ("circ12x3", 1), ("circ10x5", 1),
])
def test_block_solver_device_code_matches_the_torch_restatement(sim, name, nb):
    """The thread-block solver's device code under the block emulation (256 threads, block
    and named barriers, shared memory as a host buffer): one warp of ranks, several warps of
    ranks, group sizes that are not multiples of 8, and the padded replica count."""
    if name == "circ12x3":
        r2o = topology.circulant(12, (1, 2, 5))
    elif name == "circ10x5":
        r2o = topology.circulant(10, (1, 2, 3, 4, 5))
    else:
        r2o = topology.by_name(name)
    g, d = r2o.shape
    gen = torch.Generator().manual_seed(7)
    cnt = ((torch.randn(nb, g, d + 6, generator=gen, dtype=torch.float64) * 0.3 + 1).clamp_min(0) * 4096).floor()
    w, fixed = cnt[:, :, :d].contiguous(), cnt[:, :, d:].sum(-1)
    f, iters, conv = _solve_block(sim, r2o, w, fixed)
    ref = lp.solve_ipm(w, fixed, r2o, tol=1e-4)
    assert conv.all() and bool(((f >= 0) & (f <= 1)).all())
    if d <= 4:  # the padded variant carries extra (empty) variables, so its path differs slightly
        assert iters.tolist() == ref.iters.tolist()
        assert float((f - ref.f).abs().max()) < 1e-5
    for i in range(nb):
        _, t_opt = lp.solve_highs(w[i], fixed[i], r2o)
        mine = float(lp.rank_loads(f[i], w[i], fixed[i], r2o).max())
        assert -1e-9 < (mine - t_opt) / t_opt < 1e-3


def test_block_solver_handles_empty_groups_and_the_iteration_cap(sim):
    r2o = topology.hypercube()
    w = torch.zeros(1, 16, 2, dtype=torch.float64)
    fixed = torch.zeros(1, 16, dtype=torch.float64)
    f, iters, conv = _solve_block(sim, r2o, w, fixed)
    assert conv[0] == 1 and iters[0] == 0 and torch.equal(f, torch.ones(1, 16, 2, dtype=torch.float64))
    w = torch.rand(1, 16, 2, dtype=torch.float64, generator=torch.Generator().manual_seed(1)) * 1000
    fixed = torch.rand(1, 16, dtype=torch.float64, generator=torch.Generator().manual_seed(2)) * 1000
    f, iters, conv = _solve_block(sim, r2o, w, fixed, max_iters=1, tol=1e-9)
    assert conv[0] == 0 and iters[0] == 1 and bool(((f >= 0) & (f <= 1)).all())


def test_block_solver_warm_start_follows_the_torch_restatement(sim):
    r2o = topology.torus(8, 4)
    g, d = r2o.shape
    gen = torch.Generator().manual_seed(13)
    mean = (torch.rand(g, 8, generator=gen, dtype=torch.float64) + 0.5) * 4096
    anchor_c = np.zeros((1, g, 4 * d + 3))
    valid_c = np.zeros(1, np.int32)
    anchor_t = None
    seen = []
    for step in range(4):
        if step == 3:
            mean = mean.flip(0) * torch.linspace(0.3, 2.0, 8, dtype=torch.float64)
        cnt = (mean * (1 + 0.02 * torch.randn(g, 8, generator=gen, dtype=torch.float64))).floor().unsqueeze(0)
        w, fixed = cnt[:, :, :d].contiguous(), cnt[:, :, d:].sum(-1)
        ref = lp.solve_ipm(w, fixed, r2o, tol=1e-4, warm_start=True, anchor=anchor_t, guard=0.1)
        anchor_t = ref.anchor
        f, iters, conv = _solve_block(sim, r2o, w, fixed, anchor=anchor_c, valid=valid_c)
        assert conv[0] == 1 and int(iters[0]) == int(ref.iters[0])
        assert float((f - ref.f).abs().max()) < 1e-5
        seen.append((bool(ref.warm[0]), int(iters[0])))
    assert [s[0] for s in seen] == [False, True, True, False]
    assert seen[1][1] < seen[0][1]


def test_solver_sources_are_clean_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """The solvers' device code, compiled for the host with -fsanitize=address,undefined and run
    on a few instances in a child process: out-of-bounds shared-memory indices, misaligned
    accesses and signed overflow in the index arithmetic would abort the child."""
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    exe = tmp_path / "sim_asan"
    main_cpp = tmp_path / "main.cpp"
    main_cpp.write_text(r'''
#include <cstdio>
#include <vector>
extern "C" int lplb_sim_solve_block(int, int, const int*, const int*, int, const double*, const double*, int, double,
                                    double*, int*, int*, double*, int*, double, double);
extern "C" int lplb_sim_solve(int, int, const int*, const int*, int, const double*, const double*, int, double, double*,
                              int*, int*);
int main() {
  int bad = 0;
  for (int g : {5, 8, 19, 40}) {
    std::vector<int> r2o(g), o2r(g);
    for (int i = 0; i < g; ++i) { r2o[i] = (i + 1) % g; o2r[(i + 1) % g] = i; }
    std::vector<double> w(g), fixed(g), f(g);
    for (int i = 0; i < g; ++i) { w[i] = 100.0 + 37.0 * ((i * 7) % 11); fixed[i] = 500.0 + 13.0 * ((i * 5) % 17); }
    int iters = 0, conv = 0;
    std::vector<double> anchor((size_t)g * 7, 0.0);
    int valid = 0;
    for (int rep = 0; rep < 2; ++rep) {
      bad += lplb_sim_solve_block(g, 1, r2o.data(), o2r.data(), 1, w.data(), fixed.data(), 24, 1e-4, f.data(), &iters,
                                  &conv, anchor.data(), &valid, 0.1, 1e-3);
      bad += conv != 1;
    }
    if (g <= 32) {
      bad += lplb_sim_solve(g, 1, r2o.data(), o2r.data(), 1, w.data(), fixed.data(), 24, 1e-4, f.data(), &iters, &conv);
      bad += conv != 1;
    }
  }
  std::printf("SANITIZED_OK %d\n", bad);
  return bad;
}
''')
    build = subprocess.run(
        ["g++", "-O1", "-g", "-std=c++17", "-pthread", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
         "-fno-omit-frame-pointer", str(CSRC / "sim_solver.cpp"), str(main_cpp), "-o", str(exe)],
        capture_output=True, text=True,
    )
    if build.returncode != 0 and "sanitize" in build.stderr and ("cannot find" in build.stderr or "unrecognized" in build.stderr):
        pytest.skip("host compiler has no sanitizer runtime")
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600,
                         env=dict(__import__("os").environ, ASAN_OPTIONS="detect_leaks=0"))
    assert run.returncode == 0, run.stdout[-1000:] + run.stderr[-3000:]
    assert "SANITIZED_OK 0" in run.stdout
