import pytest
import torch

from lplb_b200 import topology


def test_named_topologies_match_published_matrices():
    # literal matrices of the reference's test constants (reference tests/utils.py:97-113)
    cube = torch.tensor([[3, 0, 1, 2, 7, 4, 5, 6], [6, 7, 4, 5, 0, 1, 2, 3]]).T
    ring = torch.tensor([[1, 2, 3, 4, 5, 6, 7, 0]]).T
    hyper = torch.tensor(
        [[3, 0, 1, 2, 7, 4, 5, 6, 11, 8, 9, 10, 15, 12, 13, 14], [12, 13, 14, 15, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]]
    ).T
    assert torch.equal(topology.cube().long(), cube)
    assert torch.equal(topology.ring(8).long(), ring)
    assert torch.equal(topology.hypercube().long(), hyper)


def test_torus_formula():
    m, n = 8, 4
    t = topology.torus(m, n)
    want = torch.tensor([[(i + 1) % m * n + j, i * n + (j + 1) % n] for i in range(m) for j in range(n)])
    assert torch.equal(t.long(), want)


@pytest.mark.parametrize("name", ["ring8", "cube", "hypercube", "torus8x4", "torus2x4", "torus4x4", "ring5"])
def test_columns_are_permutations_and_invert(name):
    r2o = topology.by_name(name)
    topology.validate_r2o(r2o)
    o2r = topology.invert_r2o(r2o)
    g, d = r2o.shape
    for col in range(d):
        for rank in range(g):
            assert int(r2o[int(o2r[rank, col]), col]) == rank
    # argsort(dim=0) is how the reference inverts (reference lplb/planner.py:67)
    assert torch.equal(o2r.long(), r2o.long().argsort(dim=0))


def test_validate_rejects_bad_matrices():
    with pytest.raises(ValueError):
        topology.validate_r2o(torch.tensor([[0], [0], [1]]))
    with pytest.raises(ValueError):
        topology.validate_r2o(torch.tensor([[0], [2], [1]]))  # rank 0 replicates itself
    topology.validate_r2o(torch.tensor([[0], [2], [1]]), allow_self_edges=True)
    with pytest.raises(ValueError):
        topology.validate_r2o(torch.tensor([1, 0]))


def test_edge_list():
    origin, holder = topology.edge_list(topology.cube())
    assert origin.tolist() == [i for i in range(8) for _ in range(2)]
    r2o = topology.cube()
    for k in range(16):
        assert int(r2o[holder[k], k % 2]) == int(origin[k])
