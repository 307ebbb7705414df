"""lplb_b200 — LP-based per-batch load balancer for expert-parallel MoE on B200.

Public surface (mirrors reference ``lplb/__init__.py:1-4`` and adds the topology
builders that the reference only ships as test constants):

* :class:`Planner` – count -> exchange -> solve -> redirect, plus expert re-placement.
* ``topology`` – ``cube()``, ``hypercube()``, ``torus(m, n)``, ``ring(n)`` ``r2o`` builders.
* ``eplb``     – the embedded placement balancer.
* ``lp``       – LP builders and float64 oracles.
"""

from . import eplb, lp, topology
from .planner import Planner, PlannerStatus
from .topology import cube, hypercube, ring, torus

__version__ = "0.1.0"

__all__ = ["Planner", "PlannerStatus", "topology", "eplb", "lp", "cube", "hypercube", "ring", "torus", "__version__"]
