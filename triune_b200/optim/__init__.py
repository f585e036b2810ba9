"""Optimizers: three-tier CentroidSteer, Muon, manifold optimizers and subspace algebra."""

from .arena import ParamArena
from .centroid import CentroidSteerOptimizer, classify_parameters, muon_update_scale
from .factory import build_optimizer
from .manifold import LowSpaceWeightProjector, QuantumUnitaryOptimizer, UnitaryManifoldOptimizer
from .muon import Muon, zeropower_via_newtonschulz5
from .subspace import batched_qr, batched_subspace_projection, cholesky_qr, polar_stiefel_retraction, subspace_projection

__all__ = [
    "ParamArena", "CentroidSteerOptimizer", "classify_parameters", "muon_update_scale", "build_optimizer",
    "LowSpaceWeightProjector", "QuantumUnitaryOptimizer", "UnitaryManifoldOptimizer", "Muon",
    "zeropower_via_newtonschulz5", "batched_qr", "batched_subspace_projection", "cholesky_qr",
    "polar_stiefel_retraction", "subspace_projection",
]
