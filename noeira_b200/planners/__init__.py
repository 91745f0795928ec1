from .trajectory import CEM, MPPI, PhysicsRollout, RandomShooting  # noqa: F401
from .ilqr import ILQR  # noqa: F401
