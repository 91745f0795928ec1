from .trajectory import CEM, MPPI, PhysicsRollout, RandomShooting  # noqa: F401
