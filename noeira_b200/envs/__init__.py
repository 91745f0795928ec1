from .batched_env import BatchedEnv, HalfCheetahEnv, HopperEnv, Physics3dBatchedEnv, PlanarChainEnv  # noqa: F401
