from .batched_env import BatchedEnv, HalfCheetahEnv, HopperEnv, Physics3dBatchedEnv, PlanarChainEnv  # noqa: F401
from .classic import CartPoleEnv, MountainCarContinuousEnv, PendulumEnv  # noqa: F401
from .lunar_lander import BipedalWalkerEnv, LunarLanderEnv  # noqa: F401
from .board_games import ConnectFour, LineGame, TicTacToe  # noqa: F401
