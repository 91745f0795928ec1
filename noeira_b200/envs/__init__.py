from .batched_env import (BatchedEnv, HalfCheetahEnv, HopperEnv, InvertedDoublePendulumEnv, InvertedPendulumEnv,  # noqa: F401
                          Physics3dBatchedEnv, PlanarChainEnv, ReacherEnv, Walker2dEnv)
from .classic import AcrobotEnv, CartPoleEnv, DiscreteActions, MountainCarContinuousEnv, PendulumEnv  # noqa: F401
from .lunar_lander import BipedalWalkerEnv, LunarLanderEnv  # noqa: F401
from .board_games import ConnectFour, LineGame, TicTacToe  # noqa: F401
from .car_racing import CarRacingDiscreteEnv, CarRacingEnv, CarRacingPixelEnv, make_track, scripted_driver  # noqa: F401
