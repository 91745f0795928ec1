from .trainer import AutoregressiveTrainer, Trainer  # noqa: F401
