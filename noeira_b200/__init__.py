"""noeira_b200 — a Blackwell (sm_100a) native physical-AI training framework.

Layout:
    nn/        Module / Param networks with explicit per-module VJPs, arena optimizers, AMP, checkpoints
    ops/       Python entry points of the hand-written CUDA kernels (csrc/*.cu)
    parallel/  symmetric heap, fused collectives, DDP / ZeRO / TP+SP strategies, CPU simulator
    physics/   batched generalized-coordinate rigid-body engine (fused step kernel + NumPy oracle)
    envs/      batched reset/step environments
    agents/    SAC, PPO, TD3, ACT, SmolVLA-style VLA and Dreamer-style world-model trainers
    models/    GPT, ViT, ResNet-18, ACT, VLA, world-model networks
    data/ io/ utils/
"""
__version__ = "0.1.0"
