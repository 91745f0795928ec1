"""AlphaZero self-play on tic-tac-toe (or connect four): batched tree search over the game rules, policy / value training.

    python examples/alphazero_tictactoe.py [--game connect4] [--iterations 20] [--device cpu]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--game", default="tictactoe", choices=["tictactoe", "connect4"])
    ap.add_argument("--iterations", type=int, default=20)
    ap.add_argument("--games", type=int, default=64)
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args()
    from noeira_b200.agents.alphazero import AlphaZeroAgent, AlphaZeroConfig
    from noeira_b200.envs import ConnectFour, TicTacToe
    game = TicTacToe(args.device) if args.game == "tictactoe" else ConnectFour(args.device)
    ag = AlphaZeroAgent(game, AlphaZeroConfig(hidden=128, n_simulations=40 if args.game == "tictactoe" else 80), device=args.device)
    for it in range(args.iterations):
        n = ag.self_play(args.games)
        for _ in range(40):
            m = ag.train_step()
        w, d, l = ag.play_vs_random(64, agent_first=it % 2 == 0)
        print(f"iteration {it:3d}  positions {n:5d}  loss {m['loss']:.3f}  vs random (64 games): {w} won / {d} drawn / {l} lost")


if __name__ == "__main__":
    main()
