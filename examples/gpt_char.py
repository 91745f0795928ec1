"""Character-level GPT on a text file (CPU or CUDA): AutoregressiveTrainer with warm-up + cosine schedule.

    python examples/gpt_char.py corpus.txt [--device cuda] [--steps 500]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("corpus")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--batch", type=int, default=32)
    args = ap.parse_args()
    from noeira_b200.data.datasets import CharCorpus
    from noeira_b200.models.gpt import GPT
    from noeira_b200.training import AutoregressiveTrainer
    corpus = CharCorpus.from_file(args.corpus)
    vocab = (corpus.vocab + 7) // 8 * 8
    model = GPT(vocab=vocab, seq=args.seq, dim=256, layers=4, heads=4, dropout=0.0).to(args.device)
    toks = torch.from_numpy(corpus.tokens).to(args.device)
    tr = AutoregressiveTrainer(model, toks, args.batch, args.seq, lr=3e-4, warmup=50, total_steps=args.steps,
                               use_cuda_graph=args.device == "cuda")
    for s in range(args.steps):
        tr.train_step()
        if (s + 1) % 50 == 0:
            print(s + 1, "loss", round(tr.mean_loss() / 50, 4))


if __name__ == "__main__":
    main()
