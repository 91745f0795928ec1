"""``python -m noeira_b200.build [--force] [-v]`` — compile the in-tree native libraries."""
import sys

from ._native import build, ptxas_report

if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=False)
    if "-v" in sys.argv:
        print(ptxas_report())
    print("built")
