"""Grid and random hyper-parameter search with CSV export (noeira/core/hyperparam/: grid / random search, CSV export)."""
from __future__ import annotations

import itertools
import random
from typing import Callable, Dict, List, Sequence


def grid(space: Dict[str, Sequence]) -> List[dict]:
    keys = list(space)
    return [dict(zip(keys, vals)) for vals in itertools.product(*[space[k] for k in keys])]


def random_configs(space: Dict[str, object], n: int, seed: int = 0) -> List[dict]:
    """A value is a list (uniform choice), ``("uniform", lo, hi)``, ``("loguniform", lo, hi)`` or ``("int", lo, hi)``."""
    import math
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        c = {}
        for k, v in space.items():
            if isinstance(v, tuple) and v and v[0] == "uniform":
                c[k] = rng.uniform(v[1], v[2])
            elif isinstance(v, tuple) and v and v[0] == "loguniform":
                c[k] = math.exp(rng.uniform(math.log(v[1]), math.log(v[2])))
            elif isinstance(v, tuple) and v and v[0] == "int":
                c[k] = rng.randint(v[1], v[2])
            else:
                c[k] = rng.choice(list(v))
        out.append(c)
    return out


def search(configs: List[dict], objective: Callable[[dict], float], maximize: bool = True, csv_path: str = None):
    rows = [{**c, "score": float(objective(c))} for c in configs]
    rows.sort(key=lambda r: r["score"], reverse=maximize)
    if csv_path:
        keys = list(rows[0])
        with open(csv_path, "w", encoding="utf-8") as f:
            f.write(",".join(keys) + "\n")
            for r in rows:
                f.write(",".join(str(r[k]) for k in keys) + "\n")
    return rows
