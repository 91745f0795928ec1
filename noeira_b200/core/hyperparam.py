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


def successive_halving(configs: List[dict], objective: Callable[[dict, int], float], min_budget: int = 1, eta: int = 3,
                       max_budget: int = 81, maximize: bool = True, csv_path: str = None):
    """Successive halving: every surviving configuration is evaluated at the current budget (``objective(config, budget)`` —
    training steps, episodes, ...), the best 1/eta move on with eta times the budget.  Returns every evaluation as rows
    ``{..config.., "budget", "score", "rung"}`` sorted best first within the last rung reached."""
    alive, budget, rung, rows = list(configs), min_budget, 0, []
    while alive:
        scored = [(float(objective(c, budget)), i, c) for i, c in enumerate(alive)]
        rows += [{**c, "budget": budget, "score": s, "rung": rung} for s, _, c in scored]
        if budget >= max_budget or len(alive) == 1:
            break
        scored.sort(key=lambda t: t[0], reverse=maximize)
        alive = [c for _, _, c in scored[: max(1, len(scored) // eta)]]
        budget, rung = min(budget * eta, max_budget), rung + 1
    rows.sort(key=lambda r: (r["rung"], r["score"] if maximize else -r["score"]), reverse=True)
    if csv_path:
        _write_csv(csv_path, rows)
    return rows


def search_tabular(agent_factory: Callable[[dict], object], env_factory: Callable[[], object], space: Dict[str, object],
                   episodes: int = 200, n_random: int = 0, seed: int = 0, csv_path: str = None):
    """Grid (or ``n_random`` random draws) over a tabular agent's hyper-parameters; the score of a configuration is the
    mean return of the last quarter of its training episodes.  ``agent_factory(config)`` builds an agent with
    ``train(env, episodes) → returns`` (``agents.tabular.TabularAgent``), ``env_factory()`` its environment."""
    configs = random_configs(space, n_random, seed) if n_random else grid(space)

    def objective(cfg):
        rets = agent_factory(cfg).train(env_factory(), episodes)
        tail = rets[-max(1, episodes // 4):]
        return sum(tail) / len(tail)

    return search(configs, objective, maximize=True, csv_path=csv_path)


def _write_csv(path: str, rows: List[dict]):
    keys = []
    for r in rows:
        keys += [k for k in r if k not in keys]
    with open(path, "w", encoding="utf-8") as f:
        f.write(",".join(keys) + "\n")
        for r in rows:
            f.write(",".join(str(r.get(k, "")) for k in keys) + "\n")
