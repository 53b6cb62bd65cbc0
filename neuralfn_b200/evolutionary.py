"""Genetic-algorithm trainer over the edge parameters of a scalar graph, evaluated with
the real executor (works for cyclic graphs and non-differentiable neurons).
Tournament selection (3), uniform crossover (0.5), Gaussian mutation (rate 0.1, scale 0.3),
2 elites, population 50 x 200 generations by default - the knobs of the reference's
``EvolutionaryTrainer`` (``neuralfn/evolutionary.py:28-188``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Sequence

import numpy as np

from .graph import NeuronGraph

__all__ = ["EvoConfig", "EvolutionaryTrainer"]


@dataclass
class EvoConfig:
    population_size: int = 50
    generations: int = 200
    mutation_rate: float = 0.1
    mutation_scale: float = 0.3
    crossover_rate: float = 0.5
    tournament_size: int = 3
    elite_count: int = 2
    loss_fn: str = "mse"
    seed: int | None = None
    init_scale: float = 1.0


class EvolutionaryTrainer:
    def __init__(self, graph: NeuronGraph, config: EvoConfig | None = None) -> None:
        self.graph = graph
        self.config = config or EvoConfig()
        self.loss_history: list[float] = []
        self._stop = False

    def stop(self) -> None:
        self._stop = True

    def _loss(self, params: np.ndarray, xs, ys) -> float:
        g = self.graph
        g.set_edge_params(params.tolist())
        total, count = 0.0, 0
        for x, y in zip(xs, ys):
            out = g.execute_flat(tuple(float(v) for v in x))
            for o, t in zip(out, y):
                if self.config.loss_fn == "bce":
                    p = min(max(o, 1e-7), 1 - 1e-7)
                    total += -(t * np.log(p) + (1 - t) * np.log(1 - p))
                else:
                    total += (o - t) ** 2
                count += 1
        return total / max(count, 1)

    def train(self, train_inputs: Sequence[Sequence[float]], train_targets: Sequence[Sequence[float]],
              on_generation: Callable[[int, float], None] | None = None) -> list[float]:
        c = self.config
        rng = np.random.default_rng(c.seed)
        base = np.asarray(self.graph.get_edge_params(), dtype=np.float64)
        n = base.size
        pop = base[None, :] + rng.normal(0.0, c.init_scale, size=(c.population_size, n))
        pop[0] = base
        fitness = np.array([self._loss(ind, train_inputs, train_targets) for ind in pop])
        for gen in range(c.generations):
            if self._stop:
                break
            order = np.argsort(fitness)
            pop, fitness = pop[order], fitness[order]
            self.loss_history.append(float(fitness[0]))
            if on_generation is not None:
                on_generation(gen, float(fitness[0]))
            nxt = [pop[i].copy() for i in range(min(c.elite_count, c.population_size))]
            while len(nxt) < c.population_size:
                def pick() -> np.ndarray:
                    cand = rng.integers(0, c.population_size, size=c.tournament_size)
                    return pop[cand[np.argmin(fitness[cand])]]
                a, b = pick(), pick()
                child = np.where(rng.random(n) < c.crossover_rate, a, b)
                mask = rng.random(n) < c.mutation_rate
                child = child + mask * rng.normal(0.0, c.mutation_scale, size=n)
                nxt.append(child)
            pop = np.stack(nxt)
            fitness = np.array([self._loss(ind, train_inputs, train_targets) for ind in pop])
        best = int(np.argmin(fitness))
        self.graph.set_edge_params(pop[best].tolist())
        self.loss_history.append(float(fitness[best]))
        return self.loss_history
