"""Differentiable stand-ins for arbitrary scalar neurons, and the Adam trainer that
optimises edge parameters through them.

``probe_neuron`` samples a neuron's transfer function (10 k uniform points in each port's
range, or [-1, 1] when unbounded), ``SurrogateModel`` is an MLP(64, 64, SiLU) fitted to the
samples with Adam for 200 epochs, ``build_surrogates`` does this for every distinct
function neuron of a graph, and ``SurrogateTrainer`` runs Adam on the flat ``[w, b] * E``
tensor through the frozen surrogates, then writes the parameters back.
Reference: ``neuralfn/surrogate.py:14-121``, ``neuralfn/trainer.py:34-203``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Sequence

import numpy as np
import torch
import torch.nn as nn

from .graph import NeuronGraph
from .neuron import NeuronDef

__all__ = ["SurrogateModel", "probe_neuron", "build_surrogates", "TrainConfig", "SurrogateTrainer"]


class SurrogateModel(nn.Module):
    def __init__(self, n_inputs: int, n_outputs: int, hidden: int = 64) -> None:
        super().__init__()
        self.net = nn.Sequential(nn.Linear(n_inputs, hidden), nn.SiLU(), nn.Linear(hidden, hidden), nn.SiLU(),
                                 nn.Linear(hidden, n_outputs))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x)

    def fit(self, xs: np.ndarray, ys: np.ndarray, epochs: int = 200, lr: float = 1e-2, batch: int = 1024) -> float:
        x = torch.as_tensor(xs, dtype=torch.float32)
        y = torch.as_tensor(ys, dtype=torch.float32)
        opt = torch.optim.Adam(self.parameters(), lr=lr)
        last = 0.0
        for _ in range(epochs):
            perm = torch.randperm(x.size(0))
            for i in range(0, x.size(0), batch):
                idx = perm[i:i + batch]
                loss = nn.functional.mse_loss(self(x[idx]), y[idx])
                opt.zero_grad()
                loss.backward()
                opt.step()
                last = float(loss.detach())
        for p in self.parameters():
            p.requires_grad = False
        return last


def probe_neuron(ndef: NeuronDef, n_samples: int = 10_000, seed: int = 0) -> tuple[np.ndarray, np.ndarray]:
    rng = np.random.default_rng(seed)
    cols = []
    for port in ndef.input_ports:
        lo, hi = port.range if port.range is not None else (-1.0, 1.0)
        cols.append(rng.uniform(lo, hi, size=n_samples))
    xs = np.stack(cols, axis=1) if cols else np.zeros((n_samples, 0))
    ys = np.array([ndef(*row) for row in xs], dtype=np.float64).reshape(n_samples, -1)
    return xs, ys


def build_surrogates(graph: NeuronGraph, n_samples: int = 10_000, epochs: int = 200, hidden: int = 64,
                     seed: int = 0) -> dict[str, SurrogateModel]:
    """One surrogate per distinct neuron definition id (function and subgraph neurons)."""
    out: dict[str, SurrogateModel] = {}
    torch.manual_seed(seed)
    for node in graph.nodes.values():
        nd = node.neuron_def
        if nd.kind == "module" or nd.id in out or nd.n_inputs == 0:
            continue
        xs, ys = probe_neuron(nd, n_samples, seed)
        model = SurrogateModel(nd.n_inputs, nd.n_outputs, hidden)
        model.fit(xs, ys, epochs=epochs)
        out[nd.id] = model
    return out


@dataclass
class TrainConfig:
    learning_rate: float = 1e-2
    epochs: int = 200
    batch_size: int = 32
    loss_fn: str = "mse"  # "mse" | "bce"
    surrogate_samples: int = 10_000
    surrogate_epochs: int = 200
    surrogate_hidden: int = 64
    seed: int = 0


class SurrogateTrainer:
    def __init__(self, graph: NeuronGraph, config: TrainConfig | None = None,
                 surrogates: dict[str, SurrogateModel] | None = None) -> None:
        if graph.has_cycles():
            raise ValueError("SurrogateTrainer needs an acyclic graph")
        self.graph = graph
        self.config = config or TrainConfig()
        self.surrogates = surrogates
        self.loss_history: list[float] = []
        self._stop = False

    def stop(self) -> None:
        self._stop = True

    def _forward(self, params: torch.Tensor, x: torch.Tensor, edge_index: dict[str, int]) -> torch.Tensor:
        g = self.graph
        values: dict[str, list[torch.Tensor]] = {}
        cur = 0
        for nid in g.input_node_ids:
            n = g.nodes[nid].neuron_def.n_outputs
            values[nid] = [x[:, cur + i] for i in range(n)]
            cur += n
        for nid in g.topological_order():
            if nid in values:
                continue
            nd = g.nodes[nid].neuron_def
            acc = [torch.zeros(x.size(0)) for _ in range(nd.n_inputs)]
            for e in g._incoming(nid):
                i = edge_index[e.id]
                src = values[e.src_node][e.src_port]
                raw = src * params[2 * i] + params[2 * i + 1]
                port = nd.input_ports[e.dst_port]
                if port.range is not None:
                    raw = raw.clamp(port.range[0], port.range[1])
                acc[e.dst_port] = acc[e.dst_port] + raw
            if nd.n_inputs == 0:
                values[nid] = [torch.zeros(x.size(0)) for _ in range(nd.n_outputs)]
                continue
            out = self.surrogates[nd.id](torch.stack(acc, dim=1))
            values[nid] = [out[:, j] for j in range(nd.n_outputs)]
        outs = [v for nid in g.output_node_ids for v in values[nid]]
        return torch.stack(outs, dim=1)

    def train(self, train_inputs: Sequence[Sequence[float]], train_targets: Sequence[Sequence[float]],
              on_epoch: Callable[[int, float], None] | None = None) -> list[float]:
        c = self.config
        torch.manual_seed(c.seed)
        if self.surrogates is None:
            self.surrogates = build_surrogates(self.graph, c.surrogate_samples, c.surrogate_epochs,
                                               c.surrogate_hidden, c.seed)
        edge_ids = sorted(self.graph.edges)
        edge_index = {eid: i for i, eid in enumerate(edge_ids)}
        params = torch.tensor(self.graph.get_edge_params(), dtype=torch.float32, requires_grad=True)
        opt = torch.optim.Adam([params], lr=c.learning_rate)
        x = torch.as_tensor(np.asarray(train_inputs, dtype=np.float32))
        y = torch.as_tensor(np.asarray(train_targets, dtype=np.float32))
        loss_fn = nn.functional.binary_cross_entropy_with_logits if c.loss_fn == "bce" else nn.functional.mse_loss
        for epoch in range(c.epochs):
            if self._stop:
                break
            perm = torch.randperm(x.size(0))
            total, n = 0.0, 0
            for i in range(0, x.size(0), c.batch_size):
                idx = perm[i:i + c.batch_size]
                loss = loss_fn(self._forward(params, x[idx], edge_index), y[idx])
                opt.zero_grad()
                loss.backward()
                opt.step()
                total += float(loss.detach()) * idx.numel()
                n += idx.numel()
            self.loss_history.append(total / max(n, 1))
            if on_epoch is not None:
                on_epoch(epoch, self.loss_history[-1])
        self.graph.set_edge_params([float(v) for v in params.detach()])
        return self.loss_history
