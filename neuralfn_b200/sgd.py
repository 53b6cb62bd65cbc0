"""Exact-gradient SGD over the edge parameters of a scalar DAG graph.

The reference ships surrogate-Adam, genetic and hybrid edge trainers but no plain
gradient trainer (``examples/xor_graph.py:59-101`` uses the former two). This module
adds one: reverse-mode differentiation straight through the scalar executor, using
the analytic Jacobians of the built-in scalar neurons (central differences for
user-defined function neurons and nested subgraphs). Forward values are exactly
those of ``NeuronGraph.execute`` - the same gather/condition/call sequence - so a
trained graph behaves identically when executed or round-tripped through JSON.

Port conditioning in the backward pass: a clamp passes gradient only inside the
range; quantisation is treated as straight-through.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Callable, Sequence

from .graph import Edge, NeuronGraph
from .port import Port
from .scalar_builtins import jacobian_for

__all__ = ["SGDConfig", "GraphSGDTrainer", "init_edge_params_normal"]


@dataclass
class SGDConfig:
    learning_rate: float = 0.5
    steps: int = 2000
    loss_fn: str = "mse"          # "mse" | "bce" (targets in {0,1}, outputs are probabilities)
    batch_mode: str = "full"      # "full": one update per step over all rows; "cyclic": one row per step
    momentum: float = 0.0
    fd_eps: float = 1e-6          # central-difference step for non built-in neurons
    log_every: int = 0
    train_bias: bool = True


def init_edge_params_normal(graph: NeuronGraph, seed: int = 0, *, std: float = 1.0,
                            bias: bool = True) -> None:
    """Draw every edge weight (and bias) from N(0, std) with ``random.Random(seed)``,
    visiting edges in sorted-id order (the order of ``get_edge_params``)."""
    rng = random.Random(seed)
    for eid in sorted(graph.edges):
        e = graph.edges[eid]
        e.weight = rng.gauss(0.0, std)
        e.bias = rng.gauss(0.0, std) if bias else 0.0


def _cond_grad(port: Port, raw: float) -> float:
    if port.range is not None:
        lo, hi = port.range
        if raw < lo or raw > hi:
            return 0.0
    return 1.0


def _numeric_jacobian(fn: Callable[..., Sequence[float]], args: Sequence[float], n_out: int,
                      eps: float) -> list[list[float]]:
    jac = [[0.0] * len(args) for _ in range(n_out)]
    for j in range(len(args)):
        hi = list(args)
        lo = list(args)
        hi[j] += eps
        lo[j] -= eps
        yh, yl = fn(*hi), fn(*lo)
        if not isinstance(yh, (tuple, list)):
            yh, yl = (yh,), (yl,)
        for i in range(n_out):
            jac[i][j] = (float(yh[i]) - float(yl[i])) / (2 * eps)
    return jac


@dataclass
class _Tape:
    values: dict[str, tuple[float, ...]] = field(default_factory=dict)
    node_inputs: dict[str, tuple[float, ...]] = field(default_factory=dict)
    raw_outputs: dict[str, tuple[float, ...]] = field(default_factory=dict)
    edge_raw: dict[str, float] = field(default_factory=dict)


class GraphSGDTrainer:
    """Gradient descent on ``[w, b]`` of every edge of an acyclic scalar graph."""

    def __init__(self, graph: NeuronGraph, config: SGDConfig | None = None) -> None:
        if graph.has_module_nodes() or graph.runtime == "torch":
            raise TypeError("GraphSGDTrainer works on scalar graphs; use TorchTrainer for module graphs")
        if graph.has_cycles():
            raise ValueError("GraphSGDTrainer needs an acyclic graph")
        self.graph = graph
        self.config = config or SGDConfig()
        self.loss_history: list[float] = []
        self._order = graph.topological_order()
        self._edge_ids = sorted(graph.edges)
        self._velocity = [0.0] * (2 * len(self._edge_ids))
        self._jac: dict[str, Callable | None] = {
            nid: jacobian_for(node.neuron_def) for nid, node in graph.nodes.items()}

    # -- forward with tape -------------------------------------------------------------
    def _forward(self, feeds: dict[str, tuple[float, ...]]) -> _Tape:
        g = self.graph
        tape = _Tape(values=dict(feeds))
        for nid in self._order:
            if nid in feeds:
                continue
            node = g.nodes[nid]
            ports = node.neuron_def.input_ports
            acc = [0.0] * len(ports)
            for e in g._incoming(nid):
                src = tape.values.get(e.src_node, ())
                if e.src_port < len(src):
                    raw = src[e.src_port] * e.weight + e.bias
                    tape.edge_raw[e.id] = raw
                    acc[e.dst_port] += ports[e.dst_port].condition(raw)
            args = tuple(acc)
            tape.node_inputs[nid] = args
            raw_out = node.neuron_def.raw_call(*args)
            if not isinstance(raw_out, (tuple, list)):
                raw_out = (raw_out,)
            raw_out = tuple(float(v) for v in raw_out)
            tape.raw_outputs[nid] = raw_out
            tape.values[nid] = tuple(p.condition(v) for v, p in zip(raw_out, node.neuron_def.output_ports))
        return tape

    # -- backward ------------------------------------------------------------------------
    def _backward(self, tape: _Tape, feeds, out_grads: dict[str, list[float]]) -> dict[str, tuple[float, float]]:
        g = self.graph
        dvals: dict[str, list[float]] = {nid: list(gr) for nid, gr in out_grads.items()}
        edge_grads: dict[str, tuple[float, float]] = {}
        for nid in reversed(self._order):
            if nid in feeds or nid not in dvals:
                continue
            node = g.nodes[nid]
            nd = node.neuron_def
            dy = dvals[nid]
            raw_out = tape.raw_outputs[nid]
            dy = [d * _cond_grad(p, r) for d, p, r in zip(dy, nd.output_ports, raw_out)]
            if not any(dy):
                continue
            args = tape.node_inputs[nid]
            jac_fn = self._jac.get(nid)
            if jac_fn is not None:
                jac = jac_fn(*args)
            else:
                jac = _numeric_jacobian(nd.raw_call, args, len(raw_out), self.config.fd_eps)
            din = [sum(dy[i] * jac[i][j] for i in range(len(dy))) for j in range(len(args))]
            for e in g._incoming(nid):
                raw = tape.edge_raw.get(e.id)
                if raw is None:
                    continue
                ge = din[e.dst_port] * _cond_grad(nd.input_ports[e.dst_port], raw)
                if ge == 0.0:
                    edge_grads.setdefault(e.id, (0.0, 0.0))
                    continue
                src_val = tape.values[e.src_node][e.src_port]
                pw, pb = edge_grads.get(e.id, (0.0, 0.0))
                edge_grads[e.id] = (pw + ge * src_val, pb + ge)
                if e.src_node not in feeds:
                    slot = dvals.setdefault(e.src_node, [0.0] * len(tape.values[e.src_node]))
                    slot[e.src_port] += ge * e.weight
        return edge_grads

    # -- loss ----------------------------------------------------------------------------
    def _loss_and_grad(self, rows_x, rows_y) -> tuple[float, list[float]]:
        g = self.graph
        in_ids, out_ids = g.input_node_ids, g.output_node_ids
        grad = [0.0] * (2 * len(self._edge_ids))
        index = {eid: i for i, eid in enumerate(self._edge_ids)}
        total = 0.0
        count = 0
        for x, y in zip(rows_x, rows_y):
            feeds, cur = {}, 0
            for nid in in_ids:
                w = g.nodes[nid].neuron_def.n_outputs
                feeds[nid] = tuple(float(v) for v in x[cur:cur + w])
                cur += w
            tape = self._forward(feeds)
            out_grads: dict[str, list[float]] = {}
            cur = 0
            for nid in out_ids:
                vals = tape.values.get(nid, ())
                gl = []
                for v in vals:
                    t = float(y[cur])
                    cur += 1
                    if self.config.loss_fn == "bce":
                        p = min(max(v, 1e-12), 1 - 1e-12)
                        import math
                        total += -(t * math.log(p) + (1 - t) * math.log(1 - p))
                        gl.append((p - t) / (p * (1 - p)))
                    else:
                        total += (v - t) ** 2
                        gl.append(2.0 * (v - t))
                    count += 1
                out_grads[nid] = gl
            for eid, (gw, gb) in self._backward(tape, feeds, out_grads).items():
                i = index[eid]
                grad[2 * i] += gw
                grad[2 * i + 1] += gb
        scale = 1.0 / max(count, 1)
        return total * scale, [v * scale for v in grad]

    def loss(self, rows_x, rows_y) -> float:
        return self._loss_and_grad(rows_x, rows_y)[0]

    def gradient(self, rows_x, rows_y) -> list[float]:
        """d(mean loss)/d(params), in ``get_edge_params`` order."""
        return self._loss_and_grad(rows_x, rows_y)[1]

    # -- training ---------------------------------------------------------------------------
    def train(self, rows_x, rows_y, on_step: Callable[[int, float], None] | None = None) -> list[float]:
        cfg = self.config
        g = self.graph
        n_rows = len(rows_x)
        for step in range(cfg.steps):
            if cfg.batch_mode == "cyclic":
                sel = [step % n_rows]
                bx, by = [rows_x[i] for i in sel], [rows_y[i] for i in sel]
            else:
                bx, by = rows_x, rows_y
            loss, grad = self._loss_and_grad(bx, by)
            params = g.get_edge_params()
            for i in range(len(params)):
                if not cfg.train_bias and i % 2 == 1:
                    continue
                self._velocity[i] = cfg.momentum * self._velocity[i] + grad[i]
                params[i] -= cfg.learning_rate * self._velocity[i]
            g.set_edge_params(params)
            self.loss_history.append(loss)
            if on_step is not None:
                on_step(step, loss)
        self.loss_history.append(self.loss(rows_x, rows_y))
        return self.loss_history
