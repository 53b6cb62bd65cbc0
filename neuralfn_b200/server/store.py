"""State behind the platform API and the MCP tool server: graph sessions, training runs,
datasets - an in-memory ``LiveStateStore`` with optional JSON snapshots on disk (the
reference keeps the same state in Redis / SQL, ``server/services`` and ``server/db*.py``).

Every operation the REST routes and the MCP tools expose lives here as a method, so both
front-ends are thin and a test can drive the store directly.
"""
from __future__ import annotations

import copy
import json
import threading
import time
import uuid
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from ..graph import Edge, NeuronGraph, NeuronInstance
from ..serialization import graph_from_json, graph_to_json

__all__ = ["LiveStateStore", "RunRecord"]


@dataclass
class RunRecord:
    id: str
    session_id: str
    kind: str
    status: str = "queued"          # queued | running | finished | failed | stopped
    created: float = field(default_factory=time.time)
    progress: list = field(default_factory=list)   # loss history
    result: dict | None = None
    error: str | None = None
    _stop: threading.Event = field(default_factory=threading.Event, repr=False)

    def public(self) -> dict:
        return {"id": self.id, "session_id": self.session_id, "kind": self.kind, "status": self.status, "created": self.created,
                "steps": len(self.progress), "last_loss": self.progress[-1] if self.progress else None, "result": self.result,
                "error": self.error}


class LiveStateStore:
    def __init__(self, snapshot_dir: str | Path | None = None) -> None:
        self._lock = threading.RLock()
        self.sessions: dict[str, NeuronGraph] = {}
        self.runs: dict[str, RunRecord] = {}
        self.snapshot_dir = Path(snapshot_dir) if snapshot_dir else None
        if self.snapshot_dir and self.snapshot_dir.exists():
            for p in sorted(self.snapshot_dir.glob("session_*.json")):
                self.sessions[p.stem[len("session_"):]] = graph_from_json(p.read_text())

    # ---- sessions / graphs --------------------------------------------------------------------
    def _snapshot(self, sid: str) -> None:
        if self.snapshot_dir:
            self.snapshot_dir.mkdir(parents=True, exist_ok=True)
            final = self.snapshot_dir / f"session_{sid}.json"
            tmp = final.with_suffix(f".tmp{threading.get_ident()}")
            tmp.write_text(graph_to_json(self.sessions[sid]))
            tmp.replace(final)  # readers never see a half-written snapshot

    def create_session(self, name: str = "untitled", graph_json: str | dict | None = None) -> str:
        with self._lock:
            sid = uuid.uuid4().hex[:12]
            if graph_json is None:
                g = NeuronGraph(name=name)
            else:
                g = graph_from_json(graph_json if isinstance(graph_json, str) else json.dumps(graph_json))
            self.sessions[sid] = g
            self._snapshot(sid)
            return sid

    def graph(self, sid: str) -> NeuronGraph:
        try:
            return self.sessions[sid]
        except KeyError:
            raise KeyError(f"unknown session {sid!r}") from None

    def get_graph(self, sid: str) -> dict:
        return self.graph(sid).to_dict()

    def replace_graph(self, sid: str, payload: dict) -> dict:
        with self._lock:
            self.graph(sid)
            self.sessions[sid] = NeuronGraph.from_dict(payload)
            self._snapshot(sid)
            return {"nodes": len(self.sessions[sid].nodes), "edges": len(self.sessions[sid].edges)}

    def list_sessions(self) -> list[dict]:
        return [{"id": sid, "name": g.name, "nodes": len(g.nodes), "edges": len(g.edges), "training_method": g.training_method}
                for sid, g in self.sessions.items()]

    def delete_session(self, sid: str) -> None:
        with self._lock:
            self.graph(sid)
            del self.sessions[sid]
            if self.snapshot_dir:
                (self.snapshot_dir / f"session_{sid}.json").unlink(missing_ok=True)

    def add_builtin_node(self, sid: str, builtin: str, *, role: str | None = None, position=(0.0, 0.0)) -> str:
        from ..builtins import BUILTIN_MAP
        from ..scalar_builtins import SPEC_BY_NAME, make_builtin
        with self._lock:
            g = self.graph(sid)
            # scalar functions win over tensor stages of the same name unless the graph runs on the tensor runtime
            if builtin in SPEC_BY_NAME and g.runtime != "torch":
                nd = make_builtin(builtin)
            elif builtin in BUILTIN_MAP:
                nd = copy.deepcopy(BUILTIN_MAP[builtin])
            else:
                raise KeyError(f"unknown builtin neuron {builtin!r}")
            nid = g.add_node(NeuronInstance(neuron_def=nd, position=tuple(position)))
            if role == "input":
                g.input_node_ids.append(nid)
            elif role == "output":
                g.output_node_ids.append(nid)
            self._snapshot(sid)
            return nid

    def remove_node(self, sid: str, node_id: str) -> None:
        with self._lock:
            if node_id not in self.graph(sid).nodes:
                raise KeyError(f"unknown node {node_id!r}")
            self.graph(sid).remove_node(node_id)
            self._snapshot(sid)

    def add_edge(self, sid: str, src_node: str, dst_node: str, src_port: int = 0, dst_port: int = 0, weight: float = 1.0,
                 bias: float = 0.0) -> str:
        with self._lock:
            eid = self.graph(sid).add_edge(Edge(src_node=src_node, src_port=src_port, dst_node=dst_node, dst_port=dst_port,
                                                weight=weight, bias=bias))
            self._snapshot(sid)
            return eid

    def remove_edge(self, sid: str, edge_id: str) -> None:
        with self._lock:
            self.graph(sid).remove_edge(edge_id)
            self._snapshot(sid)

    # ---- node / edge / settings edits ----------------------------------------------------------
    def get_node(self, sid: str, node_id: str) -> dict:
        g = self.graph(sid)
        if node_id not in g.nodes:
            raise KeyError(f"unknown node {node_id!r}")
        n = g.nodes[node_id]
        return n.to_dict() | {"incoming": [e.id for e in g.edges.values() if e.dst_node == node_id],
                              "outgoing": [e.id for e in g.edges.values() if e.src_node == node_id],
                              "is_input": node_id in g.input_node_ids, "is_output": node_id in g.output_node_ids}

    def update_node(self, sid: str, node_id: str, *, name: str | None = None, position=None, source_code: str | None = None,
                    module_config: dict | None = None) -> dict:
        """Renames / moves a node; for function neurons ``source_code`` replaces the body (graph
        source is executable code by contract, exactly as when a graph file is loaded: expose
        this only to trusted callers), for module nodes ``module_config`` is merged into the
        existing configuration."""
        from ..neuron import neuron_from_source
        with self._lock:
            g = self.graph(sid)
            if node_id not in g.nodes:
                raise KeyError(f"unknown node {node_id!r}")
            n = g.nodes[node_id]
            nd = n.neuron_def
            if source_code is not None:
                if nd.kind != "function":
                    raise ValueError("only function neurons carry source code")
                n.neuron_def = nd = neuron_from_source(source_code, name or nd.name, nd.input_ports, nd.output_ports, neuron_id=nd.id)
            if name is not None:
                nd.name = name
            if module_config is not None:
                if nd.kind != "module":
                    raise ValueError("only module nodes carry a module_config")
                nd.module_config.update(module_config)
            if position is not None:
                n.position = (float(position[0]), float(position[1]))
            g._topo = None
            self._snapshot(sid)
            return self.get_node(sid, node_id)

    def update_node_positions(self, sid: str, positions: dict[str, list[float]]) -> int:
        with self._lock:
            g = self.graph(sid)
            missing = [k for k in positions if k not in g.nodes]
            if missing:
                raise KeyError(f"unknown nodes {missing[:3]}")
            for k, (x, y) in positions.items():
                g.nodes[k].position = (float(x), float(y))
            self._snapshot(sid)
            return len(positions)

    def add_custom_node(self, sid: str, source_code: str, fn_name: str, inputs: list[dict], outputs: list[dict], position=(0.0, 0.0)) -> str:
        from ..neuron import neuron_from_source
        from ..port import Port
        with self._lock:
            nd = neuron_from_source(source_code, fn_name, [Port.from_dict(p) for p in inputs], [Port.from_dict(p) for p in outputs])
            nid = self.graph(sid).add_node(NeuronInstance(neuron_def=nd, position=tuple(position)))
            self._snapshot(sid)
            return nid

    def add_subgraph_node(self, sid: str, name: str, subgraph: dict, position=(0.0, 0.0), variant_ref: dict | None = None) -> str:
        from ..neuron import subgraph_neuron
        with self._lock:
            nd = subgraph_neuron(NeuronGraph.from_dict(subgraph), name=name, variant_ref=variant_ref)
            nid = self.graph(sid).add_node(NeuronInstance(neuron_def=nd, position=tuple(position)))
            self._snapshot(sid)
            return nid

    def update_edge(self, sid: str, edge_id: str, weight: float | None = None, bias: float | None = None) -> dict:
        with self._lock:
            g = self.graph(sid)
            if edge_id not in g.edges:
                raise KeyError(f"unknown edge {edge_id!r}")
            e = g.edges[edge_id]
            if weight is not None:
                e.weight = float(weight)
            if bias is not None:
                e.bias = float(bias)
            self._snapshot(sid)
            return e.to_dict()

    def set_io(self, sid: str, input_ids: list[str], output_ids: list[str]) -> dict:
        with self._lock:
            g = self.graph(sid)
            unknown = [i for i in (*input_ids, *output_ids) if i not in g.nodes]
            if unknown:
                raise KeyError(f"unknown nodes {unknown[:3]}")
            g.input_node_ids, g.output_node_ids = list(input_ids), list(output_ids)
            self._snapshot(sid)
            return {"inputs": g.input_node_ids, "outputs": g.output_node_ids}

    def update_graph_settings(self, sid: str, *, name: str | None = None, training_method: str | None = None, runtime: str | None = None,
                              surrogate_config: dict | None = None, evo_config: dict | None = None, torch_config: dict | None = None) -> dict:
        with self._lock:
            g = self.graph(sid)
            if training_method is not None:
                if training_method not in ("surrogate", "evolutionary", "sgd", "torch", "hybrid"):
                    raise ValueError(f"unknown training method {training_method!r}")
                g.training_method = training_method
            if runtime is not None:
                if runtime not in ("scalar", "torch"):
                    raise ValueError("runtime is 'scalar' or 'torch'")
                g.runtime = runtime
            if name is not None:
                g.name = name
            for attr, val in (("surrogate_config", surrogate_config), ("evo_config", evo_config), ("torch_config", torch_config)):
                if val is not None:
                    getattr(g, attr).update(val)
            self._snapshot(sid)
            return {"name": g.name, "training_method": g.training_method, "runtime": g.runtime, "surrogate_config": g.surrogate_config,
                    "evo_config": g.evo_config, "torch_config": g.torch_config}

    def load_gpt_template(self, sid: str, preset: str = "nanogpt", config: dict | None = None) -> dict:
        """Replaces the session's graph by the tensor graph of a model preset."""
        from ..presets import build_preset
        from ..torch_templates import build_gpt_root_graph
        with self._lock:
            self.graph(sid)
            g = build_gpt_root_graph(build_preset(preset, **(config or {})))
            self.sessions[sid] = g
            self._snapshot(sid)
            return {"nodes": len(g.nodes), "edges": len(g.edges), "runtime": g.runtime}

    # ---- variants ------------------------------------------------------------------------------
    def save_node_as_variant(self, sid: str, node_id: str, family: str, version: str, link_node: bool = True) -> dict:
        with self._lock:
            g = self.graph(sid)
            nd = g.nodes[node_id].neuron_def if node_id in g.nodes else None
            if nd is None or nd.kind != "subgraph" or nd.subgraph is None:
                raise ValueError("only subgraph nodes can be stored as variants")
            g.variant_library.setdefault(family, {})[version] = NeuronGraph.from_dict_raw(nd.subgraph.to_dict())
            if link_node:
                nd.variant_ref = {"family": family, "version": version}
            self._snapshot(sid)
            return self.list_variants(sid)

    def swap_node_variant(self, sid: str, node_id: str, family: str, version: str) -> dict:
        with self._lock:
            g = self.graph(sid)
            nd = g.nodes[node_id].neuron_def if node_id in g.nodes else None
            if nd is None or nd.kind != "subgraph":
                raise ValueError("only subgraph nodes reference variants")
            if version not in g.variant_library.get(family, {}):
                raise KeyError(f"no variant {family}@{version}")
            nd.variant_ref = {"family": family, "version": version}
            g.resolve_variant_library()
            g._topo = None
            self._snapshot(sid)
            return self.get_node(sid, node_id)

    def add_variant_node(self, sid: str, family: str, version: str, position=(0.0, 0.0)) -> str:
        g = self.graph(sid)
        if version not in g.variant_library.get(family, {}):
            raise KeyError(f"no variant {family}@{version}")
        return self.add_subgraph_node(sid, f"{family}@{version}", g.variant_library[family][version].to_dict(), position,
                                      variant_ref={"family": family, "version": version})

    def probe_node(self, sid: str, node_id: str, n_samples: int = 1000, seed: int = 0) -> dict:
        """Samples a scalar neuron over its input ranges: per-output min / max / mean."""
        import random
        g = self.graph(sid)
        if node_id not in g.nodes:
            raise KeyError(f"unknown node {node_id!r}")
        nd = g.nodes[node_id].neuron_def
        if nd.kind == "module":
            raise ValueError("module nodes are probed with trace_torch")
        rng = random.Random(seed)
        lo_hi = [(p.range[0], p.range[1]) if getattr(p, "range", None) else (-1.0, 1.0) for p in nd.input_ports]
        outs = [nd(*[rng.uniform(a, b) for a, b in lo_hi]) for _ in range(max(1, min(int(n_samples), 100000)))]
        cols = list(zip(*outs))
        return {"samples": len(outs), "outputs": [{"name": p.name, "min": min(c), "max": max(c), "mean": sum(c) / len(c)}
                                                  for p, c in zip(nd.output_ports, cols)]}

    def list_variants(self, sid: str) -> dict:
        lib = getattr(self.graph(sid), "variant_library", {}) or {}
        return {family: sorted(versions) for family, versions in lib.items()}

    def execute(self, sid: str, inputs: list[float]) -> list[float]:
        return list(self.graph(sid).execute_flat(tuple(float(v) for v in inputs)))

    def trace(self, sid: str, inputs: dict[str, list[float]]) -> Any:
        return self.graph(sid).execute_trace({k: tuple(v) for k, v in inputs.items()})

    # ---- training runs ------------------------------------------------------------------------
    def train_start(self, sid: str, inputs: list[list[float]], targets: list[list[float]], *, method: str = "sgd", steps: int = 500,
                    learning_rate: float = 0.5) -> str:
        g = self.graph(sid)
        run = RunRecord(uuid.uuid4().hex[:12], sid, method)
        self.runs[run.id] = run

        def work() -> None:
            run.status = "running"
            try:
                if method == "sgd":
                    from ..sgd import GraphSGDTrainer, SGDConfig
                    tr = GraphSGDTrainer(g, SGDConfig(learning_rate=learning_rate, steps=steps))
                    hist = tr.train(inputs, targets, on_step=lambda i, l: run.progress.append(l))
                elif method == "evolutionary":
                    from ..evolutionary import EvoConfig, EvolutionaryTrainer
                    tr = EvolutionaryTrainer(g, EvoConfig(generations=steps, seed=0))
                    hist = tr.train(inputs, targets, on_generation=lambda i, l: (run.progress.append(l), run._stop.is_set() and tr.stop()))
                elif method == "surrogate":
                    from ..surrogate import SurrogateTrainer, TrainConfig
                    tr = SurrogateTrainer(g, TrainConfig(epochs=steps, learning_rate=learning_rate, surrogate_samples=2000, surrogate_epochs=50))
                    hist = tr.train(inputs, targets, on_epoch=lambda i, l: (run.progress.append(l), run._stop.is_set() and tr.stop()))
                else:
                    raise ValueError(f"unknown training method {method!r}")
                run.result = {"final_loss": hist[-1] if hist else None, "steps": len(hist)}
                with self._lock:
                    self._snapshot(sid)
                run.status = "stopped" if run._stop.is_set() else "finished"
            except Exception as exc:  # surfaced through train_status
                run.error, run.status = f"{type(exc).__name__}: {exc}", "failed"

        threading.Thread(target=work, daemon=True, name=f"run-{run.id}").start()
        return run.id

    def train_status(self, run_id: str) -> dict:
        return self.runs[run_id].public()

    def train_stop(self, run_id: str) -> dict:
        self.runs[run_id]._stop.set()
        return self.runs[run_id].public()

    def wait(self, run_id: str, timeout: float = 60.0) -> dict:
        t0 = time.time()
        while self.runs[run_id].status in ("queued", "running") and time.time() - t0 < timeout:
            time.sleep(0.02)
        return self.runs[run_id].public()
