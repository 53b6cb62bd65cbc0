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
