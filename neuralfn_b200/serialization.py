"""Graph JSON files. ``save_graph`` writes ``json.dumps(graph.to_dict(), indent=2)``;
floats go through Python's shortest-repr encoder, so fp64 edge parameters
round-trip bit-exactly (reference: ``neuralfn/serialization.py:27-42``)."""
from __future__ import annotations

import copy
import json
from pathlib import Path
from typing import Any

from .graph import NeuronGraph

__all__ = ["save_graph", "load_graph", "graph_to_json", "graph_from_json"]


def _strip_module_state(payload: dict[str, Any]) -> dict[str, Any]:
    """Copy of a graph payload with every ``module_state`` blob emptied (recursively)."""
    out = copy.deepcopy(payload)

    def walk(g: dict[str, Any]) -> None:
        for node in g.get("nodes", {}).values():
            nd = node.get("neuron_def", {})
            if nd.get("module_state"):
                nd["module_state"] = ""
            if nd.get("subgraph"):
                walk(nd["subgraph"])
        for versions in g.get("variant_library", {}).values():
            for sub in versions.values():
                walk(sub)

    walk(out)
    return out


def graph_to_json(graph: NeuronGraph, *, include_module_state: bool = True) -> str:
    payload = graph.to_dict()
    if not include_module_state:
        payload = _strip_module_state(payload)
    return json.dumps(payload, indent=2)


def graph_from_json(text: str) -> NeuronGraph:
    return NeuronGraph.from_dict(json.loads(text))


def save_graph(graph: NeuronGraph, path: str | Path, *, include_module_state: bool = True) -> None:
    Path(path).write_text(graph_to_json(graph, include_module_state=include_module_state))


def load_graph(path: str | Path) -> NeuronGraph:
    return graph_from_json(Path(path).read_text())
