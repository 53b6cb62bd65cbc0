"""Scalar graph runtime: instances, weighted edges, DAG and cyclic execution.

Semantics follow the reference's ``neuralfn/graph.py`` (``Edge.transform`` at :63,
input gathering at :548-563, DAG walk at :472-488, damped settling at :508-546,
variant resolution at :325-411) so graph JSON and numeric results interchange,
but the executor here is index-based: adjacency, topological order and the
per-node incoming-edge lists are computed once per topology revision and reused
across ``execute`` calls (the gradient trainer calls it thousands of times).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterable, Optional

from .neuron import NeuronDef, new_id
from .port import Port

__all__ = ["NeuronInstance", "Edge", "NeuronGraph", "VARIANT_FAMILY_ALIASES"]

# A variant reference to one family may be satisfied by an entry stored under an
# allied family name (older graphs stored blocks under "transformer_block").
VARIANT_FAMILY_ALIASES: dict[str, tuple[str, ...]] = {
    "gpt2": ("transformer_block",),
    "nanogpt": ("transformer_block",),
    "llama": ("transformer_block",),
    "attn_block": ("transformer_block",),
    "transformer_block": ("attn_block",),
    "mixllama": ("attn_block",),
}


@dataclass
class NeuronInstance:
    neuron_def: NeuronDef
    instance_id: str = field(default_factory=new_id)
    position: tuple[float, float] = (0.0, 0.0)

    @property
    def name(self) -> str:
        return self.neuron_def.name

    def to_dict(self) -> dict[str, Any]:
        return {"instance_id": self.instance_id, "neuron_def": self.neuron_def.to_dict(),
                "position": list(self.position)}

    @classmethod
    def from_dict(cls, payload: dict[str, Any]) -> "NeuronInstance":
        return cls(neuron_def=NeuronDef.from_dict(payload["neuron_def"]),
                   instance_id=payload["instance_id"],
                   position=tuple(payload.get("position", [0, 0])))


@dataclass
class Edge:
    id: str = field(default_factory=new_id)
    src_node: str = ""
    src_port: int = 0
    dst_node: str = ""
    dst_port: int = 0
    weight: float = 1.0
    bias: float = 0.0

    def transform(self, value: float) -> float:
        return value * self.weight + self.bias

    def to_dict(self) -> dict[str, Any]:
        return {"id": self.id, "src_node": self.src_node, "src_port": self.src_port,
                "dst_node": self.dst_node, "dst_port": self.dst_port,
                "weight": self.weight, "bias": self.bias}

    @classmethod
    def from_dict(cls, payload: dict[str, Any]) -> "Edge":
        return cls(id=payload["id"], src_node=payload["src_node"], src_port=payload["src_port"],
                   dst_node=payload["dst_node"], dst_port=payload["dst_port"],
                   weight=payload.get("weight", 1.0), bias=payload.get("bias", 0.0))


class _Topology:
    """Derived structure of a graph: incoming edges per node and a topological order."""

    __slots__ = ("incoming", "order", "cyclic", "stamp")

    def __init__(self, graph: "NeuronGraph") -> None:
        self.stamp = graph._topology_stamp()
        self.incoming: dict[str, list[Edge]] = {nid: [] for nid in graph.nodes}
        succ: dict[str, list[str]] = {nid: [] for nid in graph.nodes}
        indeg: dict[str, int] = {nid: 0 for nid in graph.nodes}
        seen_pairs: set[tuple[str, str]] = set()
        for e in graph.edges.values():
            if e.dst_node in self.incoming:
                self.incoming[e.dst_node].append(e)
            if e.src_node in succ and e.dst_node in indeg and (e.src_node, e.dst_node) not in seen_pairs:
                seen_pairs.add((e.src_node, e.dst_node))
                succ[e.src_node].append(e.dst_node)
                indeg[e.dst_node] += 1
        ready = [nid for nid in graph.nodes if indeg[nid] == 0]
        order: list[str] = []
        head = 0
        while head < len(ready):
            nid = ready[head]
            head += 1
            order.append(nid)
            for nxt in succ[nid]:
                indeg[nxt] -= 1
                if indeg[nxt] == 0:
                    ready.append(nxt)
        self.cyclic = len(order) != len(graph.nodes)
        self.order = order


class NeuronGraph:
    """Directed graph of neuron instances joined by weighted, biased edges."""

    def __init__(self, *, name: str = "graph", training_method: str = "surrogate",
                 runtime: str = "scalar", surrogate_config: dict[str, Any] | None = None,
                 evo_config: dict[str, Any] | None = None,
                 torch_config: dict[str, Any] | None = None,
                 variant_library: dict[str, dict[str, "NeuronGraph"]] | None = None) -> None:
        self.name = name
        self.training_method = training_method
        self.runtime = runtime
        self.surrogate_config = dict(surrogate_config or {})
        self.evo_config = dict(evo_config or {})
        self.torch_config = dict(torch_config or {})
        self.variant_library: dict[str, dict[str, NeuronGraph]] = {
            fam: dict(vers) for fam, vers in dict(variant_library or {}).items()}
        self.nodes: dict[str, NeuronInstance] = {}
        self.edges: dict[str, Edge] = {}
        self.input_node_ids: list[str] = []
        self.output_node_ids: list[str] = []
        self._topo: Optional[_Topology] = None

    # ---- mutation --------------------------------------------------------------
    def add_node(self, instance: NeuronInstance) -> str:
        self.nodes[instance.instance_id] = instance
        self._topo = None
        return instance.instance_id

    def remove_node(self, node_id: str) -> None:
        self.nodes.pop(node_id, None)
        for eid in [eid for eid, e in self.edges.items() if node_id in (e.src_node, e.dst_node)]:
            del self.edges[eid]
        self.input_node_ids = [n for n in self.input_node_ids if n != node_id]
        self.output_node_ids = [n for n in self.output_node_ids if n != node_id]
        self._topo = None

    def add_edge(self, edge: Edge) -> str:
        if edge.src_node not in self.nodes or edge.dst_node not in self.nodes:
            raise ValueError("Both src and dst nodes must exist in the graph")
        self.edges[edge.id] = edge
        self._topo = None
        return edge.id

    def remove_edge(self, edge_id: str) -> None:
        self.edges.pop(edge_id, None)
        self._topo = None

    # ---- topology ----------------------------------------------------------------
    def _topology_stamp(self) -> tuple:
        return (len(self.nodes), len(self.edges),
                hash(tuple(self.nodes)), hash(tuple((e.id, e.src_node, e.dst_node) for e in self.edges.values())))

    def _topology(self) -> _Topology:
        topo = self._topo
        if topo is None or topo.stamp != self._topology_stamp():
            topo = self._topo = _Topology(self)
        return topo

    def has_cycles(self) -> bool:
        return self._topology().cyclic

    def topological_order(self) -> list[str]:
        topo = self._topology()
        if topo.cyclic:
            raise ValueError(f"Graph '{self.name}' contains a cycle; no topological order exists")
        return list(topo.order)

    def _incoming(self, node_id: str) -> list[Edge]:
        return self._topology().incoming.get(node_id, [])

    # ---- interface ports -----------------------------------------------------------
    def _interface_layout(self, ids: Iterable[str], what: str) -> list[tuple[str, int, Port]]:
        layout = []
        for nid in ids:
            node = self.nodes.get(nid)
            if node is None:
                raise ValueError(f"Graph '{self.name}' is missing {what} node '{nid}'")
            layout.extend((nid, i, p) for i, p in enumerate(node.neuron_def.output_ports))
        return layout

    def interface_input_layout(self) -> list[tuple[str, int, Port]]:
        return self._interface_layout(self.input_node_ids, "input")

    def interface_output_layout(self) -> list[tuple[str, int, Port]]:
        return self._interface_layout(self.output_node_ids, "output")

    def _aliased_ports(self, layout, aliases, direction: str) -> list[Port]:
        if aliases is not None and len(aliases) != len(layout):
            raise ValueError(f"Graph '{self.name}' has {len(layout)} {direction} ports but "
                             f"received {len(aliases)} aliases")
        names = aliases or [f"{nid}.{port.name}" for nid, _i, port in layout]
        return [Port(name=alias, range=port.range, precision=port.precision, dtype=port.dtype)
                for alias, (_nid, _i, port) in zip(names, layout)]

    def flattened_input_ports(self, aliases: list[str] | None = None) -> list[Port]:
        return self._aliased_ports(self.interface_input_layout(), aliases, "input")

    def flattened_output_ports(self, aliases: list[str] | None = None) -> list[Port]:
        return self._aliased_ports(self.interface_output_layout(), aliases, "output")

    def execute_flat(self, flat_inputs: tuple[float, ...]) -> tuple[float, ...]:
        feeds: dict[str, tuple[float, ...]] = {}
        cursor = 0
        for nid in self.input_node_ids:
            node = self.nodes.get(nid)
            if node is None:
                raise ValueError(f"Graph '{self.name}' is missing input node '{nid}'")
            width = node.neuron_def.n_outputs
            chunk = flat_inputs[cursor:cursor + width]
            if len(chunk) != width:
                raise ValueError(f"Graph '{self.name}' expected {len(self.interface_input_layout())} "
                                 f"flattened inputs but received {len(flat_inputs)}")
            feeds[nid] = tuple(float(v) for v in chunk)
            cursor += width
        if cursor != len(flat_inputs):
            raise ValueError(f"Graph '{self.name}' expected {cursor} flattened inputs but received "
                             f"{len(flat_inputs)}")
        result = self.execute(feeds)
        flat: list[float] = []
        for nid in self.output_node_ids:
            flat.extend(float(v) for v in result.get(nid, ()))
        return tuple(flat)

    # ---- structure queries ------------------------------------------------------------
    def _subgraph_defs(self):
        for node in self.nodes.values():
            nd = node.neuron_def
            if nd.kind == "subgraph" and nd.subgraph is not None:
                yield node.instance_id, nd

    def has_nested_subgraphs(self) -> bool:
        return any(True for _ in self._subgraph_defs())

    def has_module_nodes(self) -> bool:
        if any(n.neuron_def.kind == "module" for n in self.nodes.values()):
            return True
        return any(nd.subgraph.has_module_nodes() for _nid, nd in self._subgraph_defs())

    def has_recursive_subgraphs(self) -> bool:
        return self.has_nested_subgraphs()

    def validate(self, *, as_subgraph: bool = False, seen: set[int] | None = None) -> None:
        if as_subgraph:
            if not self.input_node_ids:
                raise ValueError(f"Subgraph '{self.name}' must declare input_node_ids")
            if not self.output_node_ids:
                raise ValueError(f"Subgraph '{self.name}' must declare output_node_ids")
        for kind, ids in (("input", self.input_node_ids), ("output", self.output_node_ids)):
            for nid in ids:
                if nid not in self.nodes:
                    raise ValueError(f"Graph '{self.name}' references missing {kind} node '{nid}'")
        trail = set(seen or ())
        if id(self) in trail:
            raise ValueError(f"Recursive subgraph reference detected in graph '{self.name}'")
        trail.add(id(self))
        for nid, nd in self._subgraph_defs():
            child = nd.subgraph
            child.validate(as_subgraph=True, seen=trail)
            if nd.input_aliases and len(nd.input_aliases) != len(child.interface_input_layout()):
                raise ValueError(f"Subgraph node '{nid}' input aliases do not match nested graph "
                                 f"'{child.name}'")
            if nd.output_aliases and len(nd.output_aliases) != len(child.interface_output_layout()):
                raise ValueError(f"Subgraph node '{nid}' output aliases do not match nested graph "
                                 f"'{child.name}'")
            nd.refresh_interface_ports()

    # ---- variant library ------------------------------------------------------------------
    def resolve_variant_library(self) -> None:
        """Bind every ``variant_ref`` subgraph node to a private copy of the named
        library entry. When the entry's interface does not match the node's
        declared ports, the node keeps its inline subgraph (fallback)."""
        done: dict[tuple[str, str], NeuronGraph] = {}
        in_progress: list[tuple[str, str]] = []

        def copy_of(g: NeuronGraph) -> NeuronGraph:
            return NeuronGraph.from_dict_raw(g.to_dict())

        def lookup(family: str, version: str) -> NeuronGraph:
            key = (family, version)
            if key in done:
                return done[key]
            if key in in_progress:
                chain = " -> ".join(f"{f}@{v}" for f, v in [*in_progress, key])
                raise ValueError(f"Recursive variant reference detected: {chain}")
            source = None
            for fam in (family, *VARIANT_FAMILY_ALIASES.get(family, ())):
                versions = self.variant_library.get(fam)
                if versions is not None and version in versions:
                    source = versions[version]
                    break
            if source is None:
                raise ValueError(f"Missing variant '{family}@{version}' in graph '{self.name}'")
            in_progress.append(key)
            g = copy_of(source)
            bind(g)
            g.validate(as_subgraph=True)
            in_progress.pop()
            done[key] = g
            return g

        def same_ports(have: list[Port], want: list[Port]) -> bool:
            if len(have) != len(want):
                return False
            for a, b in zip(have, want):
                ra = None if a.range is None else tuple(a.range)
                rb = None if b.range is None else tuple(b.range)
                if a.name != b.name or ra != rb or a.precision != b.precision or a.dtype != b.dtype:
                    return False
            return True

        def keep_inline(nd: NeuronDef) -> None:
            if nd.subgraph is not None:
                bind(nd.subgraph)
                nd.refresh_interface_ports()

        def bind(g: NeuronGraph) -> None:
            for node in g.nodes.values():
                nd = node.neuron_def
                if nd.kind != "subgraph":
                    continue
                ref = nd.variant_ref or {}
                if not ref:
                    keep_inline(nd)
                    continue
                family = str(ref.get("family", "")).strip()
                version = str(ref.get("version", "")).strip()
                if not family or not version:
                    raise ValueError(f"Subgraph node '{nd.name}' has an incomplete variant_ref")
                candidate = copy_of(lookup(family, version))
                try:
                    want_in = candidate.flattened_input_ports(nd.input_aliases or None)
                    want_out = candidate.flattened_output_ports(nd.output_aliases or None)
                except ValueError:
                    keep_inline(nd)
                    continue
                ok_in = not nd.input_ports or same_ports(nd.input_ports, want_in)
                ok_out = not nd.output_ports or same_ports(nd.output_ports, want_out)
                if ok_in and ok_out:
                    nd.subgraph = candidate
                    nd.refresh_interface_ports()
                else:
                    keep_inline(nd)

        for family, versions in list(self.variant_library.items()):
            self.variant_library[family] = {ver: lookup(family, ver) for ver in versions}
        bind(self)

    # ---- execution ------------------------------------------------------------------------
    def _require_scalar(self, verb: str) -> None:
        if self.runtime == "torch" or self.has_module_nodes():
            raise TypeError(f"Graph '{self.name}' uses torch module nodes and cannot be {verb} "
                            "through the scalar runtime")

    def execute(self, inputs: dict[str, tuple[float, ...]], *, max_iters: int = 50,
                damping: float = 0.5, tolerance: float = 1e-6) -> dict[str, tuple[float, ...]]:
        """Evaluate the graph. ``inputs`` maps input-node id -> values; the result
        maps output-node id -> values. Cyclic graphs settle by damped iteration."""
        self._require_scalar("executed")
        if self.has_cycles():
            values = self._settle(inputs, max_iters, damping, tolerance)
        else:
            values = self._forward(inputs)
        return {nid: values.get(nid, ()) for nid in self.output_node_ids}

    def execute_trace(self, inputs: dict[str, tuple[float, ...]], *, max_iters: int = 50,
                      damping: float = 0.5, tolerance: float = 1e-6) -> dict[str, tuple[float, ...]]:
        """Evaluate and return the activation of every node (DAG walk)."""
        self._require_scalar("traced")
        if self.has_cycles():
            return self._settle(inputs, max_iters, damping, tolerance)
        return self._forward(inputs)

    def _gather_inputs(self, nid: str, values: dict[str, tuple[float, ...]],
                       node: NeuronInstance) -> tuple[float, ...]:
        ports = node.neuron_def.input_ports
        acc = [0.0] * len(ports)
        for e in self._incoming(nid):
            src = values.get(e.src_node, ())
            if e.src_port < len(src):
                acc[e.dst_port] += ports[e.dst_port].condition(src[e.src_port] * e.weight + e.bias)
        return tuple(acc)

    def _forward(self, inputs: dict[str, tuple[float, ...]]) -> dict[str, tuple[float, ...]]:
        values: dict[str, tuple[float, ...]] = dict(inputs)
        for nid in self._topology().order:
            if nid in inputs:
                continue
            node = self.nodes[nid]
            values[nid] = node.neuron_def(*self._gather_inputs(nid, values, node))
        return values

    def _settle(self, inputs, max_iters: int, damping: float, tolerance: float):
        values: dict[str, tuple[float, ...]] = {}
        for nid, node in self.nodes.items():
            values[nid] = inputs[nid] if nid in inputs else (0.0,) * node.neuron_def.n_outputs
        keep = 1 - damping
        for _ in range(max_iters):
            nxt: dict[str, tuple[float, ...]] = {}
            worst = 0.0
            for nid, node in self.nodes.items():
                if nid in inputs:
                    nxt[nid] = inputs[nid]
                    continue
                fresh = node.neuron_def(*self._gather_inputs(nid, values, node))
                prev = values[nid]
                nxt[nid] = tuple(damping * f + keep * p for f, p in zip(fresh, prev))
                worst = max(worst, max(abs(f - p) for f, p in zip(fresh, prev)))
            values = nxt
            if worst < tolerance:
                break
        return values

    # ---- edge parameters (sorted by edge id, [w, b] interleaved) ---------------------------------
    def get_edge_params(self) -> list[float]:
        flat: list[float] = []
        for eid in sorted(self.edges):
            e = self.edges[eid]
            flat += [e.weight, e.bias]
        return flat

    def set_edge_params(self, params) -> None:
        for i, eid in enumerate(sorted(self.edges)):
            e = self.edges[eid]
            e.weight = params[2 * i]
            e.bias = params[2 * i + 1]

    def param_count(self) -> int:
        return 2 * len(self.edges)

    # ---- JSON ----------------------------------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        return {
            "name": self.name,
            "training_method": self.training_method,
            "runtime": self.runtime,
            "surrogate_config": self.surrogate_config,
            "evo_config": self.evo_config,
            "torch_config": self.torch_config,
            "variant_library": {fam: {ver: g.to_dict() for ver, g in vers.items()}
                                for fam, vers in self.variant_library.items()},
            "nodes": {nid: n.to_dict() for nid, n in self.nodes.items()},
            "edges": {eid: e.to_dict() for eid, e in self.edges.items()},
            "input_node_ids": self.input_node_ids,
            "output_node_ids": self.output_node_ids,
        }

    @classmethod
    def from_dict(cls, payload: dict[str, Any]) -> "NeuronGraph":
        g = cls.from_dict_raw(payload)
        g.resolve_variant_library()
        g.validate()
        return g

    @classmethod
    def from_dict_raw(cls, payload: dict[str, Any] | None) -> "NeuronGraph":
        if payload is None:
            raise ValueError("Cannot deserialize an empty graph payload")
        g = cls(name=payload.get("name", "graph"),
                training_method=payload.get("training_method", "surrogate"),
                runtime=payload.get("runtime", "scalar"),
                surrogate_config=payload.get("surrogate_config", {}),
                evo_config=payload.get("evo_config", {}),
                torch_config=payload.get("torch_config", {}))
        for fam, vers in payload.get("variant_library", {}).items():
            g.variant_library[fam] = {ver: cls.from_dict_raw(p) for ver, p in vers.items()}
        for nid, nd in payload.get("nodes", {}).items():
            g.nodes[nid] = NeuronInstance(neuron_def=NeuronDef.from_dict_raw(nd["neuron_def"]),
                                          instance_id=nd["instance_id"],
                                          position=tuple(nd.get("position", [0, 0])))
        for eid, ed in payload.get("edges", {}).items():
            g.edges[eid] = Edge.from_dict(ed)
        g.input_node_ids = list(payload.get("input_node_ids", []))
        g.output_node_ids = list(payload.get("output_node_ids", []))
        return g
