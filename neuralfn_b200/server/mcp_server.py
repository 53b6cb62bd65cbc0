"""Model Context Protocol tool server (JSON-RPC 2.0 over stdio): lets an agent inspect and edit
graphs, run and train them, look at datasets, presets, the semantic layer and the native
kernels. ``python -m neuralfn_b200.server.mcp_server`` speaks ``initialize``, ``tools/list``
and ``tools/call``; ``McpToolServer.call(name, args)`` is the same thing in-process.
Counterpart of the reference's ``server/mcp_server.py`` (its tools go through the REST API;
these call the shared store directly).
"""
from __future__ import annotations

import json
import sys
from typing import Any, Callable

from .store import LiveStateStore

__all__ = ["McpToolServer", "main"]


def _tool(desc: str, **props):
    required = [k for k, v in props.items() if not v.pop("optional", False)]
    return {"description": desc, "inputSchema": {"type": "object", "properties": props, "required": required}}


_S, _N, _I, _A, _O, _B = ({"type": t} for t in ("string", "number", "integer", "array", "object", "boolean"))


def _opt(schema: dict) -> dict:
    return {**schema, "optional": True}


class McpToolServer:
    def __init__(self, store: LiveStateStore | None = None) -> None:
        self.store = store or LiveStateStore()
        s = self.store
        self.tools: dict[str, tuple[dict, Callable[..., Any]]] = {
            "list_sessions": (_tool("List graph sessions."), lambda: s.list_sessions()),
            "create_session": (_tool("Create a session, optionally from graph JSON.", name=_opt(dict(_S)), graph=_opt(dict(_O))),
                               lambda name="untitled", graph=None: {"session_id": s.create_session(name, graph)}),
            "delete_session": (_tool("Delete a session.", session_id=dict(_S)), lambda session_id: s.delete_session(session_id)),
            "get_graph": (_tool("Return a session's graph as JSON.", session_id=dict(_S)), lambda session_id: s.get_graph(session_id)),
            "replace_graph": (_tool("Replace a session's graph.", session_id=dict(_S), graph=dict(_O)),
                              lambda session_id, graph: s.replace_graph(session_id, graph)),
            "list_builtin_neurons": (_tool("Names of the built-in neurons."), self._builtins),
            "add_node": (_tool("Add a built-in neuron node.", session_id=dict(_S), builtin=dict(_S), role=_opt(dict(_S))),
                         lambda session_id, builtin, role=None: {"node_id": s.add_builtin_node(session_id, builtin, role=role)}),
            "remove_node": (_tool("Remove a node and its edges.", session_id=dict(_S), node_id=dict(_S)),
                            lambda session_id, node_id: s.remove_node(session_id, node_id)),
            "add_edge": (_tool("Connect two node ports.", session_id=dict(_S), src_node=dict(_S), dst_node=dict(_S), src_port=_opt(dict(_I)),
                               dst_port=_opt(dict(_I)), weight=_opt(dict(_N)), bias=_opt(dict(_N))),
                         lambda session_id, src_node, dst_node, src_port=0, dst_port=0, weight=1.0, bias=0.0:
                         {"edge_id": s.add_edge(session_id, src_node, dst_node, src_port, dst_port, weight, bias)}),
            "remove_edge": (_tool("Remove an edge.", session_id=dict(_S), edge_id=dict(_S)),
                            lambda session_id, edge_id: s.remove_edge(session_id, edge_id)),
            "list_variants": (_tool("Variant library of a session's graph.", session_id=dict(_S)), lambda session_id: s.list_variants(session_id)),
            "get_node": (_tool("One node with its edges and roles.", session_id=dict(_S), node_id=dict(_S)), lambda session_id, node_id: s.get_node(session_id, node_id)),
            "update_node": (_tool("Rename / move a node, replace a function neuron's source, merge a module config.", session_id=dict(_S), node_id=dict(_S),
                                  name=_opt(dict(_S)), position=_opt(dict(_A)), source_code=_opt(dict(_S)), module_config=_opt(dict(_O))),
                            lambda session_id, node_id, **kw: s.update_node(session_id, node_id, **kw)),
            "update_node_positions": (_tool("Move several nodes.", session_id=dict(_S), positions=dict(_O)),
                                      lambda session_id, positions: {"moved": s.update_node_positions(session_id, positions)}),
            "add_custom_node": (_tool("Add a function neuron from Python source.", session_id=dict(_S), source_code=dict(_S), fn_name=dict(_S),
                                      inputs=dict(_A), outputs=dict(_A)),
                                lambda session_id, source_code, fn_name, inputs, outputs:
                                {"node_id": s.add_custom_node(session_id, source_code, fn_name, inputs, outputs)}),
            "add_subgraph_node": (_tool("Add a node that wraps a nested graph.", session_id=dict(_S), name=dict(_S), subgraph=dict(_O)),
                                  lambda session_id, name, subgraph: {"node_id": s.add_subgraph_node(session_id, name, subgraph)}),
            "add_variant_node": (_tool("Add a subgraph node bound to a library variant.", session_id=dict(_S), family=dict(_S), version=dict(_S)),
                                 lambda session_id, family, version: {"node_id": s.add_variant_node(session_id, family, version)}),
            "save_node_as_variant": (_tool("Store a subgraph node in the variant library.", session_id=dict(_S), node_id=dict(_S), family=dict(_S),
                                           version=dict(_S), link_node=_opt(dict(_B))),
                                     lambda session_id, node_id, family, version, link_node=True:
                                     s.save_node_as_variant(session_id, node_id, family, version, link_node)),
            "swap_node_variant": (_tool("Point a subgraph node at another library variant.", session_id=dict(_S), node_id=dict(_S), family=dict(_S),
                                        version=dict(_S)),
                                  lambda session_id, node_id, family, version: s.swap_node_variant(session_id, node_id, family, version)),
            "update_edge": (_tool("Set an edge's weight and / or bias.", session_id=dict(_S), edge_id=dict(_S), weight=_opt(dict(_N)), bias=_opt(dict(_N))),
                            lambda session_id, edge_id, weight=None, bias=None: s.update_edge(session_id, edge_id, weight, bias)),
            "set_io": (_tool("Declare the graph's input and output nodes.", session_id=dict(_S), input_ids=dict(_A), output_ids=dict(_A)),
                       lambda session_id, input_ids, output_ids: s.set_io(session_id, input_ids, output_ids)),
            "update_graph_settings": (_tool("Name, training method, runtime and trainer configs of a graph.", session_id=dict(_S), name=_opt(dict(_S)),
                                            training_method=_opt(dict(_S)), runtime=_opt(dict(_S)), surrogate_config=_opt(dict(_O)),
                                            evo_config=_opt(dict(_O)), torch_config=_opt(dict(_O))),
                                      lambda session_id, **kw: s.update_graph_settings(session_id, **kw)),
            "load_gpt_template": (_tool("Replace the graph by a model preset's tensor graph.", session_id=dict(_S), preset=_opt(dict(_S)), config=_opt(dict(_O))),
                                  lambda session_id, preset="nanogpt", config=None: s.load_gpt_template(session_id, preset, config)),
            "probe_node": (_tool("Sample a scalar neuron over its input ranges.", session_id=dict(_S), node_id=dict(_S), n_samples=_opt(dict(_I))),
                           lambda session_id, node_id, n_samples=1000: s.probe_node(session_id, node_id, n_samples)),
            "execute": (_tool("Run the scalar graph on flat inputs.", session_id=dict(_S), inputs=dict(_A)),
                        lambda session_id, inputs: {"outputs": s.execute(session_id, inputs)}),
            "trace": (_tool("Run the graph and return every node's values.", session_id=dict(_S), inputs=dict(_O)),
                      lambda session_id, inputs: s.trace(session_id, inputs)),
            "train_start": (_tool("Start training in the background.", session_id=dict(_S), inputs=dict(_A), targets=dict(_A),
                                  method=_opt(dict(_S)), steps=_opt(dict(_I)), learning_rate=_opt(dict(_N))),
                            lambda session_id, inputs, targets, method="sgd", steps=500, learning_rate=0.5:
                            {"run_id": s.train_start(session_id, inputs, targets, method=method, steps=steps, learning_rate=learning_rate)}),
            "train_status": (_tool("Status of a training run.", run_id=dict(_S)), lambda run_id: s.train_status(run_id)),
            "train_stop": (_tool("Ask a training run to stop.", run_id=dict(_S)), lambda run_id: s.train_stop(run_id)),
            "list_presets": (_tool("Names of the model presets."), self._presets),
            "build_preset": (_tool("Build a preset's model spec.", name=dict(_S)), self._build_preset),
            "trace_torch": (_tool("Compile a preset's tensor graph (tiny dimensions) and report its instructions.", name=dict(_S)), self._trace_torch),
            "dataset_info": (_tool("Describe a token-shard dataset.", path=dict(_S), seq_len=_opt(dict(_I)), batch_size=_opt(dict(_I))), self._dataset_info),
            "semantic_match": (_tool("Semantic topics found in a text.", text=dict(_S)), self._semantic_match),
            "semantic_encode": (_tool("Encode dimension -> topic pairs as a semantic vector.", topics=dict(_O)), self._semantic_encode),
            "native_info": (_tool("Kernel library, device and native engine families."), self._native_info),
            "training_plan": (_tool("Plan of a native training run (no GPU needed).", config=_opt(dict(_O))), self._plan),
        }

    # ---- tool bodies that need imports ---------------------------------------------------------
    def _builtins(self):
        from ..builtins import BUILTIN_MAP
        return sorted(BUILTIN_MAP)

    def _presets(self):
        from ..presets import PRESET_BUILDERS
        return sorted(PRESET_BUILDERS)

    def _build_preset(self, name: str):
        from ..presets import build_preset
        return build_preset(name).to_dict()

    def _trace_torch(self, name: str):
        """Builds the preset at toy dimensions, compiles its tensor graph and runs one forward."""
        import torch
        from ..presets import build_preset
        from ..torch_backend import CompiledTorchGraph
        from ..torch_templates import build_gpt_root_graph
        kw = dict(vocab_size=64, num_layers=4 if name.startswith("muse") else 2, model_dim=32, num_heads=4)
        graph = build_gpt_root_graph(build_preset(name, **kw))
        model = CompiledTorchGraph(graph)
        tok = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(0))
        loss = model(tok, tok)[0]
        return {"preset": name, "nodes": len(graph.nodes), "edges": len(graph.edges),
                "parameters": sum(p.numel() for p in model.parameters()), "loss": float(loss.detach())}

    def _dataset_info(self, path: str, seq_len: int = 1024, batch_size: int = 64):
        from ..data import TokenDataset
        return TokenDataset(path, allow_train_as_val=True).describe(seq_len, batch_size)

    def _semantic_match(self, text: str):
        from ..semantic import ConversationalVocabulary
        return ConversationalVocabulary().match_topics_in_text(text)

    def _semantic_encode(self, topics: dict):
        from ..semantic import ConversationalVocabulary, build_semantic_targets_from_topics, semantic_targets_to_vectors
        v = ConversationalVocabulary()
        t = build_semantic_targets_from_topics(topics, vocab=v)
        return {"targets": t.tolist(), "vector": semantic_targets_to_vectors(t, vocab=v)[0].tolist(), "dims": v.semantic_dim_names}

    def _native_info(self):
        from ..native_templates import NATIVE_FAMILIES
        from ..ops import _lib
        return {"kernel_library": str(_lib.lib_path()), "present": _lib.available(), "target": "sm_100a",
                "families": {k: list(v) for k, v in NATIVE_FAMILIES.items()}}

    def _plan(self, config: dict | None = None):
        from ..native_train import NativeTrainConfig, training_plan
        return training_plan(NativeTrainConfig(**(config or {})))

    # ---- protocol ------------------------------------------------------------------------------
    def list_tools(self) -> list[dict]:
        return [{"name": n, **spec} for n, (spec, _) in self.tools.items()]

    def call(self, name: str, arguments: dict | None = None) -> Any:
        if name not in self.tools:
            raise KeyError(f"unknown tool {name!r}")
        return self.tools[name][1](**(arguments or {}))

    def handle(self, msg: dict) -> dict | None:
        mid, method, params = msg.get("id"), msg.get("method"), msg.get("params") or {}
        try:
            if method == "initialize":
                result = {"protocolVersion": "2024-11-05", "serverInfo": {"name": "neuralfn_b200", "version": "0.1"},
                          "capabilities": {"tools": {}}}
            elif method == "tools/list":
                result = {"tools": self.list_tools()}
            elif method == "tools/call":
                out = self.call(params["name"], params.get("arguments"))
                result = {"content": [{"type": "text", "text": json.dumps(out, default=str)}], "isError": False}
            elif method in ("notifications/initialized", "ping"):
                result = {}
            else:
                return {"jsonrpc": "2.0", "id": mid, "error": {"code": -32601, "message": f"unknown method {method}"}}
        except Exception as exc:
            if method == "tools/call":
                return {"jsonrpc": "2.0", "id": mid,
                        "result": {"content": [{"type": "text", "text": f"{type(exc).__name__}: {exc}"}], "isError": True}}
            return {"jsonrpc": "2.0", "id": mid, "error": {"code": -32000, "message": f"{type(exc).__name__}: {exc}"}}
        return None if mid is None else {"jsonrpc": "2.0", "id": mid, "result": result}


def main() -> int:
    server = McpToolServer()
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        reply = server.handle(json.loads(line))
        if reply is not None:
            sys.stdout.write(json.dumps(reply) + "\n")
            sys.stdout.flush()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
