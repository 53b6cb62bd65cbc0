"""Graph -> ``nn.Module`` compiler of the tensor runtime.

A ``NeuronGraph`` whose nodes are ``module`` / ``subgraph`` / scalar ``function`` neurons
is lowered once into a flat *instruction list*: for every non-input node, in topological
order, the module to call and the ``(value slot, port)`` of each argument. ``forward`` then
runs the list over a slot table - no dictionary look-ups or edge scans in the hot loop.
Nested subgraphs become nested ``CompiledTorchGraph`` modules. Cycles and multi-edge
fan-in into one port are rejected (use an explicit combine node).

Reference counterpart: ``CompiledTorchGraph`` (``neuralfn/torch_backend.py:4077-4320``),
including ``trace()`` keys ``parent/child`` and ``sync_state_back``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ..graph import NeuronGraph
from ..neuron import decode_module_state_dict, encode_module_state_dict
from .stages_core import build_module

__all__ = ["CompiledTorchGraph", "build_function_module", "build_module"]


class _FunctionModule(nn.Module):
    def __init__(self, name: str, fn) -> None:
        super().__init__()
        self.fn_name, self._fn = name, fn

    def forward(self, *args: Tensor):
        return self._fn(*args)


def _softmax2(a, b):
    p = torch.softmax(torch.stack((a, b), dim=-1), dim=-1)
    return p[..., 0], p[..., 1]


def _logsoftmax2(a, b):
    p = torch.log_softmax(torch.stack((a, b), dim=-1), dim=-1)
    return p[..., 0], p[..., 1]


_TENSOR_FUNCTIONS = {
    "sigmoid": torch.sigmoid, "relu": F.relu, "tanh_neuron": torch.tanh, "tanh": torch.tanh,
    "threshold": lambda x: (x >= 0).to(x.dtype), "identity": lambda x: x, "negate": lambda x: -x,
    "add": lambda a, b: a + b, "multiply": lambda a, b: a * b, "gaussian": lambda x: torch.exp(-x * x),
    "log": lambda x: torch.log(x.clamp(min=1e-7)), "leaky_relu": lambda x: F.leaky_relu(x, 0.01),
    "prelu": lambda x: torch.where(x >= 0, x, 0.25 * x), "relu6": F.relu6, "elu": F.elu, "selu": F.selu,
    "gelu": F.gelu, "silu": F.silu, "mish": F.mish, "softplus": F.softplus, "softsign": F.softsign,
    "hard_sigmoid": F.hardsigmoid, "hard_tanh": F.hardtanh, "hard_swish": F.hardswish,
    "softmax_2": _softmax2, "logsoftmax_2": _logsoftmax2, "input": lambda x: x, "output": lambda x: x,
}


def build_function_module(name: str, tile_cuda_config: Any = None) -> nn.Module:
    """Tensor version of a built-in scalar function neuron (element-wise)."""
    try:
        return _FunctionModule(name, _TENSOR_FUNCTIONS[name])
    except KeyError:
        raise ValueError(f"Function neuron '{name}' has no tensor implementation") from None


@dataclass(frozen=True)
class _Instr:
    node_id: str
    slot: int
    kind: str
    args: tuple[tuple[int, int], ...]  # (source slot, source port)


class CompiledTorchGraph(nn.Module):
    def __init__(self, graph: NeuronGraph, *, kernel_backend: str = "auto", tile_cuda_strict: bool = False,
                 tile_cuda_report_path: str | None = None) -> None:
        super().__init__()
        self.graph = graph
        self.kernel_backend = kernel_backend
        self.resolved_kernel_backend = "sm100" if kernel_backend in ("auto", "sm100", "tile_cuda") else "torch"
        if graph.has_cycles():
            raise ValueError(f"Torch runtime does not support cyclic graphs: '{graph.name}'")
        self.order = tuple(graph.topological_order() if graph.nodes else [])
        self.node_modules = nn.ModuleDict()
        for nid, node in graph.nodes.items():
            nd = node.neuron_def
            if nd.kind == "module":
                mod = build_module(nd.module_type, nd.module_config)
                if nd.module_state:
                    mod.load_state_dict(decode_module_state_dict(nd.module_state))
                self.node_modules[nid] = mod
            elif nd.kind == "subgraph" and nd.subgraph is not None:
                self.node_modules[nid] = CompiledTorchGraph(nd.subgraph, kernel_backend=kernel_backend)
            elif nd.kind == "function":
                self.node_modules[nid] = build_function_module(nd.name)
        self._slot_of = {nid: i for i, nid in enumerate(self.order)}
        self._input_plan = tuple((self._slot_of[nid], graph.nodes[nid].neuron_def.n_outputs)
                                 for nid in graph.input_node_ids)
        self._output_slots = tuple(self._slot_of[nid] for nid in graph.output_node_ids)
        self._expected_flat_inputs = sum(n for _s, n in self._input_plan)
        self._program = self._lower(graph)

    def _lower(self, graph: NeuronGraph) -> tuple[_Instr, ...]:
        inputs = set(graph.input_node_ids)
        program = []
        for nid in self.order:
            if nid in inputs:
                continue
            nd = graph.nodes[nid].neuron_def
            n_in = nd.n_inputs
            args: list[tuple[int, int] | None] = [None] * n_in
            for e in graph._incoming(nid):
                if e.dst_port >= n_in:
                    raise ValueError(f"Edge '{e.id}' dst_port={e.dst_port} exceeds destination inputs")
                if args[e.dst_port] is not None:
                    raise ValueError(f"Torch graph '{graph.name}' has multiple incoming edges into node "
                                     f"'{nid}' port {e.dst_port}; use an explicit combine node instead")
                args[e.dst_port] = (self._slot_of[e.src_node], e.src_port)
            missing = [i for i, a in enumerate(args) if a is None]
            if missing:
                raise ValueError(f"Node '{nid}' is missing required torch inputs at ports {missing}")
            program.append(_Instr(nid, self._slot_of[nid], nd.kind, tuple(args)))  # type: ignore[arg-type]
        return tuple(program)

    # ------------------------------------------------------------------ execution --
    def _seed(self, flat_inputs: tuple[Tensor, ...]) -> list:
        if len(flat_inputs) != self._expected_flat_inputs:
            raise ValueError(f"Graph '{self.graph.name}' expected {self._expected_flat_inputs} flattened "
                             f"inputs but received {len(flat_inputs)}")
        table: list = [None] * len(self.order)
        cur = 0
        for slot, n in self._input_plan:
            table[slot] = tuple(flat_inputs[cur:cur + n])
            cur += n
        return table

    def enable_activation_checkpointing(self, enabled: bool = True) -> int:
        """Recompute decoder blocks in the backward pass instead of keeping their activations: every
        subgraph node whose id ends in ``block_<n>`` (here and in nested graphs) runs under
        ``torch.utils.checkpoint`` while gradients are enabled. Returns the number of such nodes."""
        import re
        count = 0
        self._checkpointed = set()
        for ins in self._program:
            mod = self.node_modules[ins.node_id]
            if ins.kind == "subgraph" and re.search(r"(^|_)block_\d+$", ins.node_id):
                if enabled:
                    self._checkpointed.add(ins.node_id)
                count += 1
            elif isinstance(mod, CompiledTorchGraph):
                count += mod.enable_activation_checkpointing(enabled)
        return count

    def forward(self, *flat_inputs: Tensor) -> tuple[Tensor, ...]:
        table = self._seed(flat_inputs)
        mods = self.node_modules
        ckpt = getattr(self, "_checkpointed", None)
        for ins in self._program:
            if ckpt and ins.node_id in ckpt and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                out = checkpoint(mods[ins.node_id], *[table[s][p] for s, p in ins.args], use_reentrant=False)
            else:
                out = mods[ins.node_id](*[table[s][p] for s, p in ins.args])
            table[ins.slot] = out if isinstance(out, tuple) else (tuple(out) if isinstance(out, list) else (out,))
        flat: list[Tensor] = []
        for s in self._output_slots:
            flat.extend(table[s] or ())
        return tuple(flat)

    def trace(self, *flat_inputs: Tensor):
        """Like ``forward`` but also returns every node's outputs; nested nodes appear as
        ``parent/child`` keys."""
        table = self._seed(flat_inputs)
        traces: dict[str, tuple[Tensor, ...]] = {self.order[s]: table[s] for s, _n in self._input_plan}
        for ins in self._program:
            mod = self.node_modules[ins.node_id]
            args = [table[s][p] for s, p in ins.args]
            if ins.kind == "subgraph":
                out, child = mod.trace(*args)
                for k, v in child.items():
                    traces[f"{ins.node_id}/{k}"] = v
            else:
                out = mod(*args)
            out = out if isinstance(out, tuple) else (tuple(out) if isinstance(out, list) else (out,))
            table[ins.slot] = out
            traces[ins.node_id] = out
        flat: list[Tensor] = []
        for s in self._output_slots:
            flat.extend(table[s] or ())
        return tuple(flat), traces

    # --------------------------------------------------------------------- state --
    def sync_state_back(self) -> None:
        """Write trained module weights back into the graph's ``module_state`` blobs (recursively)."""
        for nid, mod in self.node_modules.items():
            nd = self.graph.nodes[nid].neuron_def
            if isinstance(mod, CompiledTorchGraph):
                mod.sync_state_back()
            elif nd.kind == "module":
                state = {k: v.detach().cpu() for k, v in mod.state_dict().items()}
                nd.module_state = encode_module_state_dict(state) if state else ""

    def routing_modules(self) -> list[nn.Module]:
        from .stages_moe import RoutingStatsMixin
        return [m for m in self.modules() if isinstance(m, RoutingStatsMixin)]
