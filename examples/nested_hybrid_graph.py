"""A graph inside a neuron: a small sub-graph (two weighted inputs through tanh) is wrapped as a
subgraph neuron, used twice in an outer graph, and the whole thing is trained end to end with
exact-gradient SGD (gradients flow through the nested graphs' edges as well).

    python examples/nested_hybrid_graph.py
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from neuralfn_b200.graph import Edge, NeuronGraph, NeuronInstance  # noqa: E402
from neuralfn_b200.neuron import subgraph_neuron  # noqa: E402
from neuralfn_b200.scalar_builtins import make_builtin  # noqa: E402
from neuralfn_b200.sgd import GraphSGDTrainer, SGDConfig, init_edge_params_normal  # noqa: E402


def build_inner() -> NeuronGraph:
    g = NeuronGraph(name="pair_tanh")
    a, b = NeuronInstance(make_builtin("input"), instance_id="a"), NeuronInstance(make_builtin("input"), instance_id="b")
    t = NeuronInstance(make_builtin("tanh_neuron"), instance_id="t")
    for n in (a, b, t):
        g.add_node(n)
    g.add_edge(Edge(id="ia", src_node="a", dst_node="t"))
    g.add_edge(Edge(id="ib", src_node="b", dst_node="t"))
    g.input_node_ids, g.output_node_ids = ["a", "b"], ["t"]
    return g


def build_outer() -> NeuronGraph:
    inner = subgraph_neuron(build_inner(), name="pair_tanh")
    g = NeuronGraph(name="nested")
    x0, x1 = NeuronInstance(make_builtin("input"), instance_id="x0"), NeuronInstance(make_builtin("input"), instance_id="x1")
    u, v = NeuronInstance(inner, instance_id="u"), NeuronInstance(inner, instance_id="v")
    out = NeuronInstance(make_builtin("sigmoid"), instance_id="out")
    for n in (x0, x1, u, v, out):
        g.add_node(n)
    k = 0
    for src in ("x0", "x1"):
        for dst in ("u", "v"):
            g.add_edge(Edge(id=f"e{k}", src_node=src, dst_node=dst, dst_port=0 if src == "x0" else 1))
            k += 1
    g.add_edge(Edge(id="ou", src_node="u", dst_node="out"))
    g.add_edge(Edge(id="ov", src_node="v", dst_node="out"))
    g.input_node_ids, g.output_node_ids = ["x0", "x1"], ["out"]
    return g


def main() -> int:
    g = build_outer()
    init_edge_params_normal(g, seed=3)
    xs = [(0.0, 0.0), (0.0, 1.0), (1.0, 0.0), (1.0, 1.0)]
    ys = [(0.0,), (1.0,), (1.0,), (0.0,)]
    hist = GraphSGDTrainer(g, SGDConfig(learning_rate=0.5, steps=3000)).train(xs, ys)
    print(f"nested graph: MSE {hist[0]:.4f} -> {hist[-1]:.4f}")
    for x in xs:
        print(x, "->", round(g.execute({"x0": (x[0],), "x1": (x[1],)})["out"][0], 3))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
