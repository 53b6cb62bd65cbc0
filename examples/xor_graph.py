"""XOR with the scalar graph runtime: build a 2-4-1 sigmoid graph, train it with exact-gradient
SGD (fp64 N(0,1) init from seed 0, lr 0.5, 2000 steps), save it as JSON and reload it.

    python examples/xor_graph.py [out.json]
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from neuralfn_b200.graph import Edge, NeuronGraph, NeuronInstance  # noqa: E402
from neuralfn_b200.scalar_builtins import make_builtin  # noqa: E402
from neuralfn_b200.serialization import load_graph, save_graph  # noqa: E402
from neuralfn_b200.sgd import GraphSGDTrainer, SGDConfig, init_edge_params_normal  # noqa: E402

XOR_X = [(0.0, 0.0), (0.0, 1.0), (1.0, 0.0), (1.0, 1.0)]
XOR_Y = [(0.0,), (1.0,), (1.0,), (0.0,)]


def build_xor_graph(hidden: int = 4) -> NeuronGraph:
    g = NeuronGraph(name="xor")
    ins = [NeuronInstance(make_builtin("input"), instance_id=f"in{i}") for i in range(2)]
    hid = [NeuronInstance(make_builtin("sigmoid"), instance_id=f"h{i}") for i in range(hidden)]
    out = NeuronInstance(make_builtin("sigmoid"), instance_id="out")
    for n in (*ins, *hid, out):
        g.add_node(n)
    k = 0
    for i in ins:
        for h in hid:
            g.add_edge(Edge(id=f"e{k:03d}", src_node=i.instance_id, dst_node=h.instance_id))
            k += 1
    for h in hid:
        g.add_edge(Edge(id=f"e{k:03d}", src_node=h.instance_id, dst_node="out"))
        k += 1
    g.input_node_ids = [n.instance_id for n in ins]
    g.output_node_ids = ["out"]
    return g


def main(argv: list[str]) -> int:
    g = build_xor_graph()
    init_edge_params_normal(g, seed=0)
    history = GraphSGDTrainer(g, SGDConfig(learning_rate=0.5, steps=2000)).train(XOR_X, XOR_Y)
    print(f"final MSE {history[-1]:.6f} after {len(history)} steps")
    out = Path(argv[1]) if len(argv) > 1 else Path("xor_trained.json")
    save_graph(g, out)
    g2 = load_graph(out)
    for x, y in zip(XOR_X, XOR_Y):
        got = g2.execute({"in0": (x[0],), "in1": (x[1],)})["out"][0]
        print(f"{x} -> {got:.4f} (want {y[0]})")
    return 0 if history[-1] < 0.01 else 1


if __name__ == "__main__":
    raise SystemExit(main(sys.argv))
