"""Surrogate, evolutionary and hybrid edge trainers on small scalar graphs (CPU)."""
from neuralfn_b200.evolutionary import EvoConfig, EvolutionaryTrainer
from neuralfn_b200.graph import Edge, NeuronGraph, NeuronInstance
from neuralfn_b200.hybrid import HybridConfig, HybridTrainer, build_scopes
from neuralfn_b200.neuron import subgraph_neuron
from neuralfn_b200.scalar_builtins import make_builtin
from neuralfn_b200.sgd import init_edge_params_normal
from neuralfn_b200.surrogate import SurrogateTrainer, TrainConfig, build_surrogates

X = [(0.0, 0.0), (0.0, 1.0), (1.0, 0.0), (1.0, 1.0)]
Y_AND = [(0.0,), (0.0,), (0.0,), (1.0,)]


def tiny(hidden=2, name="g"):
    g = NeuronGraph(name=name)
    for i in range(2):
        g.add_node(NeuronInstance(make_builtin("input"), instance_id=f"in{i}"))
    for h in range(hidden):
        g.add_node(NeuronInstance(make_builtin("tanh_neuron"), instance_id=f"h{h}"))
    g.add_node(NeuronInstance(make_builtin("sigmoid"), instance_id="out"))
    k = 0
    for i in range(2):
        for h in range(hidden):
            g.add_edge(Edge(id=f"e{k:02d}", src_node=f"in{i}", dst_node=f"h{h}"))
            k += 1
    for h in range(hidden):
        g.add_edge(Edge(id=f"e{k:02d}", src_node=f"h{h}", dst_node="out"))
        k += 1
    g.input_node_ids, g.output_node_ids = ["in0", "in1"], ["out"]
    return g


def test_evolutionary_improves():
    g = tiny()
    init_edge_params_normal(g, seed=0)
    tr = EvolutionaryTrainer(g, EvoConfig(population_size=20, generations=25, seed=0))
    hist = tr.train(X, Y_AND)
    assert hist[-1] < hist[0] and hist[-1] < 0.1


def test_surrogate_trainer_improves():
    g = tiny()
    init_edge_params_normal(g, seed=1, std=0.5)
    sur = build_surrogates(g, n_samples=1500, epochs=30, seed=0)
    assert set(sur) == {n.neuron_def.id for n in g.nodes.values() if n.neuron_def.n_inputs}
    tr = SurrogateTrainer(g, TrainConfig(learning_rate=5e-2, epochs=150, batch_size=4, seed=0), surrogates=sur)
    hist = tr.train(X, Y_AND)
    assert hist[-1] < hist[0]


def test_hybrid_nested_scopes():
    inner = tiny(name="inner")
    inner.training_method = "evolutionary"
    init_edge_params_normal(inner, seed=2)
    outer = NeuronGraph(name="outer", training_method="sgd")
    for i in range(2):
        outer.add_node(NeuronInstance(make_builtin("input"), instance_id=f"x{i}"))
    outer.add_node(NeuronInstance(subgraph_neuron(inner, name="inner", input_aliases=["a", "b"],
                                                  output_aliases=["y"]), instance_id="sub"))
    outer.add_node(NeuronInstance(make_builtin("identity"), instance_id="o"))
    outer.add_edge(Edge(id="a", src_node="x0", dst_node="sub", dst_port=0))
    outer.add_edge(Edge(id="b", src_node="x1", dst_node="sub", dst_port=1))
    outer.add_edge(Edge(id="c", src_node="sub", dst_node="o"))
    outer.input_node_ids, outer.output_node_ids = ["x0", "x1"], ["o"]
    scopes = build_scopes(outer)
    assert [s.name for s in scopes.walk_post_order()] == ["sub", "outer"]
    tr = HybridTrainer(outer, HybridConfig(outer_rounds=2, evo_generations=8, evo_population=10, sgd_steps=60))
    hist = tr.train(X, Y_AND)
    assert hist[-1] <= tr.scope_log[0]["loss_before"]
    assert {e["method"] for e in tr.scope_log} == {"evolutionary", "sgd"}
