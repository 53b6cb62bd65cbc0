"""Graph-authored native training preflight (CPU)."""
import json

import pytest

from neuralfn_b200 import presets
from neuralfn_b200.native_graph_train import GraphPreflightError, plan_native_graph_training, shape_hash, strict_json_loads
from neuralfn_b200.serialization import graph_to_json
from neuralfn_b200.torch_templates import build_gpt_root_graph

SMALL = dict(vocab_size=64, num_layers=2, model_dim=32, num_heads=4)


def _write(tmp_path, name, preset, **kw):
    p = tmp_path / f"{name}.json"
    p.write_text(graph_to_json(build_gpt_root_graph(presets.build_preset(preset, **{**SMALL, **kw}))))
    return p


def test_plans_for_native_and_non_native_graphs(tmp_path):
    plan = plan_native_graph_training(_write(tmp_path, "a", "gpt2_qknorm"), max_steps=10)
    assert plan.ok and plan.selector == "gpt2_qknorm" and plan.route == "native-gpt" and plan.shape_sha256 == plan.rebuilt_shape_sha256
    assert plan.train_config["n_layer"] == 2 and "--template-name" in plan.trainer_argv and plan.trainer_argv[-2:] == ["--max-steps", "10"]
    assert plan_native_graph_training(_write(tmp_path, "b", "gpt2_stable")).selector == "gpt2_stable"
    ll = plan_native_graph_training(_write(tmp_path, "c", "llama"))
    assert ll.ok and ll.route == "native-llama"
    moe = plan_native_graph_training(_write(tmp_path, "d", "moe"))
    assert not moe.ok and moe.blockers
    other = plan_native_graph_training(_write(tmp_path, "e", "jamba"))
    assert not other.ok and "tensor runtime" in " ".join(other.blockers)


def test_hand_edits_and_malformed_files_are_caught(tmp_path):
    p = _write(tmp_path, "g", "gpt2")
    doc = json.loads(p.read_text())
    h0 = shape_hash(doc)
    moved = json.loads(p.read_text())
    for n in (moved["nodes"].values() if isinstance(moved["nodes"], dict) else moved["nodes"]):
        n["position"] = [1.0, 2.0]
    assert shape_hash(moved) == h0  # layout does not enter the shape
    doc["edges"].pop(sorted(doc["edges"])[-1])
    q = tmp_path / "edited.json"
    q.write_text(json.dumps(doc))
    plan = plan_native_graph_training(q)
    assert not plan.ok and "differs structurally" in " ".join(plan.blockers)
    with pytest.raises(GraphPreflightError):
        strict_json_loads(b'{"a": 1, "a": 2}')
    with pytest.raises(GraphPreflightError):
        strict_json_loads(b'{"a": NaN}')
    (tmp_path / "nograph.json").write_text("[1, 2]")
    with pytest.raises(GraphPreflightError):
        plan_native_graph_training(tmp_path / "nograph.json")


def test_materialized_sidecars(tmp_path):
    p = _write(tmp_path, "m", "gpt2_zloss")
    out = tmp_path / "artifact"
    plan = plan_native_graph_training(p, artifact_dir=out, materialize=True)
    assert plan.ok and (out / "source-graph.json").read_bytes() == p.read_bytes()
    proof = json.loads((out / "native-training-proof.json").read_text())
    assert proof["graph_sha256"] == plan.graph_sha256 and proof["ok"]
    assert json.loads((out / "native-execution-manifest.json").read_text())["status"] == "ready"
    with pytest.raises(GraphPreflightError):
        plan_native_graph_training(p, artifact_dir=out, materialize=True)  # never into an existing directory
