"""Driver of the model-parallel families on one CPU process: JSON events, checkpoints, resume."""
import json

import torch


def _events(capsys):
    return [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]


def test_ep_driver_trains_checkpoints_and_resumes(tmp_path, capsys):
    from neuralfn_b200.parallel.train import main
    common = ["--parallel", "ep", "--device", "cpu", "--n-layer", "1", "--n-head", "2", "--n-kv-head", "1", "--d-model", "64", "--vocab-size", "128",
              "--experts", "4", "--top-k", "2", "--expert-hidden", "64", "--batch-size", "2", "--seq-len", "16", "--learning-rate", "3e-3",
              "--warmup-steps", "1", "--progress-every", "1", "--output-dir", str(tmp_path)]
    assert main(common + ["--max-steps", "4", "--checkpoint-every", "2"]) == 0
    ev = _events(capsys)
    steps = [e for e in ev if e["event"] == "train_step"]
    assert [e["step"] for e in steps] == [1, 2, 3, 4] and all(e["loss"] == e["loss"] for e in steps)
    assert [e["step"] for e in ev if e["event"] == "checkpoint"] == [2, 4] and ev[-1]["event"] == "complete"
    man = json.loads((tmp_path / "step_00000004" / "manifest.json").read_text())
    assert man["optimizer_step"] == 4 and man["parallel"] == "ep" and man["config"]["n_experts"] == 4
    assert main(common + ["--max-steps", "6", "--resume"]) == 0
    ev = _events(capsys)
    assert ev[0] == {"event": "resumed", "step": 4}
    assert [e["step"] for e in ev if e["event"] == "train_step"] == [5, 6] and ev[-1]["steps"] == 2


def test_tp_driver_single_rank(tmp_path, capsys):
    from neuralfn_b200.checkpoint.safetensors_io import read_safetensors
    from neuralfn_b200.parallel.train import main
    assert main(["--parallel", "tp", "--model", "tiny", "--device", "cpu", "--batch-size", "1", "--seq-len", "16", "--max-steps", "2",
                 "--progress-every", "1", "--checkpoint-every", "2", "--output-dir", str(tmp_path)]) == 0
    ev = _events(capsys)
    assert ev[-1]["event"] == "complete" and ev[-1]["parallel"] == "tp"
    tensors, meta = read_safetensors(tmp_path / "step_00000002" / "rank000.safetensors")
    assert meta["step"] == "2" and "master.layers.0.wqkv" in tensors and tensors["adam.m"].dtype == torch.float32


def test_nfn_train_routes_parallel_families(capsys, monkeypatch):
    from neuralfn_b200.cli import nfn
    monkeypatch.setattr("torch.cuda.is_available", lambda: False)
    rc = nfn.main(["train", "--parallel", "ep", "--n-layer", "1", "--n-head", "2", "--n-kv-head", "1", "--d-model", "64", "--vocab-size", "128",
                   "--experts", "2", "--top-k-experts", "1", "--expert-hidden", "64", "--batch-size", "1", "--seq-len", "8", "--max-steps", "1",
                   "--progress-every", "1", "--checkpoint-every", "0"])
    assert rc == 0 and _events(capsys)[-1]["parallel"] == "ep"
