"""`nfn train --runtime torch` (recipes, adapters, post-training, evolutionary), `nfn eval`, `nfn migrate` on CPU."""
import json

import numpy as np
import pytest
import torch

from neuralfn_b200.cli.nfn import build_parser
from neuralfn_b200.data.shards import write_ppo_prompt_records, write_preference_records, write_sft_records

TINY = ["--device", "cpu", "--n-layer", "2", "--n-head", "2", "--d-model", "32", "--vocab-size", "64", "--seq-len", "16",
        "--batch-size", "4", "--train-rows", "16", "--warmup-steps", "0", "--progress-every", "0", "--learning-rate", "0.01"]


def _run(argv, capsys):
    a = build_parser().parse_args(argv)
    rc = a.fn(a)
    text = capsys.readouterr().out.strip()
    try:
        return rc, json.loads(text)                  # one (possibly indented) document
    except json.JSONDecodeError:
        lines = [ln for ln in text.splitlines() if ln.startswith("{")]
        return rc, json.loads(lines[-1])             # progress lines, then the report


def test_pretrain_then_eval_then_migrate(tmp_path, capsys):
    out = tmp_path / "m.pt"
    rc, rep = _run(["train", "--runtime", "torch", "--preset", "llama", *TINY, "--max-steps", "3", "--output", str(out)], capsys)
    assert rc == 0 and rep["status"] == "ok" and rep["steps"] == 3 and rep["objective"] == "ar"
    assert out.exists() and out.with_suffix(".json").exists() and out.with_suffix(".report.json").exists()
    rc, ev = _run(["eval", "--graph", str(out.with_suffix(".json")), "--weights", str(out), "--device", "cpu", "--seq-len", "16",
                   "--eval-batches", "2", "--eval-batch-size", "4", "--prompt-tokens", "1,2,3;7", "--max-new-tokens", "3",
                   "--report-path", str(tmp_path / "eval.json")], capsys)
    assert rc == 0 and 0 < ev["validation_loss"] < 10 and ev["perplexity"] == pytest.approx(np.exp(ev["validation_loss"]), rel=1e-6)
    assert [len(p["token_ids"]) for p in ev["prompt_probes"]] == [3, 3] and (tmp_path / "eval.json").exists()
    rc, dry = _run(["migrate", "graph-to-native", "--graph", str(out.with_suffix(".json")), "--dry-run"], capsys)
    assert rc == 0 and dry["status"] == "dry-run" and "compatibility" in dry
    rc, mig = _run(["migrate", "graph-to-native", "--graph", str(out.with_suffix(".json")), "--weights", str(out),
                    "--output-dir", str(tmp_path / "native")], capsys)
    assert rc == 0 and (tmp_path / "native" / "native-execution-manifest.json").exists() and mig["tensor_bytes"] > 0
    with pytest.raises(FileExistsError):
        _run(["migrate", "graph-to-native", "--graph", str(out.with_suffix(".json")), "--output-dir", str(tmp_path / "native")], capsys)
    a = build_parser().parse_args(["migrate", "muse-glimmer-lora-to-native", "--source", "x", "--output-dir", str(tmp_path / "g")])
    assert a.fn(a) == 2                                               # fails closed: not part of this build


def test_recipe_flags_select_the_graph_runtime_and_objective(tmp_path, capsys):
    rc, plan = _run(["train", "--topology", "semantic_router", "--jepa", *TINY, "--print-plan"], capsys)
    assert rc == 0 and plan["runtime"] == "torch" and plan["objective"] == "semantic_router_jepa"
    assert plan["inputs"] == ["tokens", "target_ids", "sem_targets"]
    rc, rep = _run(["train", "--preset", "semantic_moe_jepa_evo", *TINY, "--max-steps", "2", "--output", str(tmp_path / "s.pt")], capsys)
    assert rc == 0 and rep["steps"] == 2 and rep["objective"] == "semantic_moe_jepa_evo"
    rc, evo = _run(["train", "--preset", "gpt2", *TINY, "--evolutionary", "--evo-population-size", "4", "--evo-elite-count", "1",
                    "--evo-seed", "1", "--max-steps", "2", "--output", str(tmp_path / "e.pt")], capsys)
    assert rc == 0 and evo["optimization"] == "evolutionary" and evo["steps"] == 2
    rc, mu = _run(["train", "--preset", "llama", *TINY, "--optimizer-profile", "muon_adamw", "--max-steps", "2",
                   "--activation-checkpointing", "--output", str(tmp_path / "mu.pt")], capsys)
    assert rc == 0 and mu["optimizer_profile"] == "muon_adamw"


def _records(tmp_path):
    g = np.random.default_rng(0)
    n, T = 8, 16
    ids = g.integers(1, 64, (n, T))
    tg = np.roll(ids, -1, axis=1)
    mask = np.zeros((n, T), dtype=np.float32)
    mask[:, T // 2:] = 1
    d = tmp_path / "ds"
    d.mkdir()
    write_sft_records(d / "sft_train_000.sft", ids, tg, mask, None, vocab_size=64)
    other = g.integers(1, 64, (n, T))
    write_preference_records(d / "preference_train_000.preference",
                             {"input_ids": ids, "targets": tg, "loss_mask": mask},
                             {"input_ids": other, "targets": np.roll(other, -1, axis=1), "loss_mask": mask}, vocab_size=64)
    pmask = np.zeros((n, T), dtype=np.float32)
    pmask[:, :6] = 1                                                    # 6 prompt tokens, room for a response
    write_ppo_prompt_records(d / "ppo_prompt_train_000.ppo_prompt", np.where(pmask > 0, ids, 0), pmask, vocab_size=64)
    return d


def test_post_training_modes_with_adapters(tmp_path, capsys):
    ds = _records(tmp_path)
    base = tmp_path / "base.pt"
    rc, _ = _run(["train", "--runtime", "torch", "--preset", "llama", *TINY, "--max-steps", "1", "--output", str(base)], capsys)
    assert rc == 0
    common = ["--preset", "llama", *TINY, "--dataset", str(ds), "--max-steps", "2", "--base-checkpoint", str(base)]
    rc, sft = _run(["train", "--training-mode", "sft", "--adapter-type", "lora", "--lora-rank", "4", "--lora-targets", "q_proj,v_proj",
                    "--adapter-only-save", *common, "--output", str(tmp_path / "sft.pt")], capsys)
    assert rc == 0 and sft["training_mode"] == "sft" and sft["adapter"] == "lora" and sft["steps"] == 2
    adapter = torch.load(tmp_path / "sft.pt", weights_only=False)
    keys = adapter.get("state_dict", adapter)
    assert keys and all("lora" in k for k in keys)                      # adapter-only artifact
    rc, dpo = _run(["train", "--training-mode", "dpo", "--dpo-beta", "0.2", "--dpo-loss-type", "ipo", "--ref-checkpoint", str(base),
                    *common, "--output", str(tmp_path / "dpo.pt")], capsys)
    assert rc == 0 and dpo["training_mode"] == "dpo" and np.isfinite(dpo["final_loss"])
    rc, rm = _run(["train", "--training-mode", "reward_model", *common, "--output", str(tmp_path / "rm.pt")], capsys)
    assert rc == 0 and rm["training_mode"] == "reward_model"
    rc, ppo = _run(["train", "--training-mode", "ppo", "--rollout-length", "4", "--ppo-epochs-per-rollout", "1", "--kl-coef", "0.05",
                    *common, "--output", str(tmp_path / "ppo.pt")], capsys)
    assert rc == 0 and ppo["steps"] == 2 and (tmp_path / "ppo.pt").exists()
