"""CLI paths that need no GPU (plan, layout, listings, checkpoint inspection) and a GPU
end-to-end run: shards -> nfn train -> checkpoint -> resume -> nfn infer."""
import json
import subprocess
import sys

import numpy as np
import pytest


def _nfn(*args, check=True):
    p = subprocess.run([sys.executable, "-m", "neuralfn_b200.cli.nfn", *args], capture_output=True, text=True, timeout=600)
    if check:
        assert p.returncode == 0, p.stdout + p.stderr
    return p


def test_plan_layout_and_listings():
    plan = json.loads(_nfn("train", "--print-plan", "--batch-size", "16", "--gpus", "8").stdout)
    assert plan["grad_accum_steps"] == 4 and plan["effective_train_batch_tokens"] == 524288 and plan["parameters"] > 124e6
    lay = json.loads(_nfn("checkpoint-layout", "--n-layer", "2").stdout)
    assert lay["tensors"][0]["name"] == "wte" and lay["tensors"][0]["offset"] == 1024
    assert lay["file_bytes"] == 1024 + sum(t["nbytes"] for t in lay["tensors"])
    assert "gpt2_qknorm" in json.loads(_nfn("list-templates").stdout)["gpt"]
    assert len(json.loads(_nfn("list-presets").stdout)) >= 67
    assert json.loads(_nfn("native-info").stdout)["target"] == "sm_100a"
    bad = _nfn("train", "--base-model", "rwkv", "--print-plan", check=False)
    assert bad.returncode == 1 and json.loads(bad.stdout)["status"] == "error"


@pytest.mark.gpu
def test_train_resume_and_infer_end_to_end(tmp_path):
    from neuralfn_b200.data import write_legacy_shard
    rng = np.random.default_rng(0)
    data = tmp_path / "data"
    data.mkdir()
    period = rng.integers(0, 300, 97)
    write_legacy_shard(data / "fineweb_train_000000.bin", np.tile(period, 700), with_header=True)
    write_legacy_shard(data / "fineweb_val_000000.bin", np.tile(period, 60))
    out = tmp_path / "run"
    common = ["train", "--base-model", "gpt", "--template-name", "gpt2_qknorm", "--dataset", str(data), "--output-dir", str(out),
              "--batch-size", "4", "--seq-len", "64", "--train-batch-tokens", "512", "--n-layer", "2", "--n-head", "2", "--d-model", "128",
              "--vocab-size", "300", "--learning-rate", "3e-3", "--warmup-steps", "2", "--eval-every", "10", "--eval-batches", "2",
              "--train-loss-every", "5", "--checkpoint-every", "10", "--progress-every", "0"]
    r1 = json.loads(_nfn(*common, "--max-steps", "10").stdout.strip().splitlines()[-1])
    assert r1["status"] == "ok" and r1["plan"]["grad_accum_steps"] == 2 and r1["steps"] == 10
    assert r1["train_losses"][-1]["loss"] < r1["train_losses"][0]["loss"]
    assert r1["train_compute_tokens_per_second"] > 0 and (out / "DONE_00000010").exists()
    r2 = json.loads(_nfn(*common, "--max-steps", "20", "--resume").stdout.strip().splitlines()[-1])
    assert r2["resumed_from_step"] == 10 and r2["steps"] == 10 and (out / "model_00000020.bin").exists()
    assert r2["validation"]["losses"][-1]["loss"] < r1["validation"]["losses"][-1]["loss"] + 0.05
    info = json.loads(_nfn("inspect-checkpoint", str(out / "model_00000020.bin")).stdout)
    assert info["num_layers"] == 2 and len(info["sha256"]) == 64
    gen = json.loads(_nfn("infer", "--checkpoint", str(out / "model_00000020.bin"), "--prompt-tokens",
                          ",".join(map(str, period[:12])), "--max-new-tokens", "8").stdout.strip().splitlines()[-1])
    assert gen["status"] == "ok" and len(gen["generated"][0]) == 8


def test_kernel_registry_matches_the_built_library_and_examples_run():
    import subprocess
    import sys
    from pathlib import Path

    from neuralfn_b200.ops import _lib
    from neuralfn_b200.ops.registry import KERNELS, coverage_report, coverage_summary
    rows = coverage_report()
    assert len(rows) == len(KERNELS)
    if _lib.available():
        assert not [r["op"] for r in rows if r["status"] == "missing"]
        s = coverage_summary()
        assert s["native"] >= 35 and s["tensor_core_kernels"] >= 6
    root = Path(__file__).resolve().parents[1]
    out = subprocess.run([sys.executable, str(root / "examples" / "xor_graph.py"), "/tmp/nfn_xor_example.json"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "final MSE" in out.stdout


def test_gpu_picker_prefers_idle_devices(monkeypatch):
    from neuralfn_b200.utils.cuda_device import GpuInfo, parse_nvidia_smi_csv, pick_dedicated_gpu
    g = parse_nvidia_smi_csv("0, NVIDIA B200, 183359, 120000\n1, NVIDIA B200, 183359, 4\n2, NVIDIA B200, 183359, 4\nnot a row\n")
    assert [x.index for x in g] == [0, 1, 2] and pick_dedicated_gpu(g) == 1
    assert pick_dedicated_gpu([GpuInfo(0, "x", 100, 10, 1), GpuInfo(1, "x", 100, 50, 0)]) == 1
    assert pick_dedicated_gpu(g, min_free_mib=10 ** 9) is None
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "0,2")
    assert pick_dedicated_gpu(g) == 2


def test_compat_launcher_translates_llmc_flags(capsys):
    from neuralfn_b200.cli import nfn
    from neuralfn_b200.cli.compat import translate_llmc_args
    kw, notes = translate_llmc_args(["-i", "data/fineweb/train_*.bin", "-j", "data/fineweb/val_*.bin", "-o", "out", "-e", "d24", "-b", "32", "-t", "2048",
                                     "-d", "524288", "-l", "0.0003", "-u", "700", "-q", "0.1", "-c", "0.1", "-x", "100", "-z", "1", "-r", "0", "-k", "cosine"])
    assert (kw["n_layer"], kw["n_head"], kw["d_model"]) == (24, 16, 1024) and kw["dataset"] == "data/fineweb" and kw["batch_size"] == 32
    assert kw["seq_len"] == 2048 and kw["warmup_steps"] == 700 and kw["final_lr_fraction"] == 0.1 and kw["max_steps"] == 100
    assert set(notes["ignored"]) == {"-z", "-r", "val_pattern"}
    import pytest
    with pytest.raises(ValueError):
        translate_llmc_args(["-e", "gpt2_124M.bin"])
    with pytest.raises(ValueError):
        translate_llmc_args(["--bogus", "1"])
    assert nfn.main(["compat-train", "--print-plan", "--", "-e", "d12", "-b", "16", "-t", "1024", "-d", "524288"]) == 0
    plan = json.loads(capsys.readouterr().out)
    assert plan["status"] == "plan" and plan["grad_accum_steps"] == 32


def test_migrate_native_cli(tmp_path, capsys):
    from neuralfn_b200.cli import nfn
    from neuralfn_b200.presets import build_preset
    from neuralfn_b200.serialization import save_graph
    from neuralfn_b200.torch_templates import build_gpt_root_graph
    g = build_gpt_root_graph(build_preset("gpt2", vocab_size=64, num_layers=1, model_dim=32, num_heads=2))
    save_graph(g, tmp_path / "g.json")
    assert nfn.main(["migrate-native", str(tmp_path / "g.json"), str(tmp_path / "out"), "--name", "gpt2", "--stop-tokens", "1,2"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["status"] == "ok" and out["model"]["family"] in ("gpt", "gpt2") and (tmp_path / "out" / "tensors.bin").is_file()


def test_native_adapter_and_objective_flags_reach_the_glimmer_config():
    """--runtime native --adapter-type qlora / --lora-dropout / --dpo-* become fields of the native Glimmer engine's configuration;
    other families and unknown adapter kinds are refused before anything is built."""
    from neuralfn_b200.cli import nfn as cli
    from neuralfn_b200.native_train import build_model_config

    def parse(*argv):
        return cli.build_parser().parse_args(["train", *argv])

    geom = ["--base-model", "muse-glimmer", "--n-layer", "2", "--d-model", "256", "--n-head", "4", "--n-kv-head", "2", "--head-dim", "64", "--d-ff", "512",
            "--vocab-size", "512", "--seq-len", "128"]
    a = parse(*geom, "--objective", "dpo", "--dpo-beta", "0.25", "--dpo-loss-type", "ipo", "--dpo-label-smoothing", "0.1",
              "--adapter-type", "qlora", "--lora-rank", "8", "--lora-alpha", "12", "--lora-dropout", "0.05", "--qlora-group-size", "32")
    cfg = build_model_config(cli._train_config(a))
    assert (cfg.lora_rank, cfg.lora_alpha, cfg.lora_dropout, cfg.base_quant, cfg.nf4_group) == (8, 12.0, 0.05, "nf4", 32)
    assert (cfg.dpo_beta, cfg.dpo_loss_type, cfg.dpo_label_smoothing) == (0.25, "ipo", 0.1)
    plain = build_model_config(cli._train_config(parse(*geom, "--adapter-type", "lora")))
    assert plain.lora_rank == 16 and plain.base_quant == "" and plain.lora_dropout == 0.0 and plain.dpo_loss_type == "sigmoid"
    with pytest.raises(ValueError):
        cli._train_config(parse("--base-model", "llama", "--adapter-type", "lora"))
    with pytest.raises(ValueError):
        cli._train_config(parse(*geom, "--adapter-type", "randmap"))
