"""``nfn`` command line: train / infer / inspect, one JSON document per invocation on stdout.

    nfn train --base-model gpt --template-name gpt2_qknorm --dataset fineweb10B --output-dir runs/a
    nfn train --base-model llama --n-layer 16 --d-model 1024 --n-head 16 --n-kv-head 4 --print-plan
    nfn train ... --gpus 8                  # re-launches itself under torchrun, one rank per GPU
    nfn infer --checkpoint runs/a/model_00020000.bin --prompt-tokens 15496,11,995 --max-new-tokens 64
    nfn inspect-checkpoint runs/a/model_00020000.bin
    nfn list-templates | nfn list-presets | nfn native-info | nfn dataset-info PATH

Help and the template listing import neither torch nor the kernel library, so they answer
instantly (the reference's dispatcher makes the same promise, ``cli/nfn.py:322-575``).
Flag names follow the reference's native trainer (``nfn_gpt2_native_train.cpp:1093-1198``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _add_train_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--base-model", default="gpt", help="gpt | gpt2 | gpt3 | nanogpt | llama | muse-glimmer | embedding")
    p.add_argument("--objective", choices=["ar", "sft", "dpo", "reward_model"], default="ar",
                   help="native engines: ar (all families); sft / dpo / reward_model from record shards (--base-model muse-glimmer)")
    p.add_argument("--head-dim", type=int, default=0, help="muse-glimmer: attention head width (0: d_model / n_head)")
    p.add_argument("--activation-checkpoint-interval", type=int, default=0,
                   help="muse-glimmer native engine: resident layers per recomputed segment (0: keep every activation)")
    p.add_argument("--dpo-label-smoothing", type=float, default=0.0, help="--objective dpo, sigmoid loss: weight of the flipped preference")
    p.add_argument("--init-from", default="", help="--objective sft|dpo: named checkpoint directory whose weights start the run")
    p.add_argument("--template-name", default="gpt2")
    p.add_argument("--dataset", default="", help="dataset alias, directory or shard file (empty: synthetic uniform tokens)")
    p.add_argument("--output-dir", default="")
    p.add_argument("--batch-size", type=int, default=64)
    p.add_argument("--seq-len", type=int, default=1024)
    p.add_argument("--train-batch-tokens", type=int, default=524288)
    p.add_argument("--n-layer", type=int, default=12)
    p.add_argument("--n-head", type=int, default=12)
    p.add_argument("--n-kv-head", type=int, default=0)
    p.add_argument("--d-model", type=int, default=768)
    p.add_argument("--d-ff", type=int, default=0)
    p.add_argument("--vocab-size", type=int, default=50257)
    p.add_argument("--learning-rate", type=float, default=6e-4)
    p.add_argument("--lr-schedule", default="cosine", choices=["cosine", "constant"])
    p.add_argument("--final-lr-fraction", type=float, default=0.0)
    p.add_argument("--warmup-steps", type=int, default=60)
    p.add_argument("--lr-schedule-total-steps", type=int, default=0)
    p.add_argument("--weight-decay", type=float, default=0.1)
    p.add_argument("--beta1", type=float, default=0.9)
    p.add_argument("--beta2", type=float, default=0.95)
    p.add_argument("--eps", type=float, default=1e-8)
    p.add_argument("--max-grad-norm", type=float, default=1.0)
    p.add_argument("--max-steps", type=int, default=20000)
    p.add_argument("--eval-every", type=int, default=5000)
    p.add_argument("--eval-batches", type=int, default=20)
    p.add_argument("--train-loss-every", type=int, default=250)
    p.add_argument("--progress-every", type=int, default=10)
    p.add_argument("--checkpoint-every", type=int, default=5000)
    p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--resume", action="store_true")
    p.add_argument("--no-cuda-graph", action="store_true")
    p.add_argument("--gpus", type=int, default=0, help="launch this many ranks on this node (0: stay in this process)")
    p.add_argument("--print-plan", "--dry-run", dest="print_plan", action="store_true")
    p.add_argument("--embedding-dataset", action="append", default=[], help="--base-model embedding: text file, one text per line (repeatable)")
    p.add_argument("--embedding-hidden-dim", type=int, default=128)
    p.add_argument("--embedding-output-dim", type=int, default=128)
    p.add_argument("--embedding-layers", type=int, default=2)
    p.add_argument("--embedding-heads", type=int, default=4)
    p.add_argument("--embedding-max-tokens", type=int, default=128)
    p.add_argument("--embedding-pooling", choices=["mean", "cls"], default="mean")
    p.add_argument("--parallel", choices=["dp", "tp", "ep"], default="dp",
                   help="dp: data parallel dense engines (default); tp: tensor-parallel Llama over --gpus ranks; ep: expert-parallel MoE Llama")
    p.add_argument("--tp-model", default="tiny", help="--parallel tp: llama3_8b | llama_1b | tiny")
    p.add_argument("--experts", type=int, default=8)
    p.add_argument("--top-k-experts", type=int, default=2)
    p.add_argument("--expert-hidden", type=int, default=1024)


def _train_config(a):
    from ..native_train import NativeTrainConfig
    return NativeTrainConfig(
        base_model=a.base_model, template_name=a.template_name, dataset=a.dataset, output_dir=a.output_dir, batch_size=a.batch_size,
        seq_len=a.seq_len, train_batch_tokens=a.train_batch_tokens, n_layer=a.n_layer, n_head=a.n_head, n_kv_head=a.n_kv_head,
        d_model=a.d_model, d_ff=a.d_ff, vocab_size=a.vocab_size, learning_rate=a.learning_rate, lr_schedule=a.lr_schedule,
        final_lr_fraction=a.final_lr_fraction, warmup_steps=a.warmup_steps, lr_schedule_total_steps=a.lr_schedule_total_steps,
        weight_decay=a.weight_decay, beta1=a.beta1, beta2=a.beta2, eps=a.eps, max_grad_norm=a.max_grad_norm, max_steps=a.max_steps,
        eval_every=a.eval_every, eval_batches=a.eval_batches, train_loss_every=a.train_loss_every, progress_every=a.progress_every,
        checkpoint_every=a.checkpoint_every, seed=a.seed, resume=a.resume, use_cuda_graph=not a.no_cuda_graph,
        objective=a.objective, head_dim=a.head_dim, activation_checkpoint_interval=a.activation_checkpoint_interval, extra_paths={"init_from": a.init_from} if a.init_from else {},
        extra={**_native_adapter_options(a), **_native_objective_options(a)})


def _native_objective_options(a) -> dict:
    """--objective dpo: the preference loss of the native Glimmer engine (sigmoid with optional label smoothing, hinge, IPO)."""
    if getattr(a, "objective", "ar") != "dpo":
        return {}
    out = {"dpo_label_smoothing": float(getattr(a, "dpo_label_smoothing", 0.0) or 0.0)}
    if getattr(a, "dpo_beta", None) is not None:
        out["dpo_beta"] = float(a.dpo_beta)
    if getattr(a, "dpo_loss_type", None):
        out["dpo_loss_type"] = a.dpo_loss_type
    return out


def _native_adapter_options(a) -> dict:
    """--runtime native --adapter-type lora | qlora: adapter geometry for the native Glimmer engine (other families adapt in the graph
    runtime). qlora keeps the frozen projection weights as NF4 (``--qlora-group-size``)."""
    kind = getattr(a, "adapter_type", None)
    if kind in (None, "none"):
        return {}
    if kind not in ("lora", "qlora") or a.base_model.lower().replace("_", "-") not in ("muse-glimmer", "glimmer"):
        raise ValueError("the native engines train LoRA / QLoRA adapters on --base-model muse-glimmer only; drop --runtime native for the others")
    out = {"lora_rank": int(getattr(a, "lora_rank", None) or 16)}
    if getattr(a, "lora_dropout", None):
        out["lora_dropout"] = float(a.lora_dropout)
    if kind == "qlora":
        out["base_quant"] = "nf4"
        if getattr(a, "qlora_group_size", None):
            out["nf4_group"] = int(a.qlora_group_size)
    if getattr(a, "lora_alpha", None) is not None:
        out["lora_alpha"] = float(a.lora_alpha)
    if getattr(a, "lora_targets", None):
        out["lora_targets"] = tuple(t.strip() for t in a.lora_targets.split(",") if t.strip())
    return out


def _parallel_train_argv(a) -> list[str]:
    argv = ["--parallel", a.parallel, "--dataset", a.dataset, "--batch-size", str(a.batch_size), "--seq-len", str(a.seq_len), "--max-steps", str(a.max_steps),
            "--learning-rate", str(a.learning_rate), "--warmup-steps", str(a.warmup_steps), "--weight-decay", str(a.weight_decay),
            "--max-grad-norm", str(a.max_grad_norm), "--progress-every", str(a.progress_every), "--checkpoint-every", str(a.checkpoint_every),
            "--output-dir", a.output_dir, "--seed", str(a.seed)]
    if a.resume:
        argv.append("--resume")
    if a.parallel == "tp":
        return argv + ["--model", a.tp_model]
    return argv + ["--n-layer", str(a.n_layer), "--n-head", str(a.n_head), "--n-kv-head", str(a.n_kv_head or a.n_head), "--d-model", str(a.d_model),
                   "--vocab-size", str(a.vocab_size), "--experts", str(a.experts), "--top-k", str(a.top_k_experts), "--expert-hidden", str(a.expert_hidden)]


def cmd_train_embedding(a) -> int:
    import torch
    from ..embedding import EmbeddingConfig, EmbeddingEncoder, EmbeddingTrainer, read_corpus, save_embedding_model
    if not a.embedding_dataset:
        raise ValueError("--base-model embedding needs at least one --embedding-dataset FILE")
    corpus = read_corpus(a.embedding_dataset)
    torch.manual_seed(a.seed)
    cfg = EmbeddingConfig(hidden_dim=a.embedding_hidden_dim, output_dim=a.embedding_output_dim, num_layers=a.embedding_layers,
                          num_heads=a.embedding_heads, max_tokens=a.embedding_max_tokens, pooling=a.embedding_pooling)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    model = EmbeddingEncoder(cfg).to(dev)
    lr = a.learning_rate if a.learning_rate != 6e-4 else 1e-3
    trainer = EmbeddingTrainer(model, learning_rate=lr, weight_decay=a.weight_decay, warmup_steps=min(a.warmup_steps, max(1, a.max_steps // 10)),
                               max_steps=a.max_steps, grad_clip=a.max_grad_norm, seed=a.seed)

    def on_step(step, rec):
        if a.progress_every and step % a.progress_every == 0:
            print(json.dumps({"event": "train_step", "step": step, "loss": rec["total"], "mlm": rec["mlm"], "contrastive": rec["contrastive"]}), flush=True)

    hist = trainer.train(corpus, batch_size=a.batch_size, on_step=on_step)
    out = a.output_dir or "artifacts/embedding"
    save_embedding_model(model, out, trainer)
    print(json.dumps({"event": "complete", "status": "ok", "steps": len(hist), "first_loss": hist[0]["total"], "final_loss": hist[-1]["total"],
                      "texts": len(corpus), "output_dir": out}))
    return 0


def cmd_embed(a) -> int:
    from ..embedding import load_embedding_model, read_corpus
    if (a.text is None) == (a.input is None):
        raise ValueError("nfn embed needs exactly one of --text or --input")
    texts = [a.text] if a.text is not None else read_corpus([a.input])
    vecs = load_embedding_model(a.checkpoint).embed(texts)
    print(json.dumps({"dim": int(vecs.shape[1]), "embeddings": [[round(float(x), 6) for x in v] for v in vecs]}))
    return 0


def cmd_train(a) -> int:
    if a.base_model == "embedding":
        return cmd_train_embedding(a)
    from . import graph_cli
    if graph_cli.wants_graph_runtime(a):
        return graph_cli.cmd_train_graph(a)
    if getattr(a, "pipeline_parallel_size", 1) > 1:
        # pipeline stages: one process per GPU through the pipeline driver
        import subprocess
        argv = ["--stages", str(a.pipeline_parallel_size), "--dataset", a.dataset, "--batch-size", str(a.batch_size), "--seq-len", str(a.seq_len),
                "--max-steps", str(a.max_steps), "--learning-rate", str(a.learning_rate), "--n-layer", str(a.n_layer), "--n-head", str(a.n_head),
                "--d-model", str(a.d_model), "--vocab-size", str(a.vocab_size), "--seed", str(a.seed), "--output-dir", a.output_dir,
                "--base-model", "muse-glimmer" if a.base_model.lower().replace("_", "-") in ("muse-glimmer", "glimmer") else "llama",
                "--head-dim", str(a.head_dim), "--n-kv-head", str(a.n_kv_head), "--d-ff", str(a.d_ff)]
        if "RANK" in os.environ:
            from ..parallel.pp import main as pp_main
            return pp_main(argv)
        return subprocess.call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.pipeline_parallel_size}",
                                "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), "-m",
                                "neuralfn_b200.parallel.pp", *argv])
    if a.parallel in ("tp", "ep"):
        # the model-parallel families have their own driver; one process per GPU
        argv = _parallel_train_argv(a)
        if a.gpus > 1 and "RANK" not in os.environ:
            import subprocess
            return subprocess.call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr",
                                    "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), "-m", "neuralfn_b200.parallel.train", *argv])
        from ..parallel.train import main as parallel_main
        return parallel_main(argv)
    if a.print_plan:
        from ..native_train import training_plan
        print(json.dumps({"status": "plan", **training_plan(_train_config(a), max(1, a.gpus))}, indent=2))
        return 0
    if a.gpus > 1 and "RANK" not in os.environ:
        # one process per GPU: hand the same command line to the torch launcher
        import subprocess
        argv, skip = [], False
        for x in sys.argv[1:]:
            if skip:
                skip = False
            elif x == "--gpus":
                skip = True
            elif not x.startswith("--gpus="):
                argv.append(x)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", str(29500 + os.getpid() % 2000), "-m", "neuralfn_b200.cli.nfn", *argv]
        return subprocess.call(cmd)
    cfg = _train_config(a)
    from ..native_train import run_native_training
    report = run_native_training(cfg)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(report, default=str))
    return 0


def _infer_artifact(a) -> int:
    """Artifact directory: serve it over HTTP, or generate once with the session API."""
    if a.serve:
        from ..serving.openai_server import run_server
        run_server(a.checkpoint, host=a.host, port=a.port, api_key_file=a.api_key_file,
                   allow_unauthenticated_remote=a.allow_unauthenticated_remote, sessions=a.max_batch, state_db=a.state_db)
        return 0
    from ..serving import GenerationConfig, NativeInferenceModel, NativeModelLoadConfig, NGramProposer
    model = NativeInferenceModel.load(a.checkpoint, NativeModelLoadConfig(session_count=1, speculative_decoding=a.speculative_decoding))
    if getattr(a, "companion_checkpoint", ""):
        model.attach_dflash(a.companion_checkpoint)                    # a DFlash assistant exported by the distillation trainer
    if a.chat:
        from ..serving.chat import resolve_chat_renderer
        from .tui import InferTUI
        rc = InferTUI(model, resolve_chat_renderer(model.manifest.get("chat_template")), max_new_tokens=a.max_new_tokens,
                      proposer_factory=(NGramProposer if a.speculative_decoding != "off" else None)).run()
        model.close()
        return rc
    ids = model.codec.encode(a.prompt) if a.prompt is not None else [int(t) for t in a.prompt_tokens.split(",") if t]
    with model.create_session(a.seed) as s:
        s.prefill(ids)
        cfg = GenerationConfig(max_new_tokens=a.max_new_tokens, temperature=a.temperature, top_k=a.top_k or None, top_p=a.top_p, seed=a.seed,
                               stop_token_ids=tuple(model.manifest.get("stop_token_ids", ())))
        fallback = NGramProposer() if a.speculative_decoding != "off" and not getattr(a, "companion_checkpoint", "") else None
        res = s.decode(cfg, proposer=fallback)
    print(json.dumps({"status": "ok", "text": res.text, "token_ids": list(res.token_ids), "finish_reason": res.finish_reason,
                      "prompt_tokens": res.prompt_tokens, "speculative": {"proposed": res.speculative_proposed_tokens,
                                                                          "accepted": res.speculative_accepted_tokens}, "stats": model.stats()}))
    model.close()
    return 0


def cmd_infer(a) -> int:
    import os
    if os.path.isdir(a.checkpoint):
        return _infer_artifact(a)
    if a.serve:
        raise SystemExit("--serve needs an artifact directory (see neuralfn_b200.serving.write_artifact)")
    if not a.prompt_tokens:
        raise SystemExit("--prompt-tokens is required for a dense checkpoint file")
    from ..checkpoint import read_dense_model
    from ..serving import EngineConfig, ResidentEngine, Sampling
    cfg, tensors, sha = read_dense_model(a.checkpoint)
    activation = None
    moa = a.checkpoint[:-4] + ".moa.json" if a.checkpoint.endswith(".bin") else ""
    if moa and os.path.exists(moa):
        # a mixture-of-activations run: generate with the activation that was in effect when the file was written
        import re
        from ..checkpoint.dense import read_moa_sidecar
        step = int(re.search(r"model_(\d+)\.bin$", a.checkpoint).group(1))
        activation = read_moa_sidecar(os.path.dirname(a.checkpoint) or ".", step)["selection"]["activation"]
    eng = ResidentEngine(EngineConfig.gpt2(cfg, max_batch=a.max_batch, activation=activation))
    eng.load_named_tensors(tensors)
    prompts = [[int(t) for t in p.split(",") if t] for p in a.prompt_tokens.split(";")]
    out = eng.generate(prompts, max_new_tokens=a.max_new_tokens,
                       sampling=Sampling(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, seed=a.seed),
                       eos_token=a.eos_token if a.eos_token >= 0 else None)
    print(json.dumps({"status": "ok", "checkpoint_sha256": sha, "prompts": prompts, "generated": out, "mlp_activation": activation or "gelu",
                      "device_bytes": eng.device_bytes, "kernel_launches": eng.launches}))
    return 0


def cmd_inspect(a) -> int:
    from ..checkpoint import inspect_dense_model
    info = inspect_dense_model(a.path)
    info.pop("config", None)
    from ..data._rt import sha256_file
    info["sha256"] = sha256_file(a.path)
    print(json.dumps({"status": "ok", **info}, indent=2))
    return 0


def cmd_checkpoint_layout(a) -> int:
    from ..native_train import build_model_config
    cfg = build_model_config(_train_config(a))
    off, rows = 1024, []
    for s in cfg.param_specs():
        rows.append({"name": s.name, "shape": list(s.shape), "offset": off, "nbytes": 2 * s.numel, "weight_decay": s.decay})
        off += 2 * s.numel
    print(json.dumps({"status": "ok", "header_bytes": 1024, "file_bytes": off, "tensors": rows}, indent=2))
    return 0


def cmd_kernels(_a) -> int:
    from ..ops.registry import coverage_report, coverage_summary
    print(json.dumps({"summary": coverage_summary(), "kernels": coverage_report()}, indent=2))
    return 0


def cmd_families(_a) -> int:
    from ..native_registry import capability_proof_for, native_families_report
    rows = native_families_report()
    for r in rows:
        p = capability_proof_for(r["family"])
        r["native_training"], r["native_inference"], r["reasons"] = p.native_training, p.native_inference, list(p.reasons)
    print(json.dumps(rows, indent=2))
    return 0


def cmd_list_templates(_a) -> int:
    from ..native_templates import GPT_VARIANTS, LLAMA_TEMPLATES
    print(json.dumps({"gpt": list(GPT_VARIANTS), "llama": list(LLAMA_TEMPLATES)}, indent=2))
    return 0


def cmd_list_presets(_a) -> int:
    from ..presets import PRESET_BUILDERS
    print(json.dumps(sorted(PRESET_BUILDERS), indent=2))
    return 0


def cmd_native_info(_a) -> int:
    from ..ops import _lib
    info = {"kernel_library": str(_lib.lib_path()), "kernel_library_present": _lib.available(), "target": "sm_100a",
            "native_families": ["gpt", "gpt2", "gpt3", "nanogpt", "llama"],
            "fused_collectives": ["dp_reduce_adamw", "ag_gemm", "gemm_rs", "allreduce_resid_norm"]}
    try:
        import torch
        info["cuda_available"] = bool(torch.cuda.is_available())
        if torch.cuda.is_available():
            info["device"] = torch.cuda.get_device_name(0)
            info["device_count"] = torch.cuda.device_count()
    except Exception as exc:  # pragma: no cover - torch is a hard dependency elsewhere
        info["torch_error"] = str(exc)
    print(json.dumps(info, indent=2))
    return 0


def cmd_dataset_info(a) -> int:
    from ..data import TokenDataset
    ds = TokenDataset(a.path, allow_train_as_val=True)
    print(json.dumps(ds.describe(a.seq_len, a.batch_size, a.train_batch_tokens), indent=2))
    return 0


def cmd_compat_train(a) -> int:
    from ..native_train import NativeTrainConfig, run_native_training, training_plan
    from .compat import translate_llmc_args
    rest = [x for x in a.rest if x != "--"]
    kw, notes = translate_llmc_args(rest)
    cfg = NativeTrainConfig(**kw)
    if a.print_plan:
        print(json.dumps({"status": "plan", **notes, **training_plan(cfg, 1)}, indent=2))
        return 0
    report = run_native_training(cfg)
    print(json.dumps({**report, **notes}, default=str))
    return 0


def cmd_infer_tp(a) -> int:
    """Greedy / sampled generation with the tensor-parallel decoder from a Hugging Face Llama directory."""
    if a.gpus > 1 and "RANK" not in os.environ:
        import subprocess
        argv = [x for i, x in enumerate(sys.argv[1:]) if x != "--gpus" and (i == 0 or sys.argv[i] != "--gpus") and not x.startswith("--gpus=")]
        return subprocess.call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr", "127.0.0.1",
                                "--master-port", str(29500 + os.getpid() % 2000), "-m", "neuralfn_b200.cli.nfn", *argv])
    import torch
    import torch.distributed as dist
    from ..parallel.tp import TensorParallelContext
    from ..serving.tp_decode import TPLlamaDecoder
    cuda = torch.cuda.is_available() and not a.cpu
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if cuda else "gloo")
    prompts = [[int(t) for t in p.split(",") if t] for p in a.prompt_tokens.split(";") if p]
    if not prompts or len({len(p) for p in prompts}) != 1:
        raise ValueError("--prompt-tokens wants one or more ';'-separated prompts of the same length")
    need = len(prompts) * len(prompts[0])
    if need % world:
        raise ValueError(f"rows x prompt length = {need} must divide by the number of ranks ({world})")
    dec = TPLlamaDecoder.from_hf_directory(a.hf_dir, TensorParallelContext(dev), max_batch=len(prompts), max_seq=len(prompts[0]) + a.max_new_tokens + 8,
                                           use_graph=cuda and a.temperature <= 0)
    dec.set_sampling(a.temperature, a.top_k, a.top_p, a.seed)
    out = dec.generate(torch.tensor(prompts, device=dev), a.max_new_tokens).cpu().tolist()
    dec.close()
    if rank == 0:
        print(json.dumps({"status": "ok", "world_size": world, "generated": out}))
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


def cmd_migrate_native(a) -> int:
    from ..native_ir import migrate_graph_to_native
    man = migrate_graph_to_native(a.graph, a.out_dir, model_name=a.name or None, stop_token_ids=[int(x) for x in a.stop_tokens.split(",") if x])
    print(json.dumps({"status": "ok", "out_dir": a.out_dir, "model": man["model"], "capabilities": man["capabilities"],
                      "tensor_bytes": man["tensors"]["total_bytes"]}, indent=2))
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="nfn", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    t = sub.add_parser("train", help="training run (JSON report on stdout): native sm_100a engines, or the graph runtime for any preset / objective")
    _add_train_flags(t)
    from . import graph_cli
    graph_cli.add_graph_train_arguments(t)
    t.set_defaults(fn=cmd_train)
    ev = sub.add_parser("eval", help="validation loss and prompt probes of a graph trained with the graph runtime")
    graph_cli.add_eval_arguments(ev)
    ev.set_defaults(fn=graph_cli.cmd_eval)
    mig = sub.add_parser("migrate", help="lower a graph (and weights) to a native execution artifact: nfn migrate graph-to-native --graph G --output-dir D")
    graph_cli.add_migrate_arguments(mig)
    mig.set_defaults(fn=graph_cli.cmd_migrate)
    i = sub.add_parser("infer", help="generate from a dense checkpoint file or an artifact directory; --serve starts the HTTP server")
    i.add_argument("--checkpoint", required=True)
    i.add_argument("--prompt-tokens", default="", help="comma-separated ids; ';' separates prompts")
    i.add_argument("--prompt", default=None, help="text prompt (artifact directories with a text codec)")
    i.add_argument("--serve", action="store_true", help="serve the artifact over the OpenAI-compatible HTTP API")
    i.add_argument("--chat", action="store_true", help="interactive chat loop (/show /reset /mode /tokens /quit)")
    i.add_argument("--host", default="127.0.0.1")
    i.add_argument("--port", type=int, default=8000)
    i.add_argument("--api-key-file", default=None)
    i.add_argument("--allow-unauthenticated-remote", action="store_true")
    i.add_argument("--state-db", default=None, help="SQLite file behind /v1/responses and /v1/conversations")
    i.add_argument("--speculative-decoding", choices=["off", "auto", "required"], default="auto")
    i.add_argument("--companion-checkpoint", default="", help="artifact directories: DFlash assistant file (block-diffusion draft on the engine's hidden-state taps)")
    i.add_argument("--max-new-tokens", type=int, default=144)
    i.add_argument("--temperature", type=float, default=0.0)
    i.add_argument("--top-k", type=int, default=0)
    i.add_argument("--top-p", type=float, default=1.0)
    i.add_argument("--seed", type=int, default=1337)
    i.add_argument("--eos-token", type=int, default=-1)
    i.add_argument("--max-batch", type=int, default=8)
    i.set_defaults(fn=cmd_infer)
    c = sub.add_parser("inspect-checkpoint", help="validate and checksum a dense checkpoint")
    c.add_argument("path")
    c.set_defaults(fn=cmd_inspect)
    lay = sub.add_parser("checkpoint-layout", help="tensor table of the checkpoint a configuration would write")
    _add_train_flags(lay)
    lay.set_defaults(fn=cmd_checkpoint_layout)
    sub.add_parser("list-templates").set_defaults(fn=cmd_list_templates)
    sub.add_parser("list-presets").set_defaults(fn=cmd_list_presets)
    sub.add_parser("native-info").set_defaults(fn=cmd_native_info)
    sub.add_parser("kernels", help="kernel catalogue and coverage of the built library").set_defaults(fn=cmd_kernels)
    sub.add_parser("families", help="model families, their execution routes and capability proofs").set_defaults(fn=cmd_families)
    it = sub.add_parser("infer-tp", help="tensor-parallel generation from a Hugging Face Llama directory (one rank per GPU with --gpus N)")
    it.add_argument("--hf-dir", required=True)
    it.add_argument("--prompt-tokens", required=True, help="comma-separated ids; ';' separates equally long prompts")
    it.add_argument("--max-new-tokens", type=int, default=32)
    it.add_argument("--temperature", type=float, default=0.0)
    it.add_argument("--top-k", type=int, default=0)
    it.add_argument("--top-p", type=float, default=1.0)
    it.add_argument("--seed", type=int, default=0)
    it.add_argument("--gpus", type=int, default=0)
    it.add_argument("--cpu", action="store_true", help="run on CPU ranks (PyTorch fallbacks)")
    it.set_defaults(fn=cmd_infer_tp)
    em = sub.add_parser("embed", help="unit-length text vectors from an embedding model directory")
    em.add_argument("--checkpoint", required=True)
    em.add_argument("--text", default=None)
    em.add_argument("--input", default=None, help="file with one text per line")
    em.set_defaults(fn=cmd_embed)
    ct = sub.add_parser("compat-train", help="run a train_gpt2cu (llm.c) command line: nfn compat-train -- -i data -o out -e d12 -b 64 -t 1024")
    ct.add_argument("--print-plan", action="store_true")
    ct.add_argument("rest", nargs=argparse.REMAINDER)
    ct.set_defaults(fn=cmd_compat_train)
    mg = sub.add_parser("migrate-native", help="lower a graph JSON file into a native execution manifest + raw tensor bundle")
    mg.add_argument("graph")
    mg.add_argument("out_dir")
    mg.add_argument("--name", default="")
    mg.add_argument("--stop-tokens", default="")
    mg.set_defaults(fn=cmd_migrate_native)
    d = sub.add_parser("dataset-info")
    d.add_argument("path")
    d.add_argument("--seq-len", type=int, default=1024)
    d.add_argument("--batch-size", type=int, default=64)
    d.add_argument("--train-batch-tokens", type=int, default=524288)
    d.set_defaults(fn=cmd_dataset_info)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    try:
        return int(args.fn(args) or 0)
    except Exception as exc:
        print(json.dumps({"status": "error", "error": f"{type(exc).__name__}: {exc}"}))
        return 1


if __name__ == "__main__":
    raise SystemExit(main())
