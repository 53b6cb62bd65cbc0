"""Graph-runtime commands of the ``nfn`` CLI: recipe-driven training of any preset / objective through
the tensor runtime (``nfn train --runtime torch``), ``nfn eval`` and ``nfn migrate``.

Flag names follow the reference CLI (``cli/nfn_impl.py:906-1176``: recipe, fine-tuning, optimizer and
evolutionary groups; ``:5289`` eval; ``cli/nfn.py:546`` migrate) so its command lines keep working.
Artifacts: ``<output>.json`` graph, ``<output>`` weights (``.pt``), ``<output>.report.json``.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import time
from pathlib import Path
from typing import Any

TRAINING_MODES = ("pretrain", "sft", "dpo", "ppo", "reward_model")
ADAPTERS = ("none", "lora", "qlora", "randmap")

# flags whose presence on an ``nfn train`` command line selects the graph runtime
GRAPH_ONLY_FLAGS = ("training_mode", "adapter_type", "lora_rank", "lora_alpha", "lora_dropout", "lora_targets", "base_checkpoint",
                    "ref_checkpoint", "reward_checkpoint", "dpo_beta", "dpo_loss_type", "kl_coef", "ppo_clip", "ppo_vf_coef",
                    "ppo_ent_coef", "rollout_length", "ppo_epochs_per_rollout", "evolutionary", "optimizer_profile", "topology",
                    "router_mode", "use_jepa", "preset", "activation_checkpointing", "fsdp2")


def add_graph_train_arguments(p: argparse.ArgumentParser) -> None:
    r = p.add_argument_group("Recipe (graph runtime)")
    r.add_argument("--runtime", choices=("auto", "native", "torch"), default="auto",
                   help="native: the sm_100a engines; torch: the graph runtime; auto: native unless a graph-only flag is given")
    r.add_argument("--preset", default=None, help="preset name (nfn list-presets); overrides --topology/--router-mode/--jepa")
    r.add_argument("--topology", choices=("dense", "moe", "semantic_router"), default=None)
    r.add_argument("--router-mode", choices=("none", "standard", "semantic"), default=None)
    r.add_argument("--jepa", action="store_true", dest="use_jepa", default=None)
    r.add_argument("--megakernel", action="store_true", default=None)
    r.add_argument("--output", default=None, help="weights artifact path (graph JSON and report are written beside it)")
    r.add_argument("--device", default=None, help="cuda | cpu (default: cuda when available)")
    r.add_argument("--amp-dtype", choices=("float32", "bfloat16", "float16"), default=None)
    r.add_argument("--epochs", type=int, default=None)
    r.add_argument("--train-rows", type=int, default=None, help="rows of seq-len tokens to draw from the dataset (default 2048)")
    r.add_argument("--activation-checkpointing", action="store_true", default=None)
    r.add_argument("--fsdp2", action="store_true", default=None, help="shard optimizer state over the data-parallel ranks")
    r.add_argument("--pipeline-parallel-size", type=int, default=1,
                   help="pipeline stages (one process per GPU); handled by the native pipeline driver")
    ft = p.add_argument_group("Fine-tuning")
    ft.add_argument("--training-mode", choices=TRAINING_MODES, default=None)
    ft.add_argument("--adapter-type", choices=ADAPTERS, default=None)
    ft.add_argument("--lora-rank", type=int, default=None)
    ft.add_argument("--lora-alpha", type=float, default=None)
    ft.add_argument("--lora-dropout", type=float, default=None)
    ft.add_argument("--lora-targets", default=None, help="comma-separated projection names, e.g. q_proj,v_proj")
    ft.add_argument("--lora-bias", action="store_true", default=None)
    ft.add_argument("--qlora-group-size", type=int, default=None)
    ft.add_argument("--qlora-compute-dtype", default=None)
    ft.add_argument("--base-checkpoint", default=None)
    ft.add_argument("--ref-checkpoint", default=None)
    ft.add_argument("--ref-graph", default=None, help="graph JSON of the frozen reference (default: the .json beside --ref-checkpoint)")
    ft.add_argument("--reward-checkpoint", default=None)
    ft.add_argument("--reward-graph", default=None, help="graph JSON of the reward model (default: the .json beside --reward-checkpoint)")
    ft.add_argument("--adapter-only-save", action="store_true", default=None)
    ft.add_argument("--dpo-beta", type=float, default=None)
    ft.add_argument("--dpo-loss-type", choices=("sigmoid", "hinge", "ipo"), default=None)
    ft.add_argument("--kl-coef", type=float, default=None)
    ft.add_argument("--ppo-clip", type=float, default=None)
    ft.add_argument("--ppo-vf-coef", type=float, default=None)
    ft.add_argument("--ppo-ent-coef", type=float, default=None)
    ft.add_argument("--rollout-length", type=int, default=None)
    ft.add_argument("--ppo-epochs-per-rollout", type=int, default=None)
    o = p.add_argument_group("Optimizer (graph runtime)")
    o.add_argument("--optimizer-profile", default=None, help="adamw | muon_adamw | parameter_golf (see TorchTrainConfig)")
    for name in ("embed-lr", "head-lr", "tied-embed-lr", "matrix-lr", "scalar-lr", "min-lr", "muon-momentum",
                 "muon-momentum-warmup-start", "ema-decay", "ar-loss-coef", "jepa-loss-coef", "semantic-align-loss-coef",
                 "max-wallclock-seconds"):
        o.add_argument(f"--{name}", type=float, default=None)
    for name in ("lr-decay-iters", "muon-backend-steps", "muon-momentum-warmup-steps"):
        o.add_argument(f"--{name}", type=int, default=None)
    e = p.add_argument_group("Evolutionary search")
    e.add_argument("--evolutionary", action="store_true", default=None)
    e.add_argument("--evo-population-size", type=int, default=None)
    e.add_argument("--evo-mutation-rate", type=float, default=None)
    e.add_argument("--evo-mutation-scale", type=float, default=None)
    e.add_argument("--evo-crossover-rate", type=float, default=None)
    e.add_argument("--evo-tournament-size", type=int, default=None)
    e.add_argument("--evo-elite-count", type=int, default=None)
    e.add_argument("--evo-seed", type=int, default=None)


def wants_graph_runtime(a) -> bool:
    if getattr(a, "runtime", "auto") == "torch":
        return True
    if getattr(a, "runtime", "auto") == "native":
        return False
    return any(getattr(a, f, None) not in (None, False) for f in GRAPH_ONLY_FLAGS)


# ---------------------------------------------------------------------------- spec --
def build_spec_from_args(a):
    """ModelSpec from the recipe flags: a named preset, or the composition of base model, topology,
    router mode and JEPA; then the fine-tuning and loss-coefficient overrides."""
    from .. import presets
    from ..config import FineTuneSpec
    geometry = dict(vocab_size=a.vocab_size, num_layers=a.n_layer, model_dim=a.d_model, num_heads=a.n_head)
    if a.n_kv_head:
        geometry["num_kv_heads"] = a.n_kv_head
    base = {"gpt": "gpt2", "gpt3": "gpt2"}.get(a.base_model, a.base_model)
    if a.preset:
        spec = presets.build_preset(a.preset, **geometry)
    elif a.topology or a.router_mode or a.use_jepa:
        topology = a.topology or "dense"
        router = a.router_mode or ("semantic" if topology == "semantic_router" else ("standard" if topology == "moe" else "none"))
        spec = presets.build_composed_lm_spec(base_model=base if base in ("gpt2", "nanogpt", "llama") else "llama",
                                              moe=topology in ("moe", "semantic_router"), router_mode=router,
                                              use_jepa=bool(a.use_jepa), **geometry)
    else:
        name = a.template_name if a.template_name in presets.preset_names() else base
        spec = presets.build_preset(name, **geometry)
    if a.megakernel:
        spec.template.runtime = "megakernel"
    bs = spec.block_spec
    if a.adapter_type and a.adapter_type != "none":
        bs.adapter_type = a.adapter_type
        spec.template.adapter = a.adapter_type
        if a.adapter_type == "randmap" and not bs.adapter_dim:
            bs.adapter_dim = max(8, spec.model_dim // 8)
    for flag, field in (("lora_rank", "lora_rank"), ("lora_alpha", "lora_alpha"), ("lora_dropout", "lora_dropout"),
                        ("qlora_group_size", "qlora_group_size"), ("qlora_compute_dtype", "qlora_compute_dtype")):
        if getattr(a, flag, None) is not None:
            setattr(bs, field, getattr(a, flag))
    if a.lora_targets:
        bs.lora_targets = tuple(t.strip() for t in a.lora_targets.split(",") if t.strip())
    for flag in ("ema_decay", "ar_loss_coef", "jepa_loss_coef", "semantic_align_loss_coef"):
        if getattr(a, flag, None) is not None:
            setattr(spec, flag, getattr(a, flag))
    mode = a.training_mode or "pretrain"
    if mode != "pretrain" or a.base_checkpoint or (a.adapter_type and a.adapter_type != "none"):
        kw: dict[str, Any] = {"objective": mode}
        for flag, field in (("base_checkpoint", "base_checkpoint"), ("ref_checkpoint", "ref_checkpoint"),
                            ("reward_checkpoint", "reward_checkpoint"), ("dpo_beta", "beta"), ("dpo_loss_type", "dpo_loss_type"),
                            ("kl_coef", "kl_coef"), ("ppo_clip", "ppo_clip"), ("ppo_vf_coef", "ppo_vf_coef"),
                            ("ppo_ent_coef", "ppo_ent_coef"), ("rollout_length", "rollout_length"),
                            ("ppo_epochs_per_rollout", "ppo_epochs_per_rollout"), ("adapter_only_save", "adapter_only_save")):
            v = getattr(a, flag, None)
            if v is not None and field in FineTuneSpec.__dataclass_fields__:
                kw[field] = v
        # a frozen model is a (graph, weights) pair; training runs write the graph beside the weights
        for ckpt, flag, field in (("ref_checkpoint", "ref_graph", "ref_graph_path"), ("reward_checkpoint", "reward_graph", "reward_graph_path")):
            if field not in FineTuneSpec.__dataclass_fields__:
                continue
            if getattr(a, flag, None):
                kw[field] = getattr(a, flag)
            elif kw.get(ckpt) and Path(kw[ckpt]).with_suffix(".json").exists():
                kw[field] = str(Path(kw[ckpt]).with_suffix(".json"))
        spec.finetune = FineTuneSpec(**kw)
    return spec


def train_config_from_args(a, device: str):
    from ..tensor.trainer import TorchTrainConfig
    c = TorchTrainConfig(learning_rate=a.learning_rate, batch_size=a.batch_size, weight_decay=a.weight_decay, beta1=a.beta1, beta2=a.beta2,
                         adam_eps=a.eps, device=device, max_steps=a.max_steps, grad_clip_norm=a.max_grad_norm,
                         warmup_steps=a.warmup_steps, seed=a.seed, epochs=a.epochs or 1_000_000)
    if a.train_batch_tokens and a.train_batch_tokens < 524288:      # the native default means "not given"
        c.train_batch_tokens = a.train_batch_tokens
    direct = {"amp_dtype": "amp_dtype", "optimizer_profile": "optimizer_profile", "embed_lr": "embed_lr", "head_lr": "head_lr",
              "tied_embed_lr": "tied_embed_lr", "matrix_lr": "matrix_lr", "scalar_lr": "scalar_lr", "min_lr": "min_lr",
              "lr_decay_iters": "lr_decay_iters", "muon_momentum": "muon_momentum", "muon_backend_steps": "muon_backend_steps",
              "muon_momentum_warmup_start": "muon_momentum_warmup_start", "muon_momentum_warmup_steps": "muon_momentum_warmup_steps",
              "max_wallclock_seconds": "max_wallclock_seconds", "evolutionary": "evolutionary",
              "evo_population_size": "evo_population_size", "evo_mutation_rate": "evo_mutation_rate",
              "evo_mutation_scale": "evo_mutation_scale", "evo_crossover_rate": "evo_crossover_rate",
              "evo_tournament_size": "evo_tournament_size", "evo_elite_count": "evo_elite_count", "evo_seed": "evo_seed",
              "activation_checkpointing": "activation_checkpointing", "fsdp2": "fsdp2_enabled"}
    for flag, field in direct.items():
        v = getattr(a, flag, None)
        if v is not None:
            setattr(c, field, v)
    return c


# ---------------------------------------------------------------------------- data --
def load_token_rows(dataset: str, seq_len: int, rows: int, vocab_size: int, seed: int, split: str = "train"):
    """``rows`` x (seq_len + 1) int64 tokens: sequential windows of a token dataset (alias, directory
    or shard file), or uniform random ids when ``dataset`` is empty."""
    import torch
    if not dataset:
        g = torch.Generator().manual_seed(seed + (0 if split == "train" else 1))
        return torch.randint(0, vocab_size, (rows, seq_len + 1), generator=g), "synthetic uniform-random token ids"
    from ..data.shards import TokenDataset
    ds = TokenDataset(dataset, allow_train_as_val=True, require_validation=False)
    try:
        sampler = ds.sampler(split, seq_len, 1)
        out = torch.empty(rows, seq_len + 1, dtype=torch.long)
        n = 0
        for tok, tgt in sampler:
            out[n, :seq_len] = tok.reshape(-1)
            out[n, seq_len] = tgt.reshape(-1)[-1]
            n += 1
            if n >= rows:
                break
        sampler.close()
        if n == 0:
            raise ValueError(f"dataset {dataset!r} holds fewer than {seq_len + 1} tokens in split {split!r}")
        return out[:n], f"{dataset} ({split}, {n} rows)"
    finally:
        ds.close()


def _objective_inputs(graph, rows):
    """Training tensors for the root graph's inputs, by input name."""
    names = [graph.nodes[n].neuron_def.output_ports[0].name for n in graph.input_node_ids]
    x, y = rows[:, :-1], rows[:, 1:]
    table = {"tokens": x, "target_ids": y, "targets": y, "enc_tokens": x, "dec_tokens": x}
    out = {}
    for n in names:
        if n == "sem_targets":
            break                      # derived by the trainer from the tokens
        if n not in table:
            raise ValueError(f"objective input {n!r} needs a structured dataset; use the records pipeline (nfn dataset-info)")
        out[n] = table[n]
    return out, names


# ------------------------------------------------------------------------ commands --
def cmd_train_graph(a) -> int:
    import torch
    from ..inference import export_to_pt, save_adapter_checkpoint
    from ..serialization import save_graph
    from ..tensor.trainer import TorchTrainer
    from ..torch_templates import build_gpt_root_graph
    device = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    spec = build_spec_from_args(a)
    graph = build_gpt_root_graph(spec)
    graph.torch_config["device"] = device
    cfg = train_config_from_args(a, device)
    mode = spec.finetune.objective if spec.finetune is not None else "pretrain"
    plan = {"runtime": "torch", "objective": spec.template.objective, "training_mode": mode, "backbone": spec.template.backbone,
            "adapter": spec.block_spec.adapter_type, "optimization": "evolutionary" if cfg.evolutionary else "gradient",
            "optimizer_profile": cfg.optimizer_profile, "device": device, "nodes": len(graph.nodes),
            "inputs": [graph.nodes[n].neuron_def.output_ports[0].name for n in graph.input_node_ids]}
    if a.print_plan:
        print(json.dumps({"status": "plan", **plan}, indent=2))
        return 0
    if mode in ("dpo", "ppo", "reward_model", "sft") and not a.dataset:
        raise ValueError(f"--training-mode {mode} needs --dataset with structured records")
    if mode != "pretrain":
        return _train_post(a, spec, graph, cfg, plan, device)
    rows, data_note = load_token_rows(a.dataset, a.seq_len, a.train_rows or 2048, spec.vocab_size, a.seed)
    inputs, _names = _objective_inputs(graph, rows)
    trainer = TorchTrainer(graph, cfg)
    t0 = time.perf_counter()
    steps: list[dict] = []

    def on_step(info):
        steps.append(info)
        if a.progress_every and info["step"] % a.progress_every == 0:
            print(json.dumps({"event": "train_step", "step": info["step"], "loss": round(info["loss"], 6),
                              "method": info["optimization_method"], "lr": (info["learning_rates"] or [None])[0]}), flush=True)

    trainer.train(inputs, on_step=on_step)
    out = Path(a.output or (Path(a.output_dir or "artifacts/graph-run") / "model.pt"))
    out.parent.mkdir(parents=True, exist_ok=True)
    save_graph(graph, out.with_suffix(".json"))
    if getattr(a, "adapter_only_save", None) and spec.block_spec.adapter_type != "none":
        save_adapter_checkpoint(trainer.compiled, out)
    else:
        export_to_pt(trainer.compiled, out, metadata={"template_spec": spec.to_dict(), "steps": trainer.global_step})
    report = {"event": "complete", "status": "ok", **plan, "data": data_note, "steps": trainer.global_step,
              "first_loss": steps[0]["loss"] if steps else None, "final_loss": steps[-1]["loss"] if steps else None,
              "wall_seconds": round(time.perf_counter() - t0, 3), "graph": str(out.with_suffix(".json")), "weights": str(out)}
    for key in ("route_evo", "layer_evo", "routing_stats"):
        if steps and key in steps[-1]:
            report[key] = steps[-1][key]
    out.with_suffix(".report.json").write_text(json.dumps(report, indent=2, default=str))
    print(json.dumps(report, default=str))
    return 0


def _read_records(dataset: str, kind: str, rows: int) -> dict:
    """Up to ``rows`` records of a structured dataset as stacked tensors (keys as ``RecordReader.next``)."""
    import torch
    from ..data.shards import RecordReader
    rd = RecordReader(dataset, kind, "train", batch_size=1, allow_train_as_val=True)
    cols: dict[str, list] = {}
    try:
        for i, rec in enumerate(rd):
            for k, v in rec.items():
                cols.setdefault(k, []).append(v)
            if i + 1 >= rows:
                break
    finally:
        rd.close()
    if not cols:
        raise ValueError(f"dataset {dataset!r} holds no {kind} records")
    return {k: torch.cat(v, dim=0) for k, v in cols.items()}


class _PolicyWithValue:
    """tokens -> (logits, values): trunk + policy/value head of a PPO root graph, as one callable module."""

    def __new__(cls, spec):
        import torch
        from ..tensor.compiler import CompiledTorchGraph
        from ..torch_templates import GraphBuilder
        from ..torch_templates_roots import _trunk

        b = GraphBuilder("ppo_policy")
        tokens = b.input("tokens", "tokens")
        hidden, _w, _aux = _trunk(b, spec, tokens)
        pv = b.node("policy_logits_value", {"model_dim": spec.model_dim, "vocab_size": spec.vocab_size,
                                            "output_multiplier": spec.output_multiplier, "logit_softcap": spec.logit_softcap},
                    [hidden], "policy_value")
        graph = b.outputs((pv, 0), (pv, 1))

        class Policy(torch.nn.Module):
            def __init__(self) -> None:
                super().__init__()
                self.graph_module = CompiledTorchGraph(graph)

            def forward(self, ids):
                logits, values = self.graph_module(ids.long())
                return logits, values.squeeze(-1) if values.ndim == 3 else values

        return Policy()


def _train_post(a, spec, graph, cfg, plan, device) -> int:
    """SFT / DPO / reward-model runs over structured record datasets, PPO over prompt records."""
    import torch
    from ..inference import export_to_pt, load_pt_checkpoint, save_adapter_checkpoint
    from ..serialization import save_graph
    from ..tensor.trainer import TorchTrainer
    mode = spec.finetune.objective
    rows = a.train_rows or 2048
    out = Path(a.output or (Path(a.output_dir or f"artifacts/{mode}-run") / "model.pt"))
    out.parent.mkdir(parents=True, exist_ok=True)
    t0 = time.perf_counter()
    if mode == "ppo":
        from ..tensor.ppo import PPOConfig, PPOTrainer
        ft = spec.finetune
        rec = _read_records(a.dataset, "ppo_prompt", rows)
        # rollouts start from a rectangular prompt block: the shortest prompt length of the set
        prompt_len = max(1, int(rec["attention_mask"].sum(1).min()))
        prompts = rec["input_ids"].long()[:, :prompt_len]
        policy = _PolicyWithValue(spec).to(device)
        if ft.base_checkpoint:
            state, _meta = load_pt_checkpoint(ft.base_checkpoint)
            policy.graph_module.load_state_dict(state, strict=False)
        reference = _PolicyWithValue(spec).to(device).eval()
        reference.load_state_dict(policy.state_dict())
        if ft.ref_checkpoint:
            state, _meta = load_pt_checkpoint(ft.ref_checkpoint)
            reference.graph_module.load_state_dict(state, strict=False)
        for p_ in reference.parameters():
            p_.requires_grad_(False)
        if ft.reward_checkpoint:
            from ..tensor.stages_core import build_module
            frozen = build_module("reward_forward", {"reward_graph_path": ft.reward_graph_path, "reward_weights_path": ft.reward_checkpoint,
                                                     "model_dim": spec.model_dim}).to(device)

            def reward(ids, prompt_len):
                return frozen(ids).reshape(ids.size(0), -1)[:, -1]
        else:
            # without a reward model: length-normalised reference log-likelihood of the response (a smoke-test reward)
            def reward(ids, prompt_len):
                lp = torch.log_softmax(reference(ids)[0][:, prompt_len - 1:-1].float(), -1)
                return lp.gather(-1, ids[:, prompt_len:, None]).squeeze(-1).mean(1)
        pcfg = PPOConfig(learning_rate=a.learning_rate, kl_coef=ft.kl_coef, clip_range=ft.ppo_clip, value_coef=ft.ppo_vf_coef,
                         entropy_coef=ft.ppo_ent_coef, max_new_tokens=ft.rollout_length, ppo_epochs_per_rollout=ft.ppo_epochs_per_rollout,
                         minibatch_size=ft.ppo_minibatch_size, gamma=ft.gae_gamma, gae_lambda=ft.gae_lambda, seed=a.seed)
        trainer = PPOTrainer(policy, lambda ids: reference(ids)[0], reward, pcfg)
        history = []
        for step in range(a.max_steps):
            batch = prompts[(step * a.batch_size) % max(1, prompts.size(0) - a.batch_size + 1):][:a.batch_size].to(device)
            stats = trainer.step(batch)
            history.append(stats)
            if a.progress_every and (step + 1) % a.progress_every == 0:
                print(json.dumps({"event": "ppo_step", "step": step + 1, **{k: round(float(v), 6) for k, v in stats.items()
                                                                           if isinstance(v, (int, float))}}), flush=True)
        torch.save({"state_dict": policy.graph_module.state_dict(), "metadata": {"objective": "ppo", "steps": len(history)}}, out)
        save_graph(policy.graph_module.graph, out.with_suffix(".json"))
        report = {"event": "complete", "status": "ok", **plan, "steps": len(history), "weights": str(out),
                  "last": {k: float(v) for k, v in (history[-1] if history else {}).items() if isinstance(v, (int, float))},
                  "wall_seconds": round(time.perf_counter() - t0, 3)}
        print(json.dumps(report, default=str))
        return 0
    if mode == "sft":
        rec = _read_records(a.dataset, "sft", rows)
        inputs = {"tokens": rec["input_ids"].long(), "target_ids": rec["targets"].long(), "loss_mask": rec["loss_mask"]}
    else:
        rec = _read_records(a.dataset, "preference", rows)
        c, r = "chosen", "rejected"
        if mode == "dpo":
            inputs = {f"{c}_tokens": rec[f"{c}_input_ids"].long(), f"{c}_targets": rec[f"{c}_targets"].long(), f"{c}_mask": rec[f"{c}_loss_mask"],
                      f"{r}_tokens": rec[f"{r}_input_ids"].long(), f"{r}_targets": rec[f"{r}_targets"].long(), f"{r}_mask": rec[f"{r}_loss_mask"]}
        else:
            inputs = {f"{c}_tokens": rec[f"{c}_input_ids"].long(), f"{c}_mask": rec[f"{c}_loss_mask"],
                      f"{r}_tokens": rec[f"{r}_input_ids"].long(), f"{r}_mask": rec[f"{r}_loss_mask"]}
    trainer = TorchTrainer(graph, cfg)
    steps: list[dict] = []
    trainer.train(inputs, on_step=steps.append)
    save_graph(graph, out.with_suffix(".json"))
    if getattr(a, "adapter_only_save", None) and spec.block_spec.adapter_type != "none":
        save_adapter_checkpoint(trainer.compiled, out)
    else:
        export_to_pt(trainer.compiled, out, metadata={"template_spec": spec.to_dict(), "objective": mode, "steps": trainer.global_step})
    report = {"event": "complete", "status": "ok", **plan, "steps": trainer.global_step,
              "first_loss": steps[0]["loss"] if steps else None, "final_loss": steps[-1]["loss"] if steps else None,
              "wall_seconds": round(time.perf_counter() - t0, 3), "graph": str(out.with_suffix(".json")), "weights": str(out)}
    out.with_suffix(".report.json").write_text(json.dumps(report, indent=2, default=str))
    print(json.dumps(report, default=str))
    return 0


def cmd_eval(a) -> int:
    """Validation loss (and perplexity) of a trained graph on a dataset split, plus optional greedy /
    sampled continuations of prompt tokens through the KV-free graph generator."""
    import torch
    from ..inference import import_from_pt
    from ..serialization import load_graph
    graph = load_graph(a.graph)
    device = torch.device(a.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    weights = a.weights or str(Path(a.graph).with_suffix(".pt"))
    model = import_from_pt(graph, weights, strict=not a.allow_partial_weights).to(device).eval()
    spec = dict(graph.torch_config.get("template_spec") or {})
    vocab = int(spec.get("vocab_size", 0)) or 50257
    seq_len = a.context_window or a.seq_len
    rows, data_note = load_token_rows(a.dataset, seq_len, a.eval_batches * a.eval_batch_size, vocab, a.seed, split="val")
    inputs, names = _objective_inputs(graph, rows)
    tensors = list(inputs.values())
    if len(tensors) < len(names):
        from ..tensor.trainer import TorchTrainer
        tensors = TorchTrainer._complete_semantic_inputs(tensors, model, spec)
    total, count = 0.0, 0
    amp = {"bfloat16": torch.bfloat16, "float16": torch.float16}.get(a.amp_dtype or "")
    with torch.no_grad():
        for i in range(0, rows.size(0), a.eval_batch_size):
            batch = [t[i:i + a.eval_batch_size].to(device) for t in tensors]
            with torch.autocast(device_type=device.type, dtype=amp, enabled=amp is not None and device.type == "cuda"):
                loss = model(*batch)[0]
            total += float(loss) * batch[0].size(0)
            count += batch[0].size(0)
    val = total / max(count, 1)
    report: dict[str, Any] = {"status": "ok", "graph": str(a.graph), "weights": str(weights), "data": data_note, "rows": count,
                              "seq_len": seq_len, "validation_loss": val, "perplexity": math.exp(min(val, 50.0)),
                              "objective": str((spec.get("template") or {}).get("objective", "ar"))}
    if a.prompt_tokens:
        from ..config import spec_from_dict
        from ..inference import InferenceCache
        from ..tensor.compiler import CompiledTorchGraph
        from ..torch_templates import build_model_stage_graph
        # the trained graph ends in a loss; generation runs the same trunk and head as a tokens -> logits graph
        gen_model = CompiledTorchGraph(build_model_stage_graph(spec_from_dict(spec), with_loss=False)).to(device).eval()
        missing = gen_model.load_state_dict(model.state_dict(), strict=False).missing_keys
        if missing:
            raise ValueError(f"prompt probes need the autoregressive trunk of the graph; {len(missing)} tensors are absent "
                             f"(first: {missing[0]})")
        probes = []
        for j, raw in enumerate(a.prompt_tokens.split(";")):
            ids = [int(t) for t in raw.split(",") if t.strip()]
            gen = torch.Generator(device="cpu").manual_seed(a.seed + j)
            cache = InferenceCache(gen_model, max_context=seq_len)
            out_ids = cache.generate(ids, a.max_new_tokens, temperature=a.temperature, top_k=a.top_k, generator=gen)
            probes.append({"prompt_tokens": ids, "token_ids": out_ids})
        report["prompt_probes"] = probes
    text = json.dumps(report, indent=2)
    if a.report_path:
        Path(a.report_path).parent.mkdir(parents=True, exist_ok=True)
        Path(a.report_path).write_text(text)
    print(json.dumps(report))
    return 0


def add_eval_arguments(p: argparse.ArgumentParser) -> None:
    p.add_argument("--graph", required=True, help="graph JSON written by nfn train --runtime torch")
    p.add_argument("--weights", default=None, help="weights .pt (default: beside the graph)")
    p.add_argument("--dataset", default="", help="dataset alias, directory or shard (empty: synthetic tokens)")
    p.add_argument("--report-path", default=None)
    p.add_argument("--eval-batches", type=int, default=20)
    p.add_argument("--eval-batch-size", type=int, default=8)
    p.add_argument("--seq-len", type=int, default=256)
    p.add_argument("--context-window", type=int, default=0)
    p.add_argument("--prompt-tokens", default="", help="comma-separated ids; ';' separates prompts")
    p.add_argument("--max-new-tokens", type=int, default=32)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--device", default=None)
    p.add_argument("--amp-dtype", choices=("float32", "bfloat16", "float16"), default=None)
    p.add_argument("--allow-partial-weights", action="store_true")


MIGRATE_KINDS = ("graph-to-native", "muse-glimmer-to-native", "muse-glimmer-gguf-to-native", "muse-glimmer-lora-to-native")


def add_migrate_arguments(p: argparse.ArgumentParser) -> None:
    p.add_argument("kind", choices=MIGRATE_KINDS)
    p.add_argument("--graph", default=None)
    p.add_argument("--weights", default=None, help="optional .pt checkpoint exported by the graph runtime")
    p.add_argument("--output-dir", default=None, help="new artifact directory; an existing path is never overwritten")
    p.add_argument("--dry-run", action="store_true", help="validate and print the manifest without writing files")
    p.add_argument("--name", default="")
    p.add_argument("--stop-tokens", default="")
    p.add_argument("--source", default=None)
    p.add_argument("--gguf", action="append", default=[])
    p.add_argument("--geometry", default=None, help="muse-glimmer kinds: JSON (text or file) overriding the published geometry, e.g. for small test models")
    p.add_argument("--allow-extra-prefix", action="append", default=[], help="tensor-name prefix to skip (e.g. model.vision_tower.)")
    p.add_argument("--artifact", default=None)
    p.add_argument("--checkpoint", default=None)


def cmd_migrate(a) -> int:
    if a.kind in ("muse-glimmer-to-native", "muse-glimmer-gguf-to-native"):
        # published text weights -> a named-tensor checkpoint of the native Glimmer engine
        from ..checkpoint import glimmer_weights as gw
        geom = gw.GlimmerGeometry.from_json(a.geometry) if a.geometry else gw.GlimmerGeometry()
        gguf = a.kind.endswith("gguf-to-native")
        source = a.gguf if gguf else a.source
        if not source:
            raise ValueError(f"nfn migrate {a.kind} needs " + ("--gguf FILE (repeatable)" if gguf else "--source DIR"))
        extra = tuple(x for x in (a.allow_extra_prefix or []) if x)
        if a.dry_run:
            if gguf:
                from ..checkpoint.gguf import GGUFFile
                names = {}
                for path in source:
                    with GGUFFile(path) as f:
                        names.update({n: tuple(t.shape) for n, t in f.tensors.items()})
                missing = [c.source for c in gw.gguf_contracts(geom) if names.get(c.source) != c.shape]
                print(json.dumps({"status": "ok" if not missing else "mismatch", "tensors": len(names), "missing_or_misshapen": missing[:8]}))
                return 0 if not missing else 2
            print(json.dumps(gw.inspect_glimmer_safetensors(source, geom, allow_extra_prefixes=extra)))
            return 0
        if not a.output_dir:
            raise ValueError("--output-dir is required (or --dry-run)")
        man = gw.convert_glimmer_weights(source, a.output_dir, geom, gguf=gguf, allow_extra_prefixes=extra)
        print(json.dumps({"status": "ok", "output_dir": a.output_dir, **man}))
        return 0
    if a.kind != "graph-to-native":
        print(json.dumps({"status": "unsupported", "kind": a.kind,
                          "reason": "LoRA attachment to a converted Muse-Glimmer artifact is not part of this build"}), file=sys.stderr)
        return 2
    if not a.graph or not (a.output_dir or a.dry_run):
        raise ValueError("nfn migrate graph-to-native needs --graph and --output-dir (or --dry-run)")
    from ..native_ir import compatibility_report, lower_graph, migrate_graph_to_native
    from ..serialization import load_graph
    stops = [int(t) for t in a.stop_tokens.split(",") if t.strip()]
    graph = load_graph(a.graph)
    if a.weights:
        # legacy .pt weights: load them into the graph's module states before lowering
        from ..inference import import_from_pt
        import_from_pt(graph, a.weights, strict=True).sync_state_back()
    if a.dry_run:
        ir = lower_graph(graph)
        print(json.dumps({"status": "dry-run", "graph": str(a.graph), "nodes": len(ir.get("nodes", [])),
                          "compatibility": compatibility_report(ir)}, default=str))
        return 0
    if Path(a.output_dir).exists():
        raise FileExistsError(f"{a.output_dir} exists; artifacts are never overwritten")
    man = migrate_graph_to_native(graph, a.output_dir, model_name=a.name or None, stop_token_ids=stops)
    print(json.dumps({"status": "ok", "output_dir": a.output_dir, "model": man["model"], "capabilities": man["capabilities"],
                      "tensor_bytes": man["tensors"]["total_bytes"]}, default=str))
    return 0
