"""Reference arm of bench.py: the unmodified reference package (installed with
``pip --target baseline/_ref``) trained through its own public API and stock code
path - ``build_gpt2_qknorm_spec`` -> ``build_gpt_root_graph`` -> ``TorchTrainer.train``
- on the same model, batch shape, dtype and synthetic data as the framework's own arm.
Nothing from ``neuralfn_b200`` is imported here.

Single GPU: plain ``TorchTrainer``. Several GPUs: the reference's only multi-device
hook, ``TorchTrainConfig.fsdp2_enabled`` (``neuralfn/torch_backend.py:5848-5853``), with
the process group created by this launcher because the reference does not create one.
"""
from __future__ import annotations

import os
import time


def run(args, metric: str, model_name: str, baseline_tokens_per_s: float, clock_sampler_cls) -> dict:
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from neuralfn import TorchTrainConfig, TorchTrainer, build_gpt_root_graph
    from neuralfn.config import build_gpt2_qknorm_spec

    B, T = args.micro_batch, args.seq_len
    warm = max(args.warmup, 3)
    total_steps = warm + args.steps
    spec = build_gpt2_qknorm_spec(vocab_size=50257, num_layers=12, model_dim=768, num_heads=12,
                                  max_position_embeddings=1024, logit_softcap=30.0, z_loss_coef=1e-4,
                                  tie_embeddings=True)
    graph = build_gpt_root_graph(model_spec=spec)
    gen = torch.Generator().manual_seed(1234 + rank)
    rows = B * total_steps
    inputs = torch.randint(0, 50257, (rows, T), generator=gen)
    targets = torch.randint(0, 50257, (rows, T), generator=gen)
    # The reference's TorchTrainer has no learning-rate warm-up for its AdamW profile (its
    # ``warmup_steps`` field only drives the parameter-golf profile, neuralfn/torch_backend.py:6140),
    # and 6e-4 from the first step diverges on random tokens. The arm therefore runs at 1e-4, about
    # what the framework's own 60-step warm-up reaches during these few steps; timing does not
    # depend on the value.
    cfg = TorchTrainConfig(learning_rate=1e-4, epochs=4, batch_size=B, weight_decay=0.1, device="cuda",
                           amp_dtype="bfloat16", max_steps=total_steps, grad_clip_norm=1.0,
                           optimizer_profile="adamw", fsdp2_enabled=world > 1, drop_last=True)
    marks: dict[int, float] = {}
    losses: list[float] = []
    sampler = clock_sampler_cls(local)

    def on_step(info: dict) -> None:
        step = int(info["step"])
        losses.append(float(info["loss"]))
        if step == warm:
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            sampler.__enter__()
            marks["t0"] = time.perf_counter()
        elif step == total_steps:
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            marks["t1"] = time.perf_counter()
            sampler.__exit__(None, None, None)

    trainer = TorchTrainer(graph, cfg)
    trainer.train(inputs, targets, on_step=on_step)
    if "t0" not in marks or "t1" not in marks:
        raise RuntimeError(f"reference ran {len(losses)} steps, expected {total_steps}")
    ms = (marks["t1"] - marks["t0"]) * 1e3
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.destroy_process_group()
    ms = float(t[0])
    tokens = args.steps * B * T * world
    value = tokens / (ms / 1e3)
    out = {
        "impl": "reference", "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": value / baseline_tokens_per_s, "dtype": "bf16 autocast",
        "data": "synthetic uniform-random token ids, reference default init",
        "config": {"model": model_name, "global_batch": B * world, "micro_batch_per_gpu": B, "seq_len": T,
                   "parallelism": "fsdp2" if world > 1 else "single",
                   "path": "reference TorchTrainer over CompiledTorchGraph (its native CUDA build needs "
                           "CUDA >= 13.3 cuda_tile.h and non-vendored ThunderKittens sources)",
                   "timing": "host clock between the step callbacks of step W and step W+K with device "
                             "synchronisation on both sides; includes the per-step H2D batch copy and the "
                             "loss .item() the reference loop performs"},
        "clocks": sampler.summary(),
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * T * 8,
                "d2h_bytes_per_step": 4},
        "final_loss": losses[-1] if losses else None,
    }
    return out if rank == 0 else {}
