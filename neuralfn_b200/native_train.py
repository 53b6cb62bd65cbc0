"""Native dense-transformer training run: token shards -> engine -> checkpoints -> JSON report.

``run_native_training(NativeTrainConfig(...))`` is what ``nfn train`` calls. It follows the
contract of the reference's dense GPT trainer (``nfn_gpt2_native_train.cpp``: defaults
``Config :614-725``, schedule ``:5643-5676``, report keys ``:30940-31100``): micro-batches
of ``batch_size x seq_len`` tokens accumulated up to ``train_batch_tokens`` per optimizer
step, warm-up + cosine learning rate, AdamW with decay on matrices and embeddings only,
global-norm clipping on the device, periodic validation on a fixed slice, train-loss
sampling, checkpoints in the dense formats, and a report whose headline is
``train_compute_tokens_per_second`` = tokens processed / (train-loop wall - validation wall).

Data-parallel runs launch one process per GPU (``torchrun``); every rank reads its own
stride of the sequential sampler and the optimizer state is sharded across ranks.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch
import torch.distributed as dist

GPT_VARIANTS = ("gpt2", "gpt2_zloss", "gpt2_softcap", "gpt2_qknorm", "gpt2_stable", "gpt2_qknorm_softcap_zloss", "gpt2_diff", "gpt2_moa")
LLAMA_TEMPLATES = ("llama", "llama_fast", "llama_modern", "qwen3_longctx")
GLIMMER_FAMILIES = ("glimmer", "muse-glimmer", "muse_glimmer")

__all__ = ["NativeTrainConfig", "run_native_training", "build_model_config", "training_plan", "GPT_VARIANTS", "LLAMA_TEMPLATES"]


@dataclass
class NativeTrainConfig:
    base_model: str = "gpt"                 # gpt | gpt2 | gpt3 | nanogpt | llama | muse-glimmer
    objective: str = "ar"                   # muse-glimmer also trains "sft", "dpo" and "reward_model" from record shards
    head_dim: int = 0                       # muse-glimmer: 0 = d_model / n_head
    activation_checkpoint_interval: int = 0 # muse-glimmer: keep this many layers' activations, recompute the rest (0 = keep all)
    template_name: str = "gpt2"
    dataset: str = ""                       # alias under the datasets dir, directory, or file; "" = synthetic
    output_dir: str = ""
    batch_size: int = 64
    seq_len: int = 1024
    train_batch_tokens: int = 524288
    n_layer: int = 12
    n_head: int = 12
    n_kv_head: int = 0                      # llama: 0 = n_head
    d_model: int = 768
    d_ff: int = 0                           # llama: 0 = multiple of 256 near 8/3 d_model
    vocab_size: int = 50257
    learning_rate: float = 6e-4
    lr_schedule: str = "cosine"
    final_lr_fraction: float = 0.0
    warmup_steps: int = 60
    lr_schedule_total_steps: int = 0
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    max_grad_norm: float = 1.0
    max_steps: int = 20000
    eval_every: int = 5000
    eval_batches: int = 20
    train_loss_every: int = 250
    progress_every: int = 10
    checkpoint_every: int = 5000
    seed: int = 1337
    init_mode: str = "gpt2-normal"
    resume: bool = False
    allow_train_as_val: bool = True
    use_cuda_graph: bool = True
    sharded_optimizer_checkpoint: bool | None = None
    extra: dict = field(default_factory=dict)
    extra_paths: dict = field(default_factory=dict)   # "init_from": named checkpoint whose weights start a post-training run


def build_model_config(c: NativeTrainConfig):
    """Template name -> model configuration of the matching native engine."""
    fam = c.base_model.lower()
    if fam in ("gpt", "gpt2", "gpt3", "nanogpt"):
        from .models.gpt2 import GPT2Config
        name = c.template_name if c.template_name in GPT_VARIANTS else "gpt2"
        return GPT2Config.variant(name, n_layer=c.n_layer, n_head=c.n_head, d_model=c.d_model, vocab_size=c.vocab_size,
                                  max_seq_len=c.seq_len)
    if fam == "llama":
        from .models.llama import LlamaConfig
        d_ff = c.d_ff or ((int(8 * c.d_model / 3) + 255) // 256 * 256)
        return LlamaConfig(n_layer=c.n_layer, n_head=c.n_head, n_kv_head=c.n_kv_head or c.n_head, d_model=c.d_model, d_ff=d_ff,
                           vocab_size=c.vocab_size, max_seq_len=c.seq_len, qk_norm=c.template_name == "qwen3_longctx",
                           **c.extra)
    if fam in GLIMMER_FAMILIES:
        from .models.glimmer import GlimmerConfig
        d_ff = c.d_ff or 3 * c.d_model
        return GlimmerConfig(n_layer=c.n_layer, n_head=c.n_head, n_kv_head=c.n_kv_head or c.n_head, head_dim=c.head_dim or c.d_model // c.n_head,
                             d_model=c.d_model, d_ff=d_ff, vocab_size=c.vocab_size, max_seq_len=c.seq_len,
                             ckpt_every=c.activation_checkpoint_interval, **c.extra)
    raise ValueError(f"no native engine for model family {c.base_model!r} (available: gpt, gpt2, gpt3, nanogpt, llama, muse-glimmer)")


def training_plan(c: NativeTrainConfig, world: int = 1) -> dict:
    micro = c.batch_size * c.seq_len * world
    accum = max(1, -(-c.train_batch_tokens // micro))
    model = build_model_config(c)
    n_params = sum(s.numel for s in model.param_specs())
    return {"model_family": c.base_model, "template_name": c.template_name, "world_size": world,
            "microbatch_tokens": micro, "grad_accum_steps": accum, "effective_train_batch_tokens": accum * micro,
            "max_steps": c.max_steps, "parameters": n_params, "parameter_bytes_bf16": 2 * n_params,
            "optimizer_state_bytes_per_rank": 12 * n_params // world,
            "lr_schedule": {"kind": c.lr_schedule, "lr": c.learning_rate, "warmup_steps": c.warmup_steps,
                            "final_lr_fraction": c.final_lr_fraction, "horizon": c.lr_schedule_total_steps or c.max_steps}}


class _SyntheticBatches:
    """Uniform random token ids, fixed per (seed, rank): the data of the benchmark config."""

    def __init__(self, vocab: int, batch: int, seq: int, seed: int, pin: bool) -> None:
        g = torch.Generator().manual_seed(seed)
        self.tok = torch.randint(0, vocab, (batch, seq), generator=g, dtype=torch.int32)
        self.tgt = torch.randint(0, vocab, (batch, seq), generator=g, dtype=torch.int32)
        if pin:
            self.tok, self.tgt = self.tok.pin_memory(), self.tgt.pin_memory()
        self.batch_index = 0

    def __iter__(self):
        return self

    def __next__(self):
        self.batch_index += 1
        return self.tok, self.tgt


def _guard_device_status(trainer, what: str, *, sync: bool = True) -> None:
    """Raise (so the process exits non-zero and a kill-siblings launcher stops the other ranks) when
    any kernel recorded an error since the last check. ``sync=False`` only peeks at what has landed,
    which costs no pipeline stall and is what the per-interval check uses."""
    if sync:
        trainer.check_status()
        return
    from .ops import _lib
    code = int(_lib.load().nfn_status_peek())
    if code > 0:
        raise _lib.KernelLibraryError(f"{what}: device status {code} ({_lib.STATUS_NAMES.get(code, '?')}); aborting before anything is published")


def save_checkpoint_checked(trainer, out_dir, step: int, *, dense_format: bool, sharded_optimizer: bool = False, grad_accum: int = 1):
    """Write a checkpoint only after the device status word has been verified clean: a step that ran
    on stale or partial gradients must never reach a DONE marker."""
    from .checkpoint import save_dense_checkpoint
    from .checkpoint.named import save_named_checkpoint
    _guard_device_status(trainer, f"checkpoint at step {step}")
    if dense_format:
        return save_dense_checkpoint(trainer, out_dir, step, sharded_optimizer=sharded_optimizer, grad_accum=grad_accum)
    return save_named_checkpoint(trainer, out_dir, step)


def _validate(trainer, loader_factory, n_batches: int) -> tuple[float, float]:
    """Mean loss over the first ``n_batches`` validation batches (a fixed slice); forward only."""
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    total, n = 0.0, 0
    for tok, tgt in loader_factory():
        trainer.upload(tok, tgt)
        trainer.engine.forward(compute_grad_logits=False)
        total += float(trainer.engine.loss.item())
        n += 1
        if n >= n_batches:
            break
    if trainer.world > 1:
        t = torch.tensor([total, n], device=trainer.device, dtype=torch.float64)
        dist.all_reduce(t)
        total, n = float(t[0]), int(t[1])
    torch.cuda.synchronize()
    return total / max(n, 1), (time.perf_counter() - t0) * 1e3


def _run_glimmer_post_training(c: NativeTrainConfig) -> dict:
    """SFT / DPO of the native Glimmer engine from record shards (``c.dataset``); one named checkpoint at the end."""
    from .checkpoint.named import load_named_checkpoint, save_named_checkpoint
    from .parallel.dp import AdamWConfig
    from .trainers.glimmer_post import GlimmerPostTrainer
    if c.base_model.lower() not in GLIMMER_FAMILIES:
        raise ValueError(f"--objective {c.objective} has a native engine for muse-glimmer only; other families post-train in the graph runtime")
    if not c.dataset:
        raise ValueError(f"--objective {c.objective} needs --dataset: prepared {'sft' if c.objective == 'sft' else 'preference'} record shards")
    rank = dist.get_rank() if dist.is_initialized() else 0
    opt = AdamWConfig(lr=c.learning_rate, beta1=c.beta1, beta2=c.beta2, eps=c.eps, weight_decay=c.weight_decay, max_grad_norm=c.max_grad_norm,
                      warmup_steps=c.warmup_steps, total_steps=c.lr_schedule_total_steps or c.max_steps,
                      final_lr_fraction=c.final_lr_fraction, schedule=c.lr_schedule)
    post = GlimmerPostTrainer(build_model_config(c), c.batch_size, c.seq_len, c.objective, opt, seed=c.seed, use_cuda_graph=c.use_cuda_graph)
    init_from = c.extra_paths.get("init_from", "")
    if init_from and post.engine.lora:
        # adapters start fresh; the checkpoint provides the frozen base weights
        from .checkpoint import latest_step
        from .checkpoint.named import read_named_tensors
        step = latest_step(Path(init_from))
        if step is None:
            raise FileNotFoundError(f"no completed checkpoint (DONE_*) under {init_from}")
        tensors, _meta, _sha = read_named_tensors(Path(init_from) / f"weights_{step:08d}.nfnw")
        post.engine.load_base(tensors)
    elif init_from:
        load_named_checkpoint(post.trainer, Path(init_from), weights_only=True)
    report = post.fit(c.dataset, c.max_steps, allow_train_as_val=c.allow_train_as_val, log_every=c.progress_every)
    report.update({"model_family": c.base_model, "backend": "neuralfn_b200-native", "status": "ok",
                   "world_size": post.trainer.world, "architecture": asdict(post.trainer.cfg)})
    if c.output_dir:
        out_dir = Path(c.output_dir)
        save_checkpoint_checked(post.trainer, out_dir, post.trainer.opt.step_count, dense_format=False)
        if rank == 0:
            (out_dir / "train_report.json").write_text(json.dumps(report, indent=2, default=str))
    return report


def run_native_training(c: NativeTrainConfig) -> dict:
    from .checkpoint import latest_step, load_dense_checkpoint, save_dense_checkpoint
    from .checkpoint.named import load_named_checkpoint, save_named_checkpoint
    from .models.gpt2 import GPT2Config
    from .parallel.dp import AdamWConfig
    from .trainers.dense_gpt import DenseGPTTrainer

    t_start = time.perf_counter()
    if "RANK" in os.environ and not dist.is_initialized():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl")
    if c.objective != "ar":
        return _run_glimmer_post_training(c)
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    plan = training_plan(c, world)
    accum = plan["grad_accum_steps"]
    model_cfg = build_model_config(c)

    # ---- data ----
    t_data = time.perf_counter()
    dataset_info = None
    if c.dataset:
        from .data import PrefetchingLoader, TokenDataset
        ds = TokenDataset(c.dataset, allow_train_as_val=c.allow_train_as_val)
        dataset_info = ds.describe(c.seq_len, c.batch_size, c.train_batch_tokens)
        if ds.max_token("train") >= c.vocab_size:
            raise ValueError(f"dataset holds token id {ds.max_token('train')} but vocab_size is {c.vocab_size}")
        train_sampler = ds.sampler("train", c.seq_len, c.batch_size, rank, world)
        train_iter = PrefetchingLoader(train_sampler, slots=4)
        val_factory = lambda: iter(ds.sampler("val", c.seq_len, c.batch_size, rank, world))  # noqa: E731
    else:
        train_iter = _SyntheticBatches(c.vocab_size, c.batch_size, c.seq_len, c.seed + rank, pin=True)
        val_batches = _SyntheticBatches(c.vocab_size, c.batch_size, c.seq_len, c.seed + 7919 + rank, pin=True)
        val_factory = lambda: iter(val_batches)  # noqa: E731
    shard_ms = (time.perf_counter() - t_data) * 1e3

    # ---- model + optimizer ----
    opt = AdamWConfig(lr=c.learning_rate, beta1=c.beta1, beta2=c.beta2, eps=c.eps, weight_decay=c.weight_decay,
                      max_grad_norm=c.max_grad_norm, warmup_steps=c.warmup_steps,
                      total_steps=c.lr_schedule_total_steps or c.max_steps, final_lr_fraction=c.final_lr_fraction,
                      schedule=c.lr_schedule)
    trainer = DenseGPTTrainer(model_cfg, c.batch_size, c.seq_len, opt, seed=c.seed, use_cuda_graph=c.use_cuda_graph,
                              grad_accum_steps=accum)
    out_dir = Path(c.output_dir) if c.output_dir else None
    dense_format = isinstance(model_cfg, GPT2Config)  # GPT-2 family keeps the legacy dense layout
    resumed_from = None
    if c.resume and out_dir is not None and latest_step(out_dir) is not None:
        restored = (load_dense_checkpoint if dense_format else load_named_checkpoint)(trainer, out_dir)
        resumed_from = restored["step"]
        if c.dataset:
            train_sampler.seek(resumed_from * accum)  # the data cursor resumes where the run stopped
            train_iter = PrefetchingLoader(train_sampler, slots=4)
    torch.cuda.synchronize()
    setup_ms = (time.perf_counter() - t_start) * 1e3

    # ---- loop ----
    train_losses, val_losses, ckpts = [], [], []
    validation_ms = checkpoint_ms = 0.0
    first_step_ms = None
    tokens_per_opt_step = plan["effective_train_batch_tokens"]
    loop_t0 = time.perf_counter()
    step = trainer.opt.step_count
    steps_run = 0
    while step < c.max_steps:
        s0 = time.perf_counter()
        for _micro in range(accum):
            tok, tgt = next(train_iter)
            want_loss = _micro == accum - 1 and (c.train_loss_every and (step + 1) % c.train_loss_every == 0 or step + 1 == c.max_steps)
            loss = trainer.train_step(tok, tgt, return_loss=bool(want_loss))
        step = trainer.opt.step_count
        steps_run += 1
        if first_step_ms is None:
            torch.cuda.synchronize()
            first_step_ms = (time.perf_counter() - s0) * 1e3
        if loss is not None:
            train_losses.append({"step": step, "loss": loss})
        if c.progress_every and step % c.progress_every == 0:
            # a bounded device wait that ran out (straggler, lost peer) leaves a code in the status word
            # and lets the step continue on stale data: stop here rather than train on and publish it
            _guard_device_status(trainer, f"step {step}", sync=False)
            if rank == 0:
                import sys
                print(f"step {step}/{c.max_steps} lr {float(trainer.opt.hyper_host[0]):.3e}", file=sys.stderr, flush=True)
        if c.eval_every and (step % c.eval_every == 0 or step == c.max_steps):
            _guard_device_status(trainer, f"validation at step {step}")
            vl, vms = _validate(trainer, val_factory, c.eval_batches)
            validation_ms += vms
            val_losses.append({"step": step, "loss": vl})
        if out_dir is not None and c.checkpoint_every and (step % c.checkpoint_every == 0 or step == c.max_steps):
            t0 = time.perf_counter()
            digests = save_checkpoint_checked(trainer, out_dir, step, dense_format=dense_format,
                                              sharded_optimizer=c.sharded_optimizer_checkpoint, grad_accum=accum)
            checkpoint_ms += (time.perf_counter() - t0) * 1e3
            if rank == 0:
                ckpts.append({"step": step, "files": {k: {"sha256": v, "bytes": (out_dir / k).stat().st_size} for k, v in digests.items()}})
    torch.cuda.synchronize()
    loop_ms = (time.perf_counter() - loop_t0) * 1e3
    trainer.check_status()
    tokens = steps_run * tokens_per_opt_step
    compute_ms = max(loop_ms - validation_ms - checkpoint_ms, 1e-9)
    steady_ms = max(loop_ms - (first_step_ms or 0.0) - validation_ms - checkpoint_ms, 1e-9)
    report = {
        "model_family": c.base_model, "backend": "neuralfn_b200-native", "template_name": c.template_name,
        "resolved_native_template_name": c.template_name, "variant": c.template_name, "train_seed": c.seed,
        "initialization_mode": c.init_mode, "status": "ok", "torch_required": True, "world_size": world,
        "architecture": asdict(model_cfg), "plan": plan, "dataset": dataset_info, "resumed_from_step": resumed_from,
        "token_shard_resolution_wall_ms": shard_ms, "setup_wall_ms": setup_ms, "train_loop_wall_ms": loop_ms,
        "train_loop_wall_ms_per_step": loop_ms / max(steps_run, 1), "steps": steps_run, "tokens_processed": tokens,
        "train_first_step_tokens_per_second": tokens_per_opt_step / ((first_step_ms or 1e-9) / 1e3),
        "train_steady_state_tokens_per_second": (max(steps_run - 1, 0) * tokens_per_opt_step) / (steady_ms / 1e3),
        "train_timing_contract": "train_compute_tokens_per_second = tokens_processed / (train_loop_wall - validation_wall - checkpoint_wall)",
        "validation_wall_ms": validation_ms, "checkpoint_wall_ms": checkpoint_ms, "train_compute_wall_ms": compute_ms,
        "train_compute_tokens_per_second": tokens / (compute_ms / 1e3),
        "total_wall_ms": (time.perf_counter() - t_start) * 1e3, "kernel_launches_per_step": trainer.launches_per_step,
        "train_losses": train_losses, "validation": {"losses": val_losses, "fixed_validation_slice": c.eval_batches},
        "checkpoints": ckpts,
        **({f"moa_{k}": v for k, v in trainer.engine.moa.items() if k != "history"} | {"moa_selected_activation": trainer.engine.activation,
                                                                                      "moa_selection_history": trainer.engine.moa["history"][-64:]}
           if getattr(model_cfg, "moa_activations", ()) else {}),
        # per-stage CUDA-event times (NFN_NATIVE_GPT_STAGE_TIMING=1), field names of the reference's report
        "timing": trainer.timer.report() if getattr(trainer, "timer", None) is not None else {"stage_timing_enabled": False},
    }
    if out_dir is not None and rank == 0:
        out_dir.mkdir(parents=True, exist_ok=True)
        (out_dir / "train_report.json").write_text(json.dumps(report, indent=2, default=str))
    return report
