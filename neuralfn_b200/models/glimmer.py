"""Native training engine for the Muse-Glimmer decoder block (CUDA, sm_100a kernels, explicit
forward / backward over preallocated buffers like ``models/llama.py``).

Block: centred RMS norm -> packed q | k | v | gate projection -> weightless per-head QK norm with a
query scale -> rotary embedding on sliding-window layers only (every ``global_every``-th layer is global
and position-free) -> flash attention -> sigmoid output gate -> output projection -> centred post-norm
-> residual add; the same sandwich around a SwiGLU MLP. Weightless RMS norm of the embeddings, plain
RMS final norm, untied head with an output multiplier and a tanh soft-cap.

``GlimmerConfig`` provides the hooks ``DenseGPTTrainer`` needs (``param_specs`` / ``init_params_`` /
``make_engine``), so data parallelism with the sharded AdamW, CUDA-graph steps, gradient accumulation
and the named-tensor checkpoints apply unchanged. Objectives (``GlimmerEngine.objective``):

* ``"ar"``   next-token cross-entropy over all rows;
* ``"sft"``  response-only cross-entropy: ``set_loss_mask`` gives the rows that count;
* ``"reward_model"``  Bradley-Terry preference loss on a scalar head (``GlimmerConfig.reward_head=True`` adds the
  ``reward_head`` vector): the reward of a sequence is <final-norm hidden state at its last counted position, head>;
  the vocabulary head is skipped in both passes;
* ``"ppo"``  the clipped-surrogate UPDATE on a stored rollout (``GlimmerConfig.value_head=True`` adds the ``value_head``
  vector; ``set_ppo_batch`` gives old log-probabilities, advantages, returns and old values per row): the new
  log-probabilities are the negated row losses of the cross-entropy kernel, values are <final-norm hidden state, head>,
  the policy term's gradient goes back through the same kernel as a per-row scale, the value term's through the
  final norm. Same formulas as ``tensor.stages_losses._ppo_terms`` / ``masked_ppo_clipped_loss`` (masked means, advantage
  normalisation); no entropy bonus (the kernel does not form the full-distribution entropy gradient). Rollouts and
  advantages come from the caller (``tensor.ppo`` has the samplers and GAE);
* ``"dpo"``  pairwise preference loss over (chosen, rejected) halves of the batch against frozen
  reference log-probabilities (``set_reference_logps``): the sequence log-probabilities come from the
  cross-entropy kernel's row losses, and the backward pass re-runs that kernel with a per-row gradient
  scale, so no second set of logits is needed.

Reference: the native Glimmer trainer ``neuralfn/csrc/native_train/muse_glimmer_native_train.cpp``
(objective table :187 and :355-359, DPO options :125 and :192, block forward :3461-3515); the block
definition is that of ``neuralfn/torch_templates.py:493-790``; the reward head is ``MaskedRewardHeadStage`` (``neuralfn/torch_backend.py``, "masked_reward_head").
Only the sigmoid DPO loss is built here.

LoRA (``GlimmerConfig.lora_rank > 0``): the trainable flat buffer then holds only the adapters (``<projection>.lora_a`` [r, in],
``<projection>.lora_b`` [out, r], B zero at the start) of the projections named in ``lora_targets``; the base weights sit in a
frozen bf16 buffer owned by the engine (``load_base`` / ``merged_state``). Every adapted projection is the base GEMM plus two
skinny GEMMs whose second one adds ``alpha / r * t B^T`` in its epilogue; the backward pass skips every base weight gradient
(the big TN GEMMs, the norm-weight reductions and the embedding scatter), which is where LoRA's saving comes from. Reference:
the adapter options of ``muse_glimmer_native_train.cpp:187-203`` and ``inspect_native_muse_glimmer_lora_checkpoint``
(``neuralfn/native_muse_glimmer_checkpoint.py:580``). NF4 / K-quant base weights under the adapters and the PPO objective are
not in this engine (they run in the tensor runtime).

Activation checkpointing (``ckpt_every = k``): activation buffers exist for k layers only and are reused by every k-layer
segment; the input of each segment is kept, and the backward pass re-runs a segment's forward before differentiating it
(the reference's ``--activation-checkpoint-interval``, default 4: ``muse_glimmer_native_train.cpp:115,204,1045-1049``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .gpt2 import FlatLayout, ParamSpec

__all__ = ["GlimmerConfig", "GlimmerEngine", "ppo_terms_and_gradients", "glimmer_param_specs", "glimmer_lora_specs", "glimmer_reference_loss"]


@dataclass(frozen=True)
class GlimmerConfig:
    n_layer: int = 52
    n_head: int = 32
    n_kv_head: int = 2
    head_dim: int = 128
    d_model: int = 6656
    d_ff: int = 19968
    vocab_size: int = 202048
    max_seq_len: int = 4096
    window: int = 2048
    global_every: int = 4
    rope_theta: float = 500000.0
    q_scale: float = 3.87
    norm_eps: float = 1e-5
    post_norm_eps: float = 1e-8
    qk_norm_eps: float = 1e-5
    logit_softcap: float = 20.0
    output_multiplier: float = 0.19611613513818404
    z_loss: float = 0.0
    vocab_pad_to: int = 128
    dpo_beta: float = 0.1
    dpo_loss_type: str = "sigmoid"                 # sigmoid | hinge | ipo
    dpo_label_smoothing: float = 0.0                # sigmoid only: weight of the flipped preference
    reward_head: bool = False
    value_head: bool = False
    ppo_clip: float = 0.2
    ppo_vf_coef: float = 0.5
    ppo_normalize_advantages: bool = True
    lora_rank: int = 0                      # > 0: train low-rank adapters over frozen base weights
    lora_alpha: float = 32.0
    lora_targets: tuple = ("wqkvg", "wo", "w_gate_up", "w_down")
    lora_dropout: float = 0.0                      # on the input of the adapters' A matrices (training passes only)
    base_quant: str = ""                         # "" | "nf4": the frozen projection weights under the adapters as NF4 (QLoRA)
    nf4_group: int = 64
    base_seed: int = 1337                   # LoRA: seed of the frozen base weights until load_base() replaces them
    ckpt_every: int = 0                     # > 0: keep activations of this many layers only; recompute segments in backward
    # pipeline-parallel stage view: this engine owns layers [pp_layer_begin, pp_layer_end); the first stage also owns
    # the embedding, the last one the final norm and the heads (0 / 0 = whole model)
    pp_layer_begin: int = 0
    pp_layer_end: int = 0
    pp_first: bool = True
    pp_last: bool = True

    @property
    def layer_range(self) -> range:
        return range(self.pp_layer_begin, self.pp_layer_end or self.n_layer)

    @property
    def padded_vocab(self) -> int:
        p = self.vocab_pad_to
        return (self.vocab_size + p - 1) // p * p

    @property
    def att_dim(self) -> int:
        return self.n_head * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return (self.n_head + 2 * self.n_kv_head) * self.head_dim

    def is_local(self, layer: int) -> bool:
        return self.global_every <= 0 or (layer + 1) % self.global_every != 0

    # hooks used by trainers.dense_gpt.DenseGPTTrainer
    def param_specs(self) -> list[ParamSpec]:
        """The TRAINABLE tensors: the whole model, or only the adapters when ``lora_rank > 0``."""
        return glimmer_lora_specs(self) if self.lora_rank > 0 else glimmer_param_specs(self)

    def base_param_specs(self) -> list[ParamSpec]:
        return glimmer_param_specs(self)

    def init_params_(self, layout: FlatLayout, master: torch.Tensor, seed: int) -> None:
        gen = torch.Generator(device=master.device).manual_seed(seed)
        master.zero_()
        for s in layout.order:
            v = layout.view(master, s.name)
            if s.init == "normal":
                v.normal_(0.0, 0.02, generator=gen)
            elif s.init == "lora_a":
                v.normal_(0.0, 1.0 / math.sqrt(s.shape[1]), generator=gen)
            elif s.init == "resid":
                v.normal_(0.0, 0.02 / math.sqrt(2 * self.n_layer), generator=gen)
            elif s.init == "ones":
                v.fill_(1.0)
            # "zeros": centred norm weights start at 0 (scale 1 + w = 1)
        for name in ("tok_embeddings", "lm_head"):
            if name in layout.offsets:
                layout.view(master, name)[self.vocab_size:].zero_()

    def make_engine(self, layout, params, grads, batch: int, seq: int) -> "GlimmerEngine":
        return GlimmerEngine(self, layout, params, grads, batch, seq)

    @classmethod
    def from_spec(cls, spec, **over) -> "GlimmerConfig":
        bs = spec.block_spec
        kw = dict(n_layer=spec.num_layers, d_model=spec.model_dim, n_head=bs.num_heads, n_kv_head=bs.num_kv_heads or bs.num_heads,
                  head_dim=bs.head_dim, d_ff=bs.intermediate_size, vocab_size=spec.vocab_size, window=bs.window_size,
                  global_every=len(bs.layer_attention_pattern) or 0, rope_theta=bs.rope_theta, q_scale=bs.q_scale_factor,
                  norm_eps=bs.norm_eps, post_norm_eps=bs.post_norm_eps, qk_norm_eps=bs.qk_norm_eps, logit_softcap=spec.logit_softcap,
                  output_multiplier=spec.output_multiplier, z_loss=spec.z_loss_coef)
        kw.update(over)
        return cls(**kw)


def glimmer_lora_specs(cfg: GlimmerConfig) -> list[ParamSpec]:
    """Adapter tensors of this stage: A [r, in] (random) and B [out, r] (zero) per targeted projection."""
    if cfg.lora_rank % 16:
        raise ValueError("lora_rank must be a multiple of 16 (tensor-core tile granularity)")
    shapes = {s.name: s.shape for s in glimmer_param_specs(cfg)}
    specs = []
    for l in cfg.layer_range:
        for t in cfg.lora_targets:
            out_dim, in_dim = shapes[f"layers.{l}.{t}"]
            specs += [ParamSpec(f"layers.{l}.{t}.lora_a", (cfg.lora_rank, in_dim), True, "lora_a"),
                      ParamSpec(f"layers.{l}.{t}.lora_b", (out_dim, cfg.lora_rank), True, "zeros")]
    if cfg.pp_last:
        specs += [ParamSpec(n, (cfg.d_model,), False, "normal") for n, on in (("reward_head", cfg.reward_head), ("value_head", cfg.value_head)) if on]
    return specs


def glimmer_param_specs(cfg: GlimmerConfig) -> list[ParamSpec]:
    C, Fd, Vp = cfg.d_model, cfg.d_ff, cfg.padded_vocab
    specs = [ParamSpec("tok_embeddings", (Vp, C), True, "normal")] if cfg.pp_first else []
    for l in cfg.layer_range:
        p = f"layers.{l}."
        specs += [ParamSpec(p + "attn_norm", (C,), False, "zeros"), ParamSpec(p + "wqkvg", (cfg.qkv_dim + cfg.att_dim, C), True, "normal"),
                  ParamSpec(p + "wo", (C, cfg.att_dim), True, "resid"), ParamSpec(p + "post_attn_norm", (C,), False, "zeros"),
                  ParamSpec(p + "mlp_norm", (C,), False, "zeros"), ParamSpec(p + "w_gate_up", (2 * Fd, C), True, "normal"),
                  ParamSpec(p + "w_down", (C, Fd), True, "resid"), ParamSpec(p + "post_mlp_norm", (C,), False, "zeros")]
    if cfg.pp_last:
        specs += [ParamSpec("norm", (C,), False, "ones"), ParamSpec("lm_head", (Vp, C), True, "normal")]
        if cfg.lora_rank == 0:
            specs += [ParamSpec(n, (C,), False, "normal") for n, on in (("reward_head", cfg.reward_head), ("value_head", cfg.value_head)) if on]
    return specs


# ------------------------------------------------------------------------------- oracle --
def glimmer_reference_loss(cfg: GlimmerConfig, p: dict[str, torch.Tensor], tokens: torch.Tensor, targets: torch.Tensor,
                           loss_mask: torch.Tensor | None = None, hidden_out: list | None = None):
    """Plain PyTorch restatement with this engine's parameter names. Returns (loss, logits [B, T, V], row
    losses [B, T]); with ``loss_mask`` the loss is the masked mean. ``hidden_out`` (a list) receives the
    final-norm hidden states [B, T, C], which the reward head reads."""
    import torch.nn.functional as F
    B, T = tokens.shape
    hd, H, Hkv, Fd = cfg.head_dim, cfg.n_head, cfg.n_kv_head, cfg.d_ff

    def crms(x, w, eps, centered=True):
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        return y if w is None else y * (1.0 + w if centered else w)

    x = crms(p["tok_embeddings"][tokens.long()], None, cfg.norm_eps)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=x.device, dtype=torch.float32) / hd))
    ang = torch.outer(torch.arange(T, device=x.device, dtype=torch.float32), inv)
    cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)

    def rot(t):
        a, b = t[..., :hd // 2], t[..., hd // 2:]
        return torch.cat((a * cos - b * sin, b * cos + a * sin), -1)

    pos = torch.arange(T, device=x.device)
    for l in range(cfg.n_layer):
        g = lambda k: p[f"layers.{l}.{k}"]  # noqa: E731
        h = crms(x, g("attn_norm"), cfg.norm_eps)
        qkvg = h @ g("wqkvg").T
        q = qkvg[..., :H * hd].view(B, T, H, hd).transpose(1, 2)
        k = qkvg[..., H * hd:(H + Hkv) * hd].view(B, T, Hkv, hd).transpose(1, 2)
        v = qkvg[..., (H + Hkv) * hd:cfg.qkv_dim].view(B, T, Hkv, hd).transpose(1, 2)
        gate = torch.sigmoid(qkvg[..., cfg.qkv_dim:])
        q, k = crms(q, None, cfg.qk_norm_eps) * cfg.q_scale, crms(k, None, cfg.qk_norm_eps)
        local = cfg.is_local(l)
        if local:
            q, k = rot(q), rot(k)
        mask = pos[None, :] <= pos[:, None]
        if local and cfg.window > 0:
            mask = mask & (pos[None, :] > pos[:, None] - cfg.window)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=H != Hkv)
        a = a.transpose(1, 2).reshape(B, T, H * hd) * gate
        x = x + crms(a @ g("wo").T, g("post_attn_norm"), cfg.post_norm_eps)
        h = crms(x, g("mlp_norm"), cfg.norm_eps)
        gu = h @ g("w_gate_up").T
        x = x + crms((F.silu(gu[..., :Fd]) * gu[..., Fd:]) @ g("w_down").T, g("post_mlp_norm"), cfg.post_norm_eps)
    x = crms(x, p["norm"], cfg.norm_eps, centered=False)
    if hidden_out is not None:
        hidden_out.append(x)
    logits = (x @ p["lm_head"].T)[..., :cfg.vocab_size] * cfg.output_multiplier
    if cfg.logit_softcap > 0:
        logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
    lf = logits.float()
    lse = torch.logsumexp(lf, -1)
    rows = lse - lf.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1) + cfg.z_loss * lse * lse
    if loss_mask is None:
        return rows.mean(), logits, rows
    m = loss_mask.to(rows.dtype)
    return (rows * m).sum() / m.sum().clamp(min=1.0), logits, rows


DPO_LOSS_TYPES = ("sigmoid", "hinge", "ipo")


def dpo_pair_terms(z: torch.Tensor, *, beta: float, loss_type: str = "sigmoid", label_smoothing: float = 0.0):
    """Per-pair preference loss and its derivative for ``z = beta * ((pol_c - pol_r) - (ref_c - ref_r))``: ``(loss [P], d loss / d z [P])``.
    The three forms of the reference's ``dpo_pairwise_loss`` node (neuralfn/torch_backend.py, ``DPOPairwiseLossStage``): sigmoid
    ``-log sigmoid(z)`` (with label smoothing e: ``-(1 - e) log sigmoid(z) - e log sigmoid(-z)``), hinge ``relu(1 - z)`` and IPO
    ``(z - 1 / (2 beta))^2``. Written out by hand because the native engine has no autograd."""
    if loss_type == "hinge":
        return torch.relu(1.0 - z), -(z < 1.0).to(z.dtype)
    if loss_type == "ipo":
        d = z - 1.0 / (2.0 * max(float(beta), 1e-8))
        return d * d, 2.0 * d
    if loss_type != "sigmoid":
        raise ValueError(f"dpo loss type {loss_type!r}: one of {DPO_LOSS_TYPES}")
    e = float(label_smoothing)
    sp = torch.nn.functional.softplus
    return (1.0 - e) * sp(-z) + e * sp(z), -(1.0 - e) * torch.sigmoid(-z) + e * torch.sigmoid(z)


def ppo_terms_and_gradients(logp, logp_old, advantages, returns, value, value_old, mask, *, clip: float, vf_coef: float,
                            normalize_advantages: bool = True) -> dict[str, torch.Tensor]:
    """The clipped-surrogate policy term and the clipped value term over the rows with ``mask`` > 0 (masked means), and
    their gradients with respect to the per-row log-probabilities and values, written out by hand (no autograd, no host
    synchronisation: usable inside a captured step). Same terms as ``tensor.stages_losses._ppo_terms`` /
    ``masked_ppo_clipped_loss``; loss = policy + vf_coef * value."""
    m = mask.to(logp.dtype)
    denom = m.sum().clamp(min=1.0)
    adv = advantages
    if normalize_advantages:
        mean = (adv * m).sum() / denom
        adv = (adv - mean) * torch.rsqrt((((adv - mean) ** 2) * m).sum() / denom + 1e-8)
    ratio = torch.exp(logp - logp_old)
    clipped = ratio.clamp(1.0 - clip, 1.0 + clip)
    unclipped_active = ratio * adv <= clipped * adv                 # the minimum is the unclipped product (ties included)
    policy = -torch.minimum(ratio * adv, clipped * adv)
    v_clip = value_old + (value - value_old).clamp(-clip, clip)
    first = (value - returns) ** 2 >= (v_clip - returns) ** 2
    val = 0.5 * torch.where(first, (value - returns) ** 2, (v_clip - returns) ** 2)
    policy_loss, value_loss = (policy * m).sum() / denom, (val * m).sum() / denom
    inside = ((value - value_old).abs() < clip).to(value.dtype)      # derivative of the clamp
    return {"loss": policy_loss + vf_coef * value_loss, "policy_loss": policy_loss, "value_loss": value_loss,
            "clip_fraction": ((~unclipped_active).to(m.dtype) * m).sum() / denom, "approx_kl": ((logp_old - logp) * m).sum() / denom,
            "d_logp": torch.where(unclipped_active, -adv * ratio, torch.zeros_like(adv)) * m / denom,
            "d_value": torch.where(first, value - returns, (v_clip - returns) * inside) * vf_coef * m / denom}


# ------------------------------------------------------------------------------- engine --
class GlimmerEngine:
    OBJECTIVES = ("ar", "sft", "dpo", "reward_model", "ppo")

    def __init__(self, cfg: GlimmerConfig, layout: FlatLayout, params: torch.Tensor, grads: torch.Tensor, batch: int, seq: int) -> None:
        from ..ops import infer as I
        from ..ops import kernels as K
        from ..ops.gemm import gemm
        self.K, self.I, self.gemm = K, I, gemm
        self.cfg, self.layout, self.B, self.T = cfg, layout, batch, seq
        if seq > cfg.max_seq_len:
            raise ValueError("sequence longer than max_seq_len")
        if cfg.head_dim not in (64, 128):
            raise ValueError("head_dim must be 64 or 128")
        self.params, self.grads = params, grads
        self.p, self.g = layout.views(params), layout.views(grads)
        dev = params.device
        self.lora = cfg.lora_rank > 0
        self.lora_scale = cfg.lora_alpha / cfg.lora_rank if self.lora else 0.0
        if self.lora:
            # frozen base weights in their own flat buffer; self.p resolves both kinds of names, self.g only adapters
            self.base_layout = FlatLayout(cfg.base_param_specs())
            master = torch.empty(self.base_layout.n_total, device=dev, dtype=torch.float32)
            replace_cfg = GlimmerConfig(**{**cfg.__dict__, "lora_rank": 0})
            replace_cfg.init_params_(self.base_layout, master, cfg.base_seed)
            self.base = master.to(torch.bfloat16)
            del master
            self.p = {**self.base_layout.views(self.base), **self.p}
            self.q: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}      # NF4 base projections: name -> (codes, absmax)
            if cfg.base_quant:
                if cfg.base_quant != "nf4":
                    raise ValueError(f"base_quant {cfg.base_quant!r}: only 'nf4'")
                self._quantise_base()
        elif cfg.base_quant:
            raise ValueError("base_quant needs lora_rank > 0: a quantised base is frozen, only adapters train")
        if not 0.0 <= cfg.lora_dropout < 1.0:
            raise ValueError("lora_dropout must be in [0, 1)")
        self.drop_p = float(cfg.lora_dropout) if self.lora else 0.0
        self.drop_on = False                                               # set by forward(): training passes only
        if self.drop_p > 0.0 and not (cfg.pp_first and cfg.pp_last):
            raise ValueError("lora_dropout is not available on pipeline stages: a stage runs other micro-batches between a forward and its backward pass")
        if self.drop_p > 0.0:
            # masks are regenerated, not stored: a device step word advanced once per forward pass (inside the step graph) and one
            # stream id per adapted projection; the backward pass and a recomputed segment see the same word
            self.drop_step = torch.zeros(1, device=dev, dtype=torch.int64)
            self.drop_ids = {s_.name[:-len(".lora_a")]: i for i, s_ in enumerate(x for x in layout.order if x.name.endswith(".lora_a"))}
            widest = max(s_.shape[1] for s_ in layout.order if s_.name.endswith(".lora_a"))
            self.drop_x = torch.empty(batch * seq, widest, device=dev, dtype=torch.bfloat16)
            self.drop_dx = torch.empty(batch * seq, widest, device=dev, dtype=torch.bfloat16)
        N, C, Fd, Q, A = batch * seq, cfg.d_model, cfg.d_ff, cfg.qkv_dim, cfg.att_dim
        bf, f32 = torch.bfloat16, torch.float32
        e = lambda *s, dtype=bf: torch.empty(*s, device=dev, dtype=dtype)  # noqa: E731
        self.cos, self.sin = I.rope_tables(seq, cfg.head_dim, cfg.rope_theta, device=dev)
        self.ones = torch.ones(C, device=dev, dtype=bf)
        self.xe, self.re = e(N, C), e(N, dtype=f32)          # raw embeddings and the rstd of their weightless norm
        self.x0 = e(N, C)
        self.acts = [dict(n1=e(N, C), r1=e(N, dtype=f32), qkvg=e(N, Q + A), qk_rstd=e(N, cfg.n_head + cfg.n_kv_head, dtype=f32),
                          att=e(N, A), attg=e(N, A), lse=e(batch, cfg.n_head, seq, dtype=f32), br=e(N, C), rp1=e(N, dtype=f32), x1=e(N, C),
                          n2=e(N, C), r2=e(N, dtype=f32), gu=e(N, 2 * Fd), h=e(N, Fd), mb=e(N, C), rp2=e(N, dtype=f32), x2=e(N, C))
                     for _ in range(self._resident_layers())]
        n_seg = -(-len(cfg.layer_range) // len(self.acts)) if self.acts else 0
        # input of every segment of layers (segment 0 reads x0 itself); one segment = everything resident = no recompute
        self.bound = [self.x0] + [e(N, C) for _ in range(n_seg - 1)]
        if self.lora:
            for a in self.acts:
                a.update({"t_" + t: e(N, cfg.lora_rank) for t in cfg.lora_targets})
            self.d_t = e(N, cfg.lora_rank)
        self.layers = list(cfg.layer_range)
        self.nb = e(N, C)                                       # normalised branch (temporary)
        self.nf, self.rf = e(N, C), e(N, dtype=f32)
        self.mean_scratch = e(N, dtype=f32)
        self.logits = e(N, cfg.padded_vocab)
        self.row_loss = e(N, dtype=f32)
        self.loss = torch.zeros(1, device=dev, dtype=f32)
        self.d_a, self.d_b, self.d_n, self.d_br = e(N, C), e(N, C), e(N, C), e(N, C)
        self.d_h, self.d_gu = e(N, Fd), e(N, 2 * Fd)
        self.d_qkvg, self.d_attg, self.d_att = e(N, Q + A), e(N, A), e(N, A)
        self.delta = e(batch, cfg.n_head, seq, dtype=f32)
        self.scratch = e(max(64 * 2 * max(2 * Fd, Q + A, C), K.norm_fused_rows() * 3 * C), dtype=f32)
        self.ws = e(32 * 1024 * 1024, dtype=f32)
        self.tokens = torch.zeros(N, device=dev, dtype=torch.int32)
        self.tok_sorted = torch.zeros(N, device=dev, dtype=torch.int32)      # stable sort of the batch's tokens: the token-embedding gradient
        self.tok_order = torch.zeros(N, device=dev, dtype=torch.int64)       # sums equal tokens in row order (bitwise reproducible)
        self.targets = torch.zeros(N, device=dev, dtype=torch.int32)
        # objective state
        self.objective = "ar"
        self.loss_mask = torch.ones(N, device=dev, dtype=f32)       # SFT / DPO: rows that count
        self.row_scale = torch.ones(N, device=dev, dtype=f32)       # per-row gradient scale handed to the loss kernel
        self.ref_logps = torch.zeros(batch, device=dev, dtype=f32)  # DPO: frozen reference sequence log-probabilities
        self.seq_logps = torch.zeros(batch, device=dev, dtype=f32)
        self.dpo_stats = torch.zeros(3, device=dev, dtype=f32)      # loss, reward accuracy, reward margin
        self.ppo_in = torch.zeros(4, N, device=dev, dtype=f32)      # rollout: old log-probabilities, advantages, returns, old values
        self.ppo_stats = torch.zeros(4, device=dev, dtype=f32)      # policy loss, value loss, clipped fraction, approximate KL
        self.values = torch.zeros(N, device=dev, dtype=f32)
        self.timer = None

    # --------------------------------------------------------------------------- inputs --
    def set_batch(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        self.tokens.copy_(tokens.reshape(-1), non_blocking=True)
        self.targets.copy_(targets.reshape(-1), non_blocking=True)

    def set_objective(self, objective: str) -> None:
        if objective not in self.OBJECTIVES:
            raise ValueError(f"objective must be one of {self.OBJECTIVES}")
        if objective in ("dpo", "reward_model") and self.B % 2:
            raise ValueError("preference batches hold (chosen, rejected) pairs: the batch size must be even")
        if objective == "reward_model" and not self.cfg.reward_head:
            raise ValueError("the reward_model objective needs GlimmerConfig(reward_head=True)")
        if objective == "ppo" and not self.cfg.value_head:
            raise ValueError("the ppo objective needs GlimmerConfig(value_head=True)")
        self.objective = objective

    def set_loss_mask(self, mask: torch.Tensor) -> None:
        """mask [B, T] (1 = the row's target counts). Used by the ``sft`` and ``dpo`` objectives."""
        self.loss_mask.copy_(mask.reshape(-1).to(self.loss_mask.dtype), non_blocking=True)

    def set_reference_logps(self, logps: torch.Tensor) -> None:
        """[B] sequence log-probabilities of the frozen reference model (first half chosen, second half rejected)."""
        self.ref_logps.copy_(logps.reshape(-1).to(self.ref_logps.dtype), non_blocking=True)

    def _resident_layers(self) -> int:
        n = len(self.cfg.layer_range)
        return n if self.cfg.ckpt_every <= 0 else min(n, self.cfg.ckpt_every)

    # ----------------------------------------------------------------------------- LoRA --
    PROJECTIONS = ("wqkvg", "wo", "w_gate_up", "w_down")

    @torch.no_grad()
    def _quantise_base(self) -> None:
        """QLoRA: every layer projection of the frozen base becomes NF4 codes + one fp32 absmax per ``nf4_group`` values
        (the reference's ``nf4_linear`` stage, neuralfn/torch_backend.py: low nibble = even column); the bf16 copies are
        dropped - what stays in bf16 is the embedding, the head and the norm weights. A projection is decoded into one shared
        scratch buffer right before each product that reads it (``nfn_dequant_nf4``)."""
        from ..tensor.stages_linear import nf4_quantize
        names = [s.name for s in self.base_layout.order if s.name.rsplit(".", 1)[-1] in self.PROJECTIONS]
        keep = [s for s in self.base_layout.order if s.name not in set(names)]
        full = self.base_layout.views(self.base)
        biggest = 0
        for name in names:
            w = full[name]
            codes, absmax = [], []
            for r0 in range(0, w.shape[0], 1024):                  # row chunks: the nearest-code search holds 16 floats per value
                c, a = nf4_quantize(w[r0:r0 + 1024], self.cfg.nf4_group)
                codes.append(c)
                absmax.append(a)
            self.q[name] = (torch.cat(codes).contiguous(), torch.cat(absmax).contiguous())
            biggest = max(biggest, w.numel())
        small_layout = FlatLayout(keep)
        small = torch.empty(small_layout.n_total, device=self.base.device, dtype=torch.bfloat16)
        for s_ in keep:
            small_layout.view(small, s_.name).copy_(full[s_.name])
        for name in names:
            del self.p[name]
        self.base_layout, self.base = small_layout, small
        self.p.update(small_layout.views(small))
        self._wq_scratch = torch.empty(biggest, device=small.device, dtype=torch.bfloat16)

    def _w(self, name: str) -> torch.Tensor:
        """The bf16 weight of a projection: the parameter itself, or the NF4 base decoded into the scratch buffer (valid until
        the next call)."""
        q = getattr(self, "q", None)
        if not q or name not in q:
            return self.p[name]
        codes, absmax = q[name]
        out = self._wq_scratch[:codes.numel() * 2]
        self.I.dequant_nf4(codes, absmax, self.cfg.nf4_group, out=out)
        return out.view(codes.shape[0], codes.shape[1] * 2)

    def base_bytes(self) -> int:
        """Bytes the frozen base occupies on the device (bf16 tensors + NF4 codes and scales + the decode scratch)."""
        if not self.lora:
            return 0
        n = self.base.numel() * 2
        for codes, absmax in self.q.values():
            n += codes.numel() + absmax.numel() * 4
        return n + (self._wq_scratch.numel() * 2 if self.q else 0)

    def load_base(self, tensors: dict[str, torch.Tensor]) -> None:
        """Replace the frozen base weights (names and shapes of ``base_param_specs``); projections are re-quantised when the
        base is NF4."""
        if not self.lora:
            raise RuntimeError("load_base() is for LoRA engines; full fine-tuning loads weights through the trainer")
        from ..tensor.stages_linear import nf4_quantize
        for s in self.cfg.base_param_specs():
            if tuple(tensors[s.name].shape) != tuple(s.shape):
                raise ValueError(f"{s.name}: shape {tuple(tensors[s.name].shape)} instead of {tuple(s.shape)}")
            if s.name in self.q:
                w = tensors[s.name].to(self.base.device)
                parts = [nf4_quantize(w[r0:r0 + 1024], self.cfg.nf4_group) for r0 in range(0, w.shape[0], 1024)]
                self.q[s.name][0].copy_(torch.cat([c for c, _ in parts]))
                self.q[s.name][1].copy_(torch.cat([a for _, a in parts]))
            else:
                self.base_layout.view(self.base, s.name).copy_(tensors[s.name])

    @torch.no_grad()
    def merged_state(self) -> dict[str, torch.Tensor]:
        """Base weights with the adapters folded in (W + alpha / r * B A), on the host, fp32."""
        out = {s.name: self.base_layout.view(self.base, s.name).float().cpu() for s in self.base_layout.order} if self.lora else \
              {k: v.float().cpu() for k, v in self.p.items()}
        for name in getattr(self, "q", {}):
            out[name] = self._w(name).float().cpu()
        if self.lora:
            for name in list(out):
                if name + ".lora_a" in self.p:
                    out[name] += self.lora_scale * (self.p[name + ".lora_b"].float() @ self.p[name + ".lora_a"].float()).cpu()
        return out

    def _proj(self, x, name: str, out, acts: dict, key: str):
        """out = x W^T (+ alpha / r * (x A^T) B^T when the projection carries an adapter)."""
        self.gemm(x, self._w(name), out=out)
        if self.lora and name + ".lora_a" in self.p:
            t = acts["t_" + key]
            self.gemm(self._dropped(x, name), self.p[name + ".lora_a"], out=t)
            self.gemm(t, self.p[name + ".lora_b"], alpha=self.lora_scale, resid=out, out=out)
        return out

    def _proj_backward(self, dy, x, name: str, dx_out, acts: dict, key: str):
        """dx_out = dy W (+ adapter path); weight gradients of whatever is trainable."""
        gemm, p, g = self.gemm, self.p, self.g
        gemm(dy, self._w(name), b_mn=True, out=dx_out)
        if not self.lora:
            gemm(dy, x, a_mn=True, b_mn=True, workspace=self.ws, out=g[name])
        elif name + ".lora_a" in p:
            t, s = acts["t_" + key], self.lora_scale
            gemm(dy, p[name + ".lora_b"], b_mn=True, alpha=s, out=self.d_t)                          # [N, r] = s * dy B
            gemm(dy, t, a_mn=True, b_mn=True, alpha=s, workspace=self.ws, out=g[name + ".lora_b"])  # [out, r] = s * dy^T t
            gemm(self.d_t, self._dropped(x, name), a_mn=True, b_mn=True, workspace=self.ws, out=g[name + ".lora_a"])   # [r, in] = d_t^T drop(x)
            if self.drop_on:
                dxd = self.drop_dx[:, :x.shape[1]]
                gemm(self.d_t, p[name + ".lora_a"], b_mn=True, out=dxd)                              # d drop(x) = d_t A
                self.K.dropout_apply(dxd, dx_out, self.drop_p, seed=self.cfg.base_seed, stream_id=self.drop_ids[name], step=self.drop_step,
                                     accumulate=True)                                                 # dx += mask * d drop(x) / (1 - p)
            else:
                gemm(self.d_t, p[name + ".lora_a"], b_mn=True, resid=dx_out, out=dx_out)            # + d_t A
        return dx_out

    def _dropped(self, x: torch.Tensor, name: str) -> torch.Tensor:
        """The adapter branch's input: x itself, or x under this pass's dropout mask of projection ``name`` (in a scratch buffer
        valid until the next call)."""
        if not self.drop_on:
            return x
        xd = self.drop_x[:, :x.shape[1]]
        return self.K.dropout_apply(x, xd, self.drop_p, seed=self.cfg.base_seed, stream_id=self.drop_ids[name], step=self.drop_step)

    def _gw(self, name: str):
        """Gradient slot of a base tensor: None (= not computed) when only adapters train."""
        return None if self.lora else self.g[name]

    def set_ppo_batch(self, logp_old: torch.Tensor, advantages: torch.Tensor, returns: torch.Tensor, value_old: torch.Tensor) -> None:
        """Per-row rollout records [B, T] (rows that do not count are masked by ``set_loss_mask``)."""
        for i, t in enumerate((logp_old, advantages, returns, value_old)):
            self.ppo_in[i].copy_(t.reshape(-1).to(self.ppo_in.dtype), non_blocking=True)

    def _views(self, t):
        cfg = self.cfg
        q_end, k_end = cfg.n_head * cfg.head_dim, (cfg.n_head + cfg.n_kv_head) * cfg.head_dim
        return t[:, :q_end], t[:, q_end:k_end], t[:, k_end:cfg.qkv_dim], t[:, cfg.qkv_dim:]

    # -------------------------------------------------------------------------- forward --
    def _layer_forward(self, l: int, a: dict, x: torch.Tensor) -> torch.Tensor:
        K, I, cfg, p = self.K, self.I, self.cfg, self.p
        B, T = self.B, self.T
        Hq, Hkv, hd, Fd = cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.d_ff
        rms = dict(mode=K.NORM_RMS, mean=self.mean_scratch)
        pre, local = f"layers.{l}.", cfg.is_local(l)
        K.norm_forward(x, p[pre + "attn_norm"], None, eps=cfg.norm_eps, centered=True, out=a["n1"], rstd=a["r1"], **rms)
        self._proj(a["n1"], pre + "wqkvg", a["qkvg"], a, "wqkvg")
        K.qk_norm_forward(a["qkvg"], Hq, Hkv, hd, eps=cfg.qk_norm_eps, q_scale=cfg.q_scale, rstd=a["qk_rstd"])
        if local:
            I.rope_inplace(a["qkvg"], T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=self.cos, sin=self.sin, convention="hf")
        q, k, v, gate = self._views(a["qkvg"])
        K.attention_forward(q, k, v, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, causal=True,
                            window=cfg.window if local else 0, out=a["att"], lse=a["lse"])
        K.sigmoid_gate_forward(a["att"], gate, a["attg"])
        self._proj(a["attg"], pre + "wo", a["br"], a, "wo")
        K.norm_forward(a["br"], p[pre + "post_attn_norm"], None, eps=cfg.post_norm_eps, centered=True, out=self.nb, rstd=a["rp1"], **rms)
        torch.add(x, self.nb, out=a["x1"])
        K.norm_forward(a["x1"], p[pre + "mlp_norm"], None, eps=cfg.norm_eps, centered=True, out=a["n2"], rstd=a["r2"], **rms)
        self._proj(a["n2"], pre + "w_gate_up", a["gu"], a, "w_gate_up")
        I.swiglu_forward(a["gu"], Fd, out=a["h"])
        self._proj(a["h"], pre + "w_down", a["mb"], a, "w_down")
        K.norm_forward(a["mb"], p[pre + "post_mlp_norm"], None, eps=cfg.post_norm_eps, centered=True, out=self.nb, rstd=a["rp2"], **rms)
        torch.add(a["x1"], self.nb, out=a["x2"])
        return a["x2"]

    def forward(self, *, compute_grad_logits: bool = True, grad_scale: float | None = None) -> torch.Tensor:
        K, I, gemm, cfg, p = self.K, self.I, self.gemm, self.cfg, self.p
        B, T, N = self.B, self.T, self.B * self.T
        Hq, Hkv, hd, Fd = cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.d_ff
        rms = dict(mode=K.NORM_RMS, mean=self.mean_scratch)
        self.drop_on = self.drop_p > 0.0 and compute_grad_logits              # adapter dropout: training passes only
        if self.drop_on:
            K.counter_add(self.drop_step.view(torch.int32)[:1], 1)           # new masks for this pass, also when a graph replays it
        if cfg.pp_first:
            K.embedding_forward(self.tokens, p["tok_embeddings"], None, T=T, out=self.xe)
            K.norm_forward(self.xe, self.ones, None, eps=cfg.norm_eps, out=self.x0, rstd=self.re, **rms)
        x = self.x0  # later stages: filled by the pipeline runtime with the previous stage's output
        k = len(self.acts)
        for i, l in enumerate(self.layers):
            if i and i % k == 0:
                self.bound[i // k].copy_(x)      # the slot that holds x is reused by the layers of this segment
                x = self.bound[i // k]
            x = self._layer_forward(l, self.acts[i % k], x)
        if not cfg.pp_last:
            return x  # handed to the next stage
        K.norm_forward(x, p["norm"], None, eps=cfg.norm_eps, out=self.nf, rstd=self.rf, **rms)
        if self.objective == "reward_model":
            return self._reward_loss()
        if self.objective == "ppo":
            torch.mv(self.nf.float(), p["value_head"].float(), out=self.values)
        if cfg.logit_softcap > 0:
            gemm(self.nf, p["lm_head"], act="tanh_cap", act_param=cfg.logit_softcap, alpha=cfg.output_multiplier, out=self.logits)
        else:
            gemm(self.nf, p["lm_head"], alpha=cfg.output_multiplier, out=self.logits)
        return self._loss(compute_grad_logits, grad_scale)

    def _ce(self, write_grad: bool, grad_scale: float, loss_scale: float, row_scale, z: float | None = None) -> None:
        cfg = self.cfg
        self.K.cross_entropy(self.logits, self.targets, vocab=cfg.vocab_size, cap=cfg.logit_softcap,
                             z_coef=cfg.z_loss if z is None else z, grad_scale=grad_scale,
                             loss_scale=loss_scale, row_scale=row_scale, write_grad=write_grad, row_loss=self.row_loss, mean_loss=self.loss)

    def _loss(self, compute_grad: bool, grad_scale: float | None) -> torch.Tensor:
        N = self.B * self.T
        if self.objective == "ar":
            self._ce(compute_grad, 1.0 / N if grad_scale is None else grad_scale, 1.0 / N, None)
            return self.loss
        if self.objective == "sft":
            # masked mean: every counted row weighs 1 / (number of counted rows)
            torch.div(self.loss_mask, self.loss_mask.sum().clamp(min=1.0), out=self.row_scale)
            self._ce(compute_grad, 1.0 if grad_scale is None else grad_scale * N, 1.0, self.row_scale)
            return self.loss
        if self.objective == "ppo":
            return self._ppo_loss(compute_grad, grad_scale)
        # DPO: pass 1 leaves the logits intact and yields the row losses = -log p(target)
        self._ce(False, 1.0, 1.0, None, z=0.0)
        half = self.B // 2
        torch.sum((self.row_loss * self.loss_mask).view(self.B, self.T), dim=1, out=self.seq_logps)
        self.seq_logps.neg_()
        pol, ref = self.seq_logps, self.ref_logps
        margin = self.cfg.dpo_beta * ((pol[:half] - pol[half:]) - (ref[:half] - ref[half:]))
        per, d_per = dpo_pair_terms(margin, beta=self.cfg.dpo_beta, loss_type=self.cfg.dpo_loss_type, label_smoothing=self.cfg.dpo_label_smoothing)
        self.dpo_stats[0] = per.mean()
        self.dpo_stats[1] = (margin > 0).float().mean()
        self.dpo_stats[2] = margin.mean()
        self.loss.copy_(self.dpo_stats[:1])
        if compute_grad:
            # d loss / d logp_chosen = beta * (d loss / d z) / pairs, the opposite for rejected; logp = -sum(row loss)
            coef = -self.cfg.dpo_beta * d_per / half
            per_seq = torch.cat([coef, -coef])                      # d loss / d (sum of row losses) per sequence
            torch.mul(self.loss_mask.view(self.B, self.T), per_seq.unsqueeze(1), out=self.row_scale.view(self.B, self.T))
            keep = self.loss.clone()
            self._ce(True, 1.0 if grad_scale is None else grad_scale * N, 1.0, self.row_scale, z=0.0)
            self.loss.copy_(keep)                                   # the kernel's own mean is not the DPO loss
        return self.loss

    def _ppo_loss(self, compute_grad: bool, grad_scale: float | None) -> torch.Tensor:
        """Clipped surrogate + clipped value loss over the counted rows; leaves d loss / d logits in the logits buffer and
        d loss / d value per row in ``self._d_value`` when ``compute_grad``."""
        cfg, N = self.cfg, self.B * self.T
        self._ce(False, 1.0, 1.0, None, z=0.0)                      # row losses = -log p(action)
        logp_old, adv, ret, v_old = self.ppo_in
        out = ppo_terms_and_gradients(-self.row_loss, logp_old, adv, ret, self.values, v_old, self.loss_mask, clip=cfg.ppo_clip,
                                      vf_coef=cfg.ppo_vf_coef, normalize_advantages=cfg.ppo_normalize_advantages)
        self.ppo_stats.copy_(torch.stack([out["policy_loss"], out["value_loss"], out["clip_fraction"], out["approx_kl"]]))
        self.loss.copy_(out["loss"].reshape(1))
        if compute_grad:
            gs = 1.0 if grad_scale is None else grad_scale * N
            # log p = -(row loss): the loss kernel's per-row scale is -d loss / d log p
            torch.neg(out["d_logp"], out=self.row_scale)
            self._d_value = out["d_value"] * gs
            keep = self.loss.clone()
            self._ce(True, gs, 1.0, self.row_scale, z=0.0)
            self.loss.copy_(keep)
        return self.loss

    def _reward_rows(self) -> torch.Tensor:
        """Flat row index of the last counted position of every sequence (a sequence without one reads position 0)."""
        pos = torch.arange(self.T, device=self.loss_mask.device)
        last = torch.where(self.loss_mask.view(self.B, self.T) > 0, pos, -1).amax(1).clamp(min=0)
        return last + torch.arange(self.B, device=last.device) * self.T

    def _reward_loss(self) -> torch.Tensor:
        half = self.B // 2
        rows = self._reward_rows()
        r = self.nf[rows].float() @ self.p["reward_head"].float()
        margin = r[:half] - r[half:]
        self.seq_logps.copy_(r)                                 # the rewards, chosen then rejected
        self.dpo_stats[0] = torch.nn.functional.softplus(-margin).mean()
        self.dpo_stats[1] = (margin > 0).float().mean()
        self.dpo_stats[2] = margin.mean()
        self.loss.copy_(self.dpo_stats[:1])
        coef = torch.sigmoid(-margin) / half
        self._d_reward = torch.cat([-coef, coef])               # d loss / d reward per sequence
        return self.loss

    def _reward_backward(self) -> None:
        """d(final-norm output) has one non-zero row per sequence; the vocabulary head gets no gradient."""
        rows, dr = self._reward_rows(), self._d_reward
        self.d_n.zero_()
        self.d_n[rows] = (dr[:, None] * self.p["reward_head"].float()[None, :]).to(self.d_n.dtype)
        self.g["reward_head"].copy_((dr[:, None] * self.nf[rows].float()).sum(0))
        if "value_head" in self.g:
            self.g["value_head"].zero_()
        if not self.lora:
            self.g["lm_head"].zero_()

    # ------------------------------------------------------------------------- backward --
    def _layer_backward(self, l: int, a: dict, x_in: torch.Tensor, dx: torch.Tensor, spare: torch.Tensor):
        """Gradients of one layer. ``dx`` is d(layer output); returns (d(layer input), the other scratch buffer)."""
        K, I, cfg, p = self.K, self.I, self.cfg, self.p
        B, T = self.B, self.T
        Hq, Hkv, hd, Fd = cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.d_ff
        sc, rms = self.scratch, dict(mode=K.NORM_RMS)
        pre, local = f"layers.{l}.", cfg.is_local(l)
        # MLP sandwich: x2 = x1 + post_norm(w_down(swiglu(w_gate_up(norm(x1)))))
        K.norm_backward(dx, a["mb"], p[pre + "post_mlp_norm"], None, a["rp2"], self._gw(pre + "post_mlp_norm"), None, sc, centered=True,
                        out=self.d_br, **rms)
        self._proj_backward(self.d_br, a["h"], pre + "w_down", self.d_h, a, "w_down")
        I.swiglu_backward(a["gu"], self.d_h, Fd, out=self.d_gu)
        self._proj_backward(self.d_gu, a["n2"], pre + "w_gate_up", self.d_n, a, "w_gate_up")
        K.norm_backward(self.d_n, a["x1"], p[pre + "mlp_norm"], None, a["r2"], self._gw(pre + "mlp_norm"), None, sc, centered=True, dresid=dx,
                        out=spare, **rms)
        dx, spare = spare, dx
        # attention sandwich: x1 = x + post_norm(wo(att * sigmoid(gate)))
        K.norm_backward(dx, a["br"], p[pre + "post_attn_norm"], None, a["rp1"], self._gw(pre + "post_attn_norm"), None, sc, centered=True,
                        out=self.d_br, **rms)
        self._proj_backward(self.d_br, a["attg"], pre + "wo", self.d_attg, a, "wo")
        q, k, v, gate = self._views(a["qkvg"])
        dq, dk, dv, dgate = self._views(self.d_qkvg)
        K.sigmoid_gate_backward(self.d_attg, a["att"], gate, self.d_att, dgate)
        K.attention_backward(self.d_att, q, k, v, a["att"], a["lse"], B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, causal=True,
                             window=cfg.window if local else 0, dq=dq, dk=dk, dv=dv, delta=self.delta)
        if local:
            I.rope_inplace(self.d_qkvg, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=self.cos, sin=self.sin, convention="hf",
                           backward=True)
            # the norm backward needs the normalised, un-rotated q / k: undo the rotation of the saved copy
            I.rope_inplace(a["qkvg"], T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, cos=self.cos, sin=self.sin, convention="hf",
                           backward=True)
        K.qk_norm_backward(self.d_qkvg, a["qkvg"], a["qk_rstd"], Hq, Hkv, hd, q_scale=cfg.q_scale)
        self._proj_backward(self.d_qkvg, a["n1"], pre + "wqkvg", self.d_n, a, "wqkvg")
        K.norm_backward(self.d_n, x_in, p[pre + "attn_norm"], None, a["r1"], self._gw(pre + "attn_norm"), None, sc, centered=True, dresid=dx,
                        out=spare, **rms)
        dx, spare = spare, dx
        return dx, spare

    def backward(self) -> None:
        K, I, gemm, cfg, p, g = self.K, self.I, self.gemm, self.cfg, self.p, self.g
        B, T = self.B, self.T
        Hq, Hkv, hd, Fd = cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.d_ff
        sc, ws, mult = self.scratch, self.ws, cfg.output_multiplier
        rms = dict(mode=K.NORM_RMS)
        dx, spare = self.d_a, self.d_b  # later stages: d_a was filled with the next stage's input gradient
        if cfg.pp_last:
            if self.objective == "reward_model":
                self._reward_backward()
            else:
                gemm(self.logits, p["lm_head"], b_mn=True, alpha=mult, out=self.d_n)
                if not self.lora:
                    gemm(self.logits, self.nf, a_mn=True, b_mn=True, alpha=mult, out=g["lm_head"])
                if "reward_head" in g:
                    g["reward_head"].zero_()
                if self.objective == "ppo":
                    # the value head reads the same final-norm rows: its gradient joins theirs
                    self.d_n.add_((self._d_value[:, None] * p["value_head"].float()[None, :]).to(self.d_n.dtype))
                    g["value_head"].copy_(torch.mv(self.nf.float().t(), self._d_value))
                elif "value_head" in g:
                    g["value_head"].zero_()
            x_last = self.acts[(len(self.layers) - 1) % len(self.acts)]["x2"] if self.acts else self.x0
            K.norm_backward(self.d_n, x_last, p["norm"], None, self.rf, self._gw("norm"), None, sc, out=dx, **rms)
        k, L = len(self.acts), len(self.layers)
        for seg in range((L - 1) // k if L else -1, -1, -1):
            lo, hi = seg * k, min(L, seg * k + k)
            if hi != L:
                # the slots hold a later segment by now: run this segment's forward again from its saved input
                x = self.bound[seg]
                for i in range(lo, hi):
                    x = self._layer_forward(self.layers[i], self.acts[i % k], x)
            for i in range(hi - 1, lo - 1, -1):
                x_in = self.acts[(i - 1) % k]["x2"] if i > lo else self.bound[seg]
                dx, spare = self._layer_backward(self.layers[i], self.acts[i % k], x_in, dx, spare)
        self.d_input = dx  # gradient w.r.t. this stage's input (sent to the previous stage)
        if cfg.pp_first and not self.lora:
            # weightless norm of the embeddings, then the scatter into the table
            K.norm_backward(dx, self.xe, self.ones, None, self.re, None, None, sc, out=spare, **rms)
            g["tok_embeddings"].zero_()
            st_, od_ = K.sort_tokens(self.tokens, self.tok_sorted, self.tok_order)
            K.embedding_backward(spare, self.tokens, g["tok_embeddings"], None, B=B, T=T, sorted_tokens=st_, order=od_)

    def logits_view(self) -> torch.Tensor:
        return self.logits.view(self.B, self.T, -1)[..., :self.cfg.vocab_size]

    @torch.no_grad()
    def sequence_logps(self, tokens: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """[B] masked sequence log-probabilities of a batch under the CURRENT parameters (forward only): what a
        frozen copy of the model contributes as the DPO reference."""
        keep = self.objective
        self.set_batch(tokens, targets)
        self.set_loss_mask(mask)
        self.objective = "dpo"
        self.forward(compute_grad_logits=False)
        self.objective = keep
        return self.seq_logps.clone()
