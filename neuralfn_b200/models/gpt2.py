"""Dense GPT-2 family (gpt2, gpt2_zloss, gpt2_softcap, gpt2_qknorm, gpt2_stable) as an
explicit forward/backward engine over the sm_100a kernel library.

The engine owns flat bf16 parameter and gradient buffers (so the data-parallel
reduce-scatter/AdamW kernels can address them by offset), per-layer activation
stashes, and issues every kernel of a training step itself - there is no autograd
tape in the hot path, which makes the whole step capturable in one CUDA graph.

Layer math and variant semantics follow the reference's native dense trainer
(``neuralfn/csrc/native_gpt2/nfn_gpt2_native_train.cpp:25816-25965`` forward block,
``:771-789`` variants, init ``:23194-23240``): pre-LN blocks, tanh-GELU, tied LM head
over a vocabulary padded to a multiple of 64... (50257 -> 50304), weightless per-head
RMS on Q and K after the bias when ``qk_norm``, ``cap*tanh(logit/cap)`` when
``logit_softcap``, and ``z * lse^2`` added to the token loss when ``z_loss``.
A plain PyTorch fp32 implementation of the same math (``reference_forward``) is the
oracle for the tests and the CPU path.
"""
from __future__ import annotations

import contextlib
import math
from dataclasses import dataclass, field
from typing import Iterator

import torch
import torch.nn.functional as F

__all__ = ["GPT2Config", "ParamSpec", "gpt2_param_specs", "FlatLayout", "GPT2Engine",
           "reference_forward", "init_gpt2_params_"]


@dataclass
class GPT2Config:
    n_layer: int = 12
    n_head: int = 12
    d_model: int = 768
    vocab_size: int = 50257
    max_seq_len: int = 1024
    mlp_mult: int = 4
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    logit_softcap: float = 0.0
    z_loss: float = 0.0
    ln_eps: float = 1e-5
    vocab_pad_to: int = 128
    differential: bool = False          # differential attention (two softmaxes on the halves of each head)
    diff_lambda_init: float = 0.8
    diff_norm_eps: float = 1e-5
    mlp_activation: str = "gelu"        # gelu (tanh form) | relu | silu | relu2
    # mixture of activations: at step 1 and every `moa_interval` steps each candidate's loss is probed on the current
    # batch over the SHARED weights and training continues with the lowest (empty = single activation)
    moa_activations: tuple = ()
    moa_interval: int = 50

    @property
    def padded_vocab(self) -> int:
        p = self.vocab_pad_to
        return (self.vocab_size + p - 1) // p * p

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_head

    # hooks used by trainers.dense_gpt.DenseGPTTrainer (every model family provides them)
    def param_specs(self) -> "list[ParamSpec]":
        return gpt2_param_specs(self) + diff_param_specs(self)

    def init_params_(self, layout: "FlatLayout", master: torch.Tensor, seed: int) -> None:
        init_gpt2_params_(self, layout, master, seed)

    def make_engine(self, layout, params, grads, batch: int, seq: int) -> "GPT2Engine":
        return GPT2Engine(self, layout, params, grads, batch, seq)

    @classmethod
    def variant(cls, name: str, **kw) -> "GPT2Config":
        """Named dense variants: defaults z=1e-4, cap=30, qk-norm as in the reference presets
        (``neuralfn/config.py:900-949``)."""
        table = {
            "gpt2": {},
            "gpt2_zloss": {"z_loss": 1e-4},
            "gpt2_softcap": {"logit_softcap": 30.0},
            "gpt2_qknorm": {"qk_norm": True},
            "gpt2_stable": {"qk_norm": True, "z_loss": 1e-4},
            "gpt2_qknorm_softcap_zloss": {"qk_norm": True, "logit_softcap": 30.0, "z_loss": 1e-4},
            "gpt2_diff": {"differential": True, "diff_lambda_init": 0.8},
            "gpt2_moa": {"moa_activations": ("gelu", "relu", "silu", "relu2"), "moa_interval": 50},
        }
        if name not in table:
            raise KeyError(f"unknown dense GPT variant {name!r}")
        return cls(**{**table[name], **kw})


MLP_ACTIVATIONS = ("gelu", "relu", "silu", "relu2")      # pointwise, weight-preserving: they share c_fc / c_proj


def mlp_activation_reference(x: torch.Tensor, name: str) -> torch.Tensor:
    import torch.nn.functional as F
    if name == "gelu":
        return F.gelu(x, approximate="tanh")
    if name == "relu":
        return F.relu(x)
    if name == "silu":
        return F.silu(x)
    if name == "relu2":
        return F.relu(x).square()
    raise ValueError(f"unknown MLP activation {name!r} (one of {MLP_ACTIVATIONS})")


@dataclass(frozen=True)
class ParamSpec:
    name: str
    shape: tuple[int, ...]
    decay: bool
    init: str  # "normal" | "resid" | "zeros" | "ones"

    @property
    def numel(self) -> int:
        return math.prod(self.shape)


def gpt2_param_specs(cfg: GPT2Config) -> list[ParamSpec]:
    """Tensors in dense-checkpoint order (wte, wpe, per layer ..., ln_f)."""
    C, L, Vp, T = cfg.d_model, cfg.n_layer, cfg.padded_vocab, cfg.max_seq_len
    H = cfg.mlp_mult * C
    specs = [ParamSpec("wte", (Vp, C), True, "normal"), ParamSpec("wpe", (T, C), True, "normal")]
    for l in range(L):
        p = f"h.{l}."
        specs += [
            ParamSpec(p + "ln_1.weight", (C,), False, "ones"), ParamSpec(p + "ln_1.bias", (C,), False, "zeros"),
            ParamSpec(p + "attn.c_attn.weight", (3 * C, C), True, "normal"),
            ParamSpec(p + "attn.c_attn.bias", (3 * C,), False, "zeros"),
            ParamSpec(p + "attn.c_proj.weight", (C, C), True, "resid"),
            ParamSpec(p + "attn.c_proj.bias", (C,), False, "zeros"),
            ParamSpec(p + "ln_2.weight", (C,), False, "ones"), ParamSpec(p + "ln_2.bias", (C,), False, "zeros"),
            ParamSpec(p + "mlp.c_fc.weight", (H, C), True, "normal"),
            ParamSpec(p + "mlp.c_fc.bias", (H,), False, "zeros"),
            ParamSpec(p + "mlp.c_proj.weight", (C, H), True, "resid"),
            ParamSpec(p + "mlp.c_proj.bias", (C,), False, "zeros"),
        ]
    specs += [ParamSpec("ln_f.weight", (C,), False, "ones"), ParamSpec("ln_f.bias", (C,), False, "zeros")]
    return specs


def diff_param_specs(cfg: GPT2Config) -> list[ParamSpec]:
    """Side parameters of the differential variant: one learned lambda per layer, kept in an 8-element
    (16-byte) slot of the flat buffers (element 0 is the value). They are not part of the dense model
    file; checkpoints carry them as ``diff_parameters_*.bin`` / ``diff_optimizer_*.bin`` sidecars, as the
    reference does (``neuralfn/csrc/native_gpt2/nfn_gpt2_native_train.cpp:4402-4430``)."""
    if not cfg.differential:
        return []
    return [ParamSpec(f"h.{l}.attn.diff_lambda", (8,), False, "lambda") for l in range(cfg.n_layer)]


class FlatLayout:
    """Offsets of named tensors inside one flat buffer: all weight-decayed tensors
    first, then the rest, each start aligned to 8 elements (16 bytes for bf16) and the
    total padded so it splits evenly into ``world`` shards of a multiple of 8."""

    def __init__(self, specs: list[ParamSpec], world: int = 1, align: int = 8) -> None:
        self.specs = {s.name: s for s in specs}
        self.order = [s for s in specs if s.decay] + [s for s in specs if not s.decay]
        self.offsets: dict[str, int] = {}
        cur = 0
        for s in self.order:
            if not s.decay and "n_decay" not in self.__dict__:
                self.n_decay = cur
            self.offsets[s.name] = cur
            cur += (s.numel + align - 1) // align * align
        if "n_decay" not in self.__dict__:
            self.n_decay = cur
        self.n_used = cur
        quantum = align * world
        self.n_total = (cur + quantum - 1) // quantum * quantum
        self.world = world
        self.shard = self.n_total // world

    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        s = self.specs[name]
        o = self.offsets[name]
        return flat[o:o + s.numel].view(*s.shape)

    def views(self, flat: torch.Tensor) -> dict[str, torch.Tensor]:
        return {s.name: self.view(flat, s.name) for s in self.order}


def init_gpt2_params_(cfg: GPT2Config, layout: FlatLayout, master: torch.Tensor, seed: int = 1337) -> None:
    """gpt2-normal initialisation into an fp32 flat buffer: N(0, 0.02) for embeddings and
    input projections, N(0, 0.02/sqrt(2L)) for the two residual projections, zero biases,
    unit LayerNorm weights, zero rows for the vocabulary padding."""
    gen = torch.Generator(device=master.device)
    gen.manual_seed(seed)
    master.zero_()
    for s in layout.order:
        v = layout.view(master, s.name)
        if s.init == "normal":
            v.normal_(0.0, 0.02, generator=gen)
        elif s.init == "resid":
            v.normal_(0.0, 0.02 / math.sqrt(2 * cfg.n_layer), generator=gen)
        elif s.init == "ones":
            v.fill_(1.0)
        elif s.init == "lambda":
            v[0] = cfg.diff_lambda_init
    layout.view(master, "wte")[cfg.vocab_size:].zero_()


# ------------------------------------------------------------------------ oracle --
def reference_forward(cfg: GPT2Config, params: dict[str, torch.Tensor], tokens: torch.Tensor,
                      targets: torch.Tensor | None = None, activation: str | None = None):
    """Plain PyTorch restatement (any dtype/device). Returns (loss, logits[B,T,V]). ``activation`` overrides the
    configured MLP activation (what a mixture-of-activations run has currently selected)."""
    B, T = tokens.shape
    C, nh, hd = cfg.d_model, cfg.n_head, cfg.head_dim
    x = params["wte"][tokens] + params["wpe"][:T]
    for l in range(cfg.n_layer):
        p = f"h.{l}."
        h = F.layer_norm(x, (C,), params[p + "ln_1.weight"], params[p + "ln_1.bias"], cfg.ln_eps)
        qkv = F.linear(h, params[p + "attn.c_attn.weight"], params[p + "attn.c_attn.bias"])
        q, k, v = (t.view(B, T, nh, hd).transpose(1, 2) for t in qkv.split(C, dim=-1))
        if cfg.qk_norm:
            q = q * torch.rsqrt(q.float().pow(2).mean(-1, keepdim=True) + cfg.qk_norm_eps).to(q.dtype)
            k = k * torch.rsqrt(k.float().pow(2).mean(-1, keepdim=True) + cfg.qk_norm_eps).to(k.dtype)
        if cfg.differential:
            half = hd // 2
            a1 = F.scaled_dot_product_attention(q[..., :half], k[..., :half], v, is_causal=True)
            a2 = F.scaled_dot_product_attention(q[..., half:], k[..., half:], v, is_causal=True)
            d = a1 - params[p + "attn.diff_lambda"][0].to(a1.dtype) * a2
            a = (d.float() * torch.rsqrt(d.float().pow(2).mean(-1, keepdim=True) + cfg.diff_norm_eps)).to(d.dtype) * (1.0 - cfg.diff_lambda_init)
        else:
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        a = a.transpose(1, 2).reshape(B, T, C)
        x = x + F.linear(a, params[p + "attn.c_proj.weight"], params[p + "attn.c_proj.bias"])
        h = F.layer_norm(x, (C,), params[p + "ln_2.weight"], params[p + "ln_2.bias"], cfg.ln_eps)
        h = mlp_activation_reference(F.linear(h, params[p + "mlp.c_fc.weight"], params[p + "mlp.c_fc.bias"]), activation or cfg.mlp_activation)
        x = x + F.linear(h, params[p + "mlp.c_proj.weight"], params[p + "mlp.c_proj.bias"])
    x = F.layer_norm(x, (C,), params["ln_f.weight"], params["ln_f.bias"], cfg.ln_eps)
    logits = F.linear(x, params["wte"])[..., :cfg.vocab_size]
    if cfg.logit_softcap > 0:
        logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
    loss = None
    if targets is not None:
        lf = logits.float().view(-1, cfg.vocab_size)
        lse = torch.logsumexp(lf, dim=-1)
        tv = lf.gather(1, targets.view(-1, 1).long()).squeeze(1)
        loss = (lse - tv + cfg.z_loss * lse * lse).mean()
    return loss, logits


# ------------------------------------------------------------------------ engine --
@dataclass
class _LayerActs:
    ln1: torch.Tensor
    ln1_mean: torch.Tensor
    ln1_rstd: torch.Tensor
    qkv: torch.Tensor
    qk_rstd: torch.Tensor | None
    att: torch.Tensor
    lse: torch.Tensor
    x1: torch.Tensor
    ln2: torch.Tensor
    ln2_mean: torch.Tensor
    ln2_rstd: torch.Tensor
    fc_pre: torch.Tensor
    fc_act: torch.Tensor
    x2: torch.Tensor
    diff_a: torch.Tensor | None = None      # differential variant: both attentions' outputs [N, 2C]
    diff_rstd: torch.Tensor | None = None


class GPT2Engine:
    """Forward/backward of the dense GPT over preallocated buffers (CUDA only).

    ``params``/``grads`` are flat bf16 buffers supplied by the caller (plain CUDA
    tensors, or symmetric-memory tensors when data parallel); the optimizer lives in
    ``neuralfn_b200.parallel.dp``.
    """

    def __init__(self, cfg: GPT2Config, layout: FlatLayout, params: torch.Tensor, grads: torch.Tensor,
                 batch: int, seq: int) -> None:
        from ..ops import kernels as K
        from ..ops.gemm import gemm
        self.K, self.gemm = K, gemm
        self.cfg, self.layout = cfg, layout
        self.B, self.T = batch, seq
        if seq > cfg.max_seq_len:
            raise ValueError("sequence longer than max_seq_len")
        self.params, self.grads = params, grads
        self.p = layout.views(params)
        self.g = layout.views(grads)
        dev = params.device
        N, C, Hd = batch * seq, cfg.d_model, cfg.mlp_mult * cfg.d_model
        bf, f32 = torch.bfloat16, torch.float32
        e = lambda *s, dtype=bf: torch.empty(*s, device=dev, dtype=dtype)  # noqa: E731
        self.x0 = e(N, C)
        self.acts = [
            _LayerActs(ln1=e(N, C), ln1_mean=e(N, dtype=f32), ln1_rstd=e(N, dtype=f32), qkv=e(N, 3 * C),
                       qk_rstd=e(N, 2 * cfg.n_head, dtype=f32) if cfg.qk_norm else None, att=e(N, C),
                       lse=e(batch, cfg.n_head * (2 if cfg.differential else 1), seq, dtype=f32), x1=e(N, C), ln2=e(N, C),
                       ln2_mean=e(N, dtype=f32), ln2_rstd=e(N, dtype=f32), fc_pre=e(N, Hd),
                       fc_act=e(N, Hd), x2=e(N, C),
                       diff_a=e(N, 2 * C) if cfg.differential else None,
                       diff_rstd=e(N * cfg.n_head, dtype=f32) if cfg.differential else None)
            for _ in range(cfg.n_layer)]
        if cfg.differential:
            if cfg.head_dim not in (64, 128):
                raise ValueError("the differential variant needs head_dim 64 or 128")
            # every head runs as two zero-padded pseudo-heads through the ordinary flash kernels
            self.q2, self.d_a2, self.dq2 = e(N, 2 * C), e(N, 2 * C), e(N, 2 * C)
            self.diff_partial = e(K.diff_partials(), dtype=f32)
        self.lnf = e(N, C)
        self.lnf_mean, self.lnf_rstd = e(N, dtype=f32), e(N, dtype=f32)
        self.logits = e(N, cfg.padded_vocab)
        self.row_loss = e(N, dtype=f32)
        self.loss = torch.zeros(1, device=dev, dtype=f32)
        # backward temporaries (shared by all layers)
        self.d_res_a, self.d_res_b = e(N, C), e(N, C)
        self.d_ln = e(N, C)
        self.d_fc = e(N, Hd)
        self.d_qkv = e(N, 3 * C)
        self.d_att = e(N, C)
        self.delta = e(batch, cfg.n_head * (2 if cfg.differential else 1), seq, dtype=f32)
        self.dq_accum = e(N, C, dtype=f32)
        self.scratch = e(max(64 * 2 * max(Hd, 3 * C), K.norm_fused_rows() * 3 * C), dtype=f32)
        self.ws = e(32 * 1024 * 1024, dtype=f32)  # split-K partial slices of the weight-gradient GEMMs
        self.tokens = torch.zeros(N, device=dev, dtype=torch.int32)
        self.tok_sorted = torch.zeros(N, device=dev, dtype=torch.int32)      # stable sort of the batch's tokens: the token-embedding gradient
        self.tok_order = torch.zeros(N, device=dev, dtype=torch.int64)       # sums equal tokens in row order (bitwise reproducible)
        self.targets = torch.zeros(N, device=dev, dtype=torch.int32)
        self.timer = None  # optional utils.stage_timing.StageTimer (eager runs only)
        # MLP activation in effect (epilogue name of the FC GEMM and its derivative in the projection's input-gradient GEMM)
        if cfg.mlp_activation not in MLP_ACTIVATIONS or any(a not in MLP_ACTIVATIONS for a in cfg.moa_activations):
            raise ValueError(f"MLP activations must come from {MLP_ACTIVATIONS}")
        self.activation = cfg.moa_activations[0] if cfg.moa_activations else cfg.mlp_activation
        self.moa = {"probe_runs": 0, "candidate_evals": 0, "selected_activation_changes": 0, "last_probe_losses": {}, "history": []}
        # data-parallel overlap: called as hook(lo, hi) from the backward pass as soon as the weight
        # gradients of a group of layers (one contiguous flat range) are final
        self.grad_ready_hook = None
        self.grad_bucket_layers = max(1, -(-cfg.n_layer // 6))

    def _layer_range(self, l_lo: int, l_hi: int) -> tuple[int, int]:
        """Flat range of the decayed weights of layers l_lo..l_hi (inclusive)."""
        lay = self.layout
        last = f"h.{l_hi}.mlp.c_proj.weight"
        hi = lay.offsets[last] + (lay.specs[last].numel + 7) // 8 * 8
        return lay.offsets[f"h.{l_lo}.attn.c_attn.weight"], hi

    def _stage(self, name: str):
        t = self.timer
        return t.stage(name) if t is not None and t.enabled else contextlib.nullcontext()

    # ------------------------------------------------------------------ forward --
    def forward(self, *, compute_grad_logits: bool = True, grad_scale: float | None = None) -> torch.Tensor:
        """Runs on ``self.tokens``/``self.targets``. Leaves d(loss)/d(logits) in ``self.logits``
        when ``compute_grad_logits``; returns the mean-loss tensor (device, fp32[1])."""
        K, gemm, cfg, p = self.K, self.gemm, self.cfg, self.p
        B, T, N = self.B, self.T, self.B * self.T
        C, nh, hd = cfg.d_model, cfg.n_head, cfg.head_dim
        st = self._stage
        with st("embedding_residual.forward"):
            K.embedding_forward(self.tokens, p["wte"], p["wpe"], T=T, out=self.x0)
        x = self.x0
        for l, a in enumerate(self.acts):
            pre = f"h.{l}."
            with st("block_forward"):
                with st("block_forward.attention.ln1"):
                    K.norm_forward(x, p[pre + "ln_1.weight"], p[pre + "ln_1.bias"], eps=cfg.ln_eps,
                                   mode=K.NORM_LAYER, out=a.ln1, mean=a.ln1_mean, rstd=a.ln1_rstd)
                with st("block_forward.attention.qkv"):
                    gemm(a.ln1, p[pre + "attn.c_attn.weight"], bias=p[pre + "attn.c_attn.bias"], out=a.qkv)
                if cfg.qk_norm:
                    with st("block_forward.attention.qk_norm"):
                        K.qk_norm_forward(a.qkv, nh, nh, hd, eps=cfg.qk_norm_eps, rstd=a.qk_rstd)
                with st("block_forward.attention.sdpa"):
                    if cfg.differential:
                        K.diff_q_expand(a.qkv[:, :C], self.q2, nh, hd)
                        K.attention_forward(self.q2, a.qkv[:, C:2 * C], a.qkv[:, 2 * C:], B=B, T=T, n_q_heads=2 * nh,
                                            n_kv_heads=nh, head_dim=hd, causal=True, scale=(hd // 2) ** -0.5,
                                            out=a.diff_a, lse=a.lse)
                        K.diff_combine(a.diff_a, p[pre + "attn.diff_lambda"], 1.0 - cfg.diff_lambda_init, cfg.diff_norm_eps,
                                       a.att, a.diff_rstd, nh, hd)
                    else:
                        K.attention_forward(a.qkv[:, :C], a.qkv[:, C:2 * C], a.qkv[:, 2 * C:], B=B, T=T,
                                            n_q_heads=nh, n_kv_heads=nh, head_dim=hd, causal=True,
                                            out=a.att, lse=a.lse)
                with st("block_forward.attention.proj_residual"):
                    gemm(a.att, p[pre + "attn.c_proj.weight"], bias=p[pre + "attn.c_proj.bias"], resid=x, out=a.x1)
                with st("block_forward.mlp.ln2"):
                    K.norm_forward(a.x1, p[pre + "ln_2.weight"], p[pre + "ln_2.bias"], eps=cfg.ln_eps,
                                   mode=K.NORM_LAYER, out=a.ln2, mean=a.ln2_mean, rstd=a.ln2_rstd)
                with st("block_forward.mlp.fc_gelu"):
                    gemm(a.ln2, p[pre + "mlp.c_fc.weight"], bias=p[pre + "mlp.c_fc.bias"], act=self.mlp_act,
                         save_pre=a.fc_pre, out=a.fc_act)
                with st("block_forward.mlp.proj_residual"):
                    gemm(a.fc_act, p[pre + "mlp.c_proj.weight"], bias=p[pre + "mlp.c_proj.bias"], resid=a.x1,
                         out=a.x2)
            x = a.x2
        with st("lm_head.final_norm"):
            K.norm_forward(x, p["ln_f.weight"], p["ln_f.bias"], eps=cfg.ln_eps, mode=K.NORM_LAYER,
                           out=self.lnf, mean=self.lnf_mean, rstd=self.lnf_rstd)
        with st("lm_head_backward.logits"):
            if cfg.logit_softcap > 0:
                gemm(self.lnf, p["wte"], act="tanh_cap", act_param=cfg.logit_softcap, out=self.logits)
            else:
                gemm(self.lnf, p["wte"], out=self.logits)
        with st("lm_head_backward.ce"):
            K.cross_entropy(self.logits, self.targets, vocab=cfg.vocab_size, cap=cfg.logit_softcap,
                            z_coef=cfg.z_loss, grad_scale=(1.0 / N if grad_scale is None else grad_scale),
                            loss_scale=1.0 / N, write_grad=compute_grad_logits, row_loss=self.row_loss,
                            mean_loss=self.loss)
        return self.loss

    # ----------------------------------------------------------------- backward --
    def backward(self) -> None:
        """Consumes d(logits) left by ``forward`` and writes every gradient (no accumulation:
        each call overwrites ``self.grads``)."""
        K, gemm, cfg, p, g = self.K, self.gemm, self.cfg, self.p, self.g
        B, T = self.B, self.T
        C, nh, hd = cfg.d_model, cfg.n_head, cfg.head_dim
        sc = self.scratch
        dlogits = self.logits
        st = self._stage
        # tied head: d(lnf) and d(wte)
        with st("lm_head_backward.dhidden"):
            gemm(dlogits, p["wte"], b_mn=True, out=self.d_ln)
        with st("lm_head_backward.dweight"):
            gemm(dlogits, self.lnf, a_mn=True, b_mn=True, out=g["wte"])
        x_last = self.acts[-1].x2 if self.acts else self.x0
        dx, spare = self.d_res_a, self.d_res_b
        L = cfg.n_layer
        # every norm backward also returns the column sum of the residual-stream gradient it
        # produces, which is the bias gradient of the projection that wrote that stream
        with st("final_norm_backward"):
            K.norm_backward(self.d_ln, x_last, p["ln_f.weight"], self.lnf_mean, self.lnf_rstd, g["ln_f.weight"], g["ln_f.bias"], sc,
                            mode=K.NORM_LAYER, out=dx, dx_colsum=g[f"h.{L - 1}.mlp.c_proj.bias"] if L > 0 else None)
        for l in range(cfg.n_layer - 1, -1, -1):
            a = self.acts[l]
            pre = f"h.{l}."
            x_in = self.acts[l - 1].x2 if l > 0 else self.x0
            with st("block_backward"):
                # ---- MLP branch: x2 = c_proj(gelu(c_fc(ln2))) + x1 ----
                with st("block_backward.mlp_proj.dinput"):
                    gemm(dx, p[pre + "mlp.c_proj.weight"], b_mn=True, act=self.mlp_act, dact_pre=a.fc_pre,
                         out=self.d_fc)
                with st("block_backward.mlp_proj.dweight_bias"):
                    gemm(dx, a.fc_act, a_mn=True, b_mn=True, workspace=self.ws, out=g[pre + "mlp.c_proj.weight"])
                with st("block_backward.mlp_fc.dinput"):
                    gemm(self.d_fc, p[pre + "mlp.c_fc.weight"], b_mn=True, out=self.d_ln)
                with st("block_backward.mlp_fc.dweight_bias"):
                    gemm(self.d_fc, a.ln2, a_mn=True, b_mn=True, workspace=self.ws, out=g[pre + "mlp.c_fc.weight"])
                    K.colsum(self.d_fc, g[pre + "mlp.c_fc.bias"], sc)
                with st("block_backward.ln2_residual.fused_affine_dinput_add"):
                    K.norm_backward(self.d_ln, a.x1, p[pre + "ln_2.weight"], a.ln2_mean, a.ln2_rstd, g[pre + "ln_2.weight"], g[pre + "ln_2.bias"], sc,
                                    mode=K.NORM_LAYER, dresid=dx, out=spare, dx_colsum=g[pre + "attn.c_proj.bias"])
                dx, spare = spare, dx  # dx now holds d(x1)
                # ---- attention branch: x1 = c_proj(att) + x ----
                with st("block_backward.attn_proj.dinput"):
                    gemm(dx, p[pre + "attn.c_proj.weight"], b_mn=True, out=self.d_att)
                with st("block_backward.attn_proj.dweight_bias"):
                    gemm(dx, a.att, a_mn=True, b_mn=True, workspace=self.ws, out=g[pre + "attn.c_proj.weight"])
                with st("block_backward.attn_sdpa"):
                    if cfg.differential:
                        K.diff_combine_backward(self.d_att, a.diff_a, p[pre + "attn.diff_lambda"], 1.0 - cfg.diff_lambda_init,
                                                a.diff_rstd, self.d_a2, self.diff_partial, g[pre + "attn.diff_lambda"], nh, hd)
                        K.diff_q_expand(a.qkv[:, :C], self.q2, nh, hd)      # recomputed: cheaper than keeping [N, 2C] per layer
                        K.attention_backward(self.d_a2, self.q2, a.qkv[:, C:2 * C], a.qkv[:, 2 * C:], a.diff_a, a.lse, B=B, T=T,
                                             n_q_heads=2 * nh, n_kv_heads=nh, head_dim=hd, causal=True, scale=(hd // 2) ** -0.5,
                                             dq=self.dq2, dk=self.d_qkv[:, C:2 * C], dv=self.d_qkv[:, 2 * C:], delta=self.delta)
                        K.diff_q_collapse(self.dq2, self.d_qkv[:, :C], nh, hd)
                    else:
                        K.attention_backward(self.d_att, a.qkv[:, :C], a.qkv[:, C:2 * C], a.qkv[:, 2 * C:], a.att,
                                             a.lse, B=B, T=T, n_q_heads=nh, n_kv_heads=nh, head_dim=hd, causal=True,
                                             dq=self.d_qkv[:, :C], dk=self.d_qkv[:, C:2 * C], dv=self.d_qkv[:, 2 * C:],
                                             delta=self.delta, dq_accum=self.dq_accum)
                if cfg.qk_norm:
                    with st("block_backward.qk_norm"):
                        K.qk_norm_backward(self.d_qkv, a.qkv, a.qk_rstd, nh, nh, hd)
                with st("block_backward.qkv.dinput"):
                    gemm(self.d_qkv, p[pre + "attn.c_attn.weight"], b_mn=True, out=self.d_ln)
                with st("block_backward.qkv.dweight_bias"):
                    gemm(self.d_qkv, a.ln1, a_mn=True, b_mn=True, workspace=self.ws, out=g[pre + "attn.c_attn.weight"])
                    K.colsum(self.d_qkv, g[pre + "attn.c_attn.bias"], sc)
                with st("block_backward.ln1_residual.fused_affine_dinput_add"):
                    K.norm_backward(self.d_ln, x_in, p[pre + "ln_1.weight"], a.ln1_mean, a.ln1_rstd, g[pre + "ln_1.weight"], g[pre + "ln_1.bias"], sc,
                                    mode=K.NORM_LAYER, dresid=dx, out=spare,
                                    dx_colsum=g[f"h.{l - 1}.mlp.c_proj.bias"] if l > 0 else None)
                dx, spare = spare, dx
            if self.grad_ready_hook is not None and l % self.grad_bucket_layers == 0:
                self.grad_ready_hook(*self._layer_range(l, min(l + self.grad_bucket_layers, cfg.n_layer) - 1))
        with st("embedding_backward"):
            st_, od_ = K.sort_tokens(self.tokens, self.tok_sorted, self.tok_order)
            K.embedding_backward(dx, self.tokens, g["wte"], g["wpe"][:T], B=B, T=T, sorted_tokens=st_, order=od_)
        if T < cfg.max_seq_len:
            g["wpe"][T:].zero_()

    @property
    def mlp_act(self) -> str:
        return "gelu_tanh" if self.activation == "gelu" else self.activation

    @property
    def graph_key(self) -> str:
        """Distinguishes captured step graphs whose kernels differ (the activation is baked into the launches)."""
        return self.activation

    def moa_probe_due(self, step: int) -> bool:
        """``step`` = 1-based number of the optimizer step about to run."""
        cfg = self.cfg
        return bool(cfg.moa_activations) and cfg.moa_interval > 0 and (step == 1 or step % cfg.moa_interval == 0)

    @torch.no_grad()
    def moa_select(self, step: int) -> str:
        """Forward-only loss of every candidate activation on the batch in the buffers; keeps the lowest.
        Mirrors ``maybe_probe_moa`` (``nfn_gpt2_native_train.cpp:28074-28108``)."""
        previous, losses = self.activation, {}
        for name in self.cfg.moa_activations:
            self.activation = name
            self.forward(compute_grad_logits=False)
            losses[name] = float(self.loss.item())
        finite = {k: v for k, v in losses.items() if math.isfinite(v)}
        self.activation = min(finite, key=finite.get) if finite else previous
        m = self.moa
        m["probe_runs"] += 1
        m["candidate_evals"] += len(losses)
        m["selected_activation_changes"] += int(self.activation != previous)
        m["last_probe_losses"] = losses
        m["history"].append({"step": step, "selected": self.activation})
        return self.activation

    def set_batch(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        """Copy a batch (any integer dtype, host or device) into the engine's int32 inputs."""
        self.tokens.copy_(tokens.reshape(-1), non_blocking=True)
        self.targets.copy_(targets.reshape(-1), non_blocking=True)

    def logits_view(self) -> torch.Tensor:
        return self.logits.view(self.B, self.T, -1)[..., :self.cfg.vocab_size]
