"""Tensor stages, part 2: linear layers (plain, ternary, FP8, MX, LoRA, NF4, RandMap),
activations and gated MLPs. Reference semantics: ``neuralfn/torch_backend.py:597-1097,
2418-2470,1665-1727``."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .stages_core import stage


@stage("linear")
class LinearStage(nn.Module):
    def __init__(self, input_dim: int, output_dim: int, bias: bool = False) -> None:
        super().__init__()
        self.proj = nn.Linear(input_dim, output_dim, bias=bias)
        nn.init.normal_(self.proj.weight, std=0.02)
        if bias:
            nn.init.zeros_(self.proj.bias)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["input_dim"]), int(cfg["output_dim"]), bool(cfg.get("bias", False)))

    def forward(self, x: Tensor) -> Tensor:
        from .kernel_bridge import linear
        return linear(x, self.proj.weight, self.proj.bias)


@stage("bitlinear_ternary")
class BitLinearTernaryStage(nn.Module):
    """BitNet b1.58: weights quantised to {-1, 0, +1} * mean|w| with a straight-through estimator,
    activations to int8 per token."""

    def __init__(self, input_dim: int, output_dim: int) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(output_dim, input_dim))
        nn.init.normal_(self.weight, std=0.02)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["input_dim"]), int(cfg["output_dim"]))

    def forward(self, x: Tensor) -> Tensor:
        w = self.weight
        scale = w.abs().mean().clamp(min=1e-5)
        wq = (w / scale).round().clamp(-1, 1) * scale
        wq = w + (wq - w).detach()
        ax = x.abs().amax(dim=-1, keepdim=True).clamp(min=1e-5)
        xq = (x * 127.0 / ax).round().clamp(-128, 127) * ax / 127.0
        xq = x + (xq - x).detach()
        return F.linear(xq, wq.to(x.dtype))


def _fake_quant_fp8(t: Tensor, fmt: str, amax: Tensor) -> Tensor:
    dtype = torch.float8_e5m2 if fmt == "e5m2" else torch.float8_e4m3fn
    fmax = 57344.0 if fmt == "e5m2" else 448.0
    scale = fmax / amax.clamp(min=1e-12)
    q = (t.float() * scale).clamp(-fmax, fmax).to(dtype).float() / scale
    return t + (q.to(t.dtype) - t).detach()


@stage("fp8_linear")
class FP8LinearStage(nn.Module):
    """Linear with FP8 (E4M3/E5M2) fake-quantised weights and activations, delayed scaling from an
    amax history; gradients pass straight through."""

    def __init__(self, input_dim: int, output_dim: int, bias: bool = False, fp8_format: str = "e4m3",
                 amax_history_len: int = 16, use_stochastic_rounding: bool = True) -> None:
        super().__init__()
        self.proj = nn.Linear(input_dim, output_dim, bias=bias)
        nn.init.normal_(self.proj.weight, std=0.02)
        self.fp8_format = fp8_format
        self.use_stochastic_rounding = use_stochastic_rounding
        self.register_buffer("amax_x", torch.zeros(amax_history_len))
        self.register_buffer("amax_w", torch.zeros(amax_history_len))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["input_dim"]), int(cfg["output_dim"]), bool(cfg.get("bias", False)),
                   str(cfg.get("fp8_format", "e4m3")), int(cfg.get("amax_history_len", 16)),
                   bool(cfg.get("use_stochastic_rounding", True)))

    def _amax(self, hist: Tensor, t: Tensor) -> Tensor:
        cur = t.detach().abs().amax().float()
        if self.training:
            hist.copy_(torch.roll(hist, 1))
            hist[0] = cur
        return torch.maximum(hist.amax(), cur)

    def forward(self, x: Tensor) -> Tensor:
        xq = _fake_quant_fp8(x, self.fp8_format, self._amax(self.amax_x, x))
        wq = _fake_quant_fp8(self.proj.weight, self.fp8_format, self._amax(self.amax_w, self.proj.weight))
        return F.linear(xq, wq.to(x.dtype), None if self.proj.bias is None else self.proj.bias.to(x.dtype))


_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def _fake_quant_mx(t: Tensor, fmt: str, block: int) -> Tensor:
    """Micro-scaling: blocks of ``block`` values share a power-of-two scale; elements are
    E2M1 (mxfp4) or E4M3 (mxfp8)."""
    shape = t.shape
    pad = (-shape[-1]) % block
    f = F.pad(t.float(), (0, pad)).reshape(*shape[:-1], -1, block)
    amax = f.abs().amax(-1, keepdim=True).clamp(min=1e-30)
    emax = 2.0 if fmt == "mxfp4" else 8.0
    scale = torch.exp2(torch.floor(torch.log2(amax)) - emax)
    y = f / scale
    if fmt == "mxfp4":
        grid = _E2M1.to(y.device)
        idx = (y.abs().unsqueeze(-1) - grid).abs().argmin(-1)
        q = grid[idx] * y.sign()
    else:
        q = y.clamp(-448, 448).to(torch.float8_e4m3fn).float()
    out = (q * scale).reshape(*shape[:-1], -1)[..., :shape[-1]].to(t.dtype)
    return t + (out - t).detach()


@stage("mx_linear")
class MXLinearStage(nn.Module):
    def __init__(self, input_dim: int, output_dim: int, bias: bool = False, mx_format: str = "mxfp4",
                 mx_block_size: int = 32) -> None:
        super().__init__()
        self.proj = nn.Linear(input_dim, output_dim, bias=bias)
        nn.init.normal_(self.proj.weight, std=0.02)
        self.mx_format, self.mx_block_size = mx_format, int(mx_block_size)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["input_dim"]), int(cfg["output_dim"]), bool(cfg.get("bias", False)),
                   str(cfg.get("mx_format", "mxfp4")), int(cfg.get("mx_block_size", 32)))

    def forward(self, x: Tensor) -> Tensor:
        wq = _fake_quant_mx(self.proj.weight, self.mx_format, self.mx_block_size)
        xq = _fake_quant_mx(x, self.mx_format, self.mx_block_size)
        return F.linear(xq, wq.to(x.dtype), None if self.proj.bias is None else self.proj.bias.to(x.dtype))


@stage("lora_linear")
class LoRALinearStage(nn.Module):
    """y = base(x) + (alpha / r) * B(A(dropout(x))); A kaiming-uniform, B zero, base frozen by the
    fine-tune pre-hook."""

    def __init__(self, input_dim: int, output_dim: int, rank: int = 8, alpha: float = 16.0,
                 dropout: float = 0.0, bias: bool = False, merge_on_eval: bool = False) -> None:
        super().__init__()
        self.base = nn.Linear(input_dim, output_dim, bias=bias)
        nn.init.normal_(self.base.weight, std=0.02)
        self.lora_A = nn.Parameter(torch.empty(rank, input_dim))
        self.lora_B = nn.Parameter(torch.zeros(output_dim, rank))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.scaling = float(alpha) / float(rank)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        self.merge_on_eval = merge_on_eval
        self.rank = rank

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["input_dim"]), int(cfg["output_dim"]), int(cfg.get("rank", 8)),
                   float(cfg.get("alpha", 16.0)), float(cfg.get("dropout", 0.0)), bool(cfg.get("bias", False)),
                   bool(cfg.get("merge_on_eval", False)))

    def merged_weight(self) -> Tensor:
        return self.base.weight + self.scaling * (self.lora_B @ self.lora_A)

    def forward(self, x: Tensor) -> Tensor:
        if not self.training and self.merge_on_eval:
            return F.linear(x, self.merged_weight().to(x.dtype),
                            None if self.base.bias is None else self.base.bias.to(x.dtype))
        y = self.base(x)
        upd = F.linear(F.linear(self.dropout(x), self.lora_A.to(x.dtype)), self.lora_B.to(x.dtype))
        return y + self.scaling * upd


NF4_CODEBOOK = torch.tensor([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
    0.7229568362236023, 1.0])


def nf4_quantize(weight: Tensor, group_size: int = 64) -> tuple[Tensor, Tensor]:
    """Per-row groups of ``group_size`` values -> (packed uint8 codes [out, in/2], fp32 absmax
    [out, in/group]). Low nibble = even column."""
    out_dim, in_dim = weight.shape
    if in_dim % group_size or in_dim % 2:
        raise ValueError("NF4 needs input_dim divisible by the group size and by 2")
    w = weight.float().reshape(out_dim, in_dim // group_size, group_size)
    absmax = w.abs().amax(-1).clamp(min=1e-12)
    normed = w / absmax.unsqueeze(-1)
    codes = (normed.unsqueeze(-1) - NF4_CODEBOOK.to(w.device)).abs().argmin(-1).to(torch.uint8)
    codes = codes.reshape(out_dim, in_dim)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return packed.contiguous(), absmax.contiguous()


def nf4_dequantize(packed: Tensor, absmax: Tensor, group_size: int = 64) -> Tensor:
    out_dim = packed.shape[0]
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(out_dim, -1).long()
    vals = NF4_CODEBOOK.to(packed.device)[codes]
    return (vals.reshape(out_dim, -1, group_size) * absmax.unsqueeze(-1)).reshape(out_dim, -1)


@stage("nf4_linear")
class NF4LinearStage(nn.Module):
    """QLoRA linear: frozen NF4 base (group-64 absmax) + trainable rank-r LoRA."""

    def __init__(self, input_dim: int, output_dim: int, rank: int = 8, alpha: float = 16.0,
                 dropout: float = 0.0, bias: bool = False, group_size: int = 64,
                 compute_dtype: str = "bf16") -> None:
        super().__init__()
        self.input_dim, self.output_dim, self.group_size = input_dim, output_dim, group_size
        w = torch.empty(output_dim, input_dim)
        nn.init.normal_(w, std=0.02)
        packed, absmax = nf4_quantize(w, group_size)
        self.register_buffer("packed_weight", packed)
        self.register_buffer("absmax", absmax)
        self.bias = nn.Parameter(torch.zeros(output_dim)) if bias else None
        self.lora_A = nn.Parameter(torch.empty(rank, input_dim))
        self.lora_B = nn.Parameter(torch.zeros(output_dim, rank))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.scaling = float(alpha) / float(rank)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        self.compute_dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}.get(
            compute_dtype, torch.bfloat16)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["input_dim"]), int(cfg["output_dim"]), int(cfg.get("rank", 8)),
                   float(cfg.get("alpha", 16.0)), float(cfg.get("dropout", 0.0)), bool(cfg.get("bias", False)),
                   int(cfg.get("group_size", 64)), str(cfg.get("compute_dtype", "bf16")))

    def load_base_weight(self, weight: Tensor) -> None:
        packed, absmax = nf4_quantize(weight.detach().to(self.packed_weight.device), self.group_size)
        self.packed_weight.copy_(packed)
        self.absmax.copy_(absmax)

    def dequantized_weight(self) -> Tensor:
        return nf4_dequantize(self.packed_weight, self.absmax, self.group_size)

    def forward(self, x: Tensor) -> Tensor:
        from .kernel_bridge import nf4_lora_linear
        return nf4_lora_linear(x, self.packed_weight, self.absmax, self.group_size, self.lora_A, self.lora_B,
                               self.scaling, self.bias, self.dropout)


@stage("randmap_adapter")
class RandMapAdapterStage(nn.Module):
    """Frozen random down-projection, trainable up-projection (zero init), added to the input."""

    def __init__(self, model_dim: int, adapter_dim: int) -> None:
        super().__init__()
        self.register_buffer("down", torch.randn(adapter_dim, model_dim) / math.sqrt(model_dim))
        self.up = nn.Parameter(torch.zeros(model_dim, adapter_dim))

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["adapter_dim"]))

    def forward(self, x: Tensor) -> Tensor:
        return x + F.linear(F.gelu(F.linear(x, self.down.to(x.dtype))), self.up.to(x.dtype))


# ------------------------------------------------------------------ activations / MLPs --
def _fn_stage(name: str, fn):
    cls = type(name, (nn.Module,), {"forward": lambda self, *a: fn(*a),
                                    "from_config": classmethod(lambda c, cfg: c())})
    return cls


GeluStage = stage("gelu")(_fn_stage("GeluStage", lambda x: F.gelu(x)))
SigmoidFunctionStage = stage("sigmoid")(_fn_stage("SigmoidFunctionStage", torch.sigmoid))
SiluFunctionStage = stage("silu")(_fn_stage("SiluFunctionStage", F.silu))
MultiplyFunctionStage = stage("multiply")(_fn_stage("MultiplyFunctionStage", lambda a, b: a * b))


@stage("dropout")
class DropoutStage(nn.Module):
    def __init__(self, p: float = 0.1) -> None:
        super().__init__()
        self.drop = nn.Dropout(p)

    @classmethod
    def from_config(cls, cfg):
        return cls(float(cfg.get("p", 0.1)))

    def forward(self, x: Tensor) -> Tensor:
        return self.drop(x)


def swiglu_hidden(model_dim: int, mlp_mult: float, multiple_of: int | None) -> int:
    hidden = int(model_dim * mlp_mult)
    if multiple_of:
        hidden = (hidden + multiple_of - 1) // multiple_of * multiple_of
    return hidden


@stage("swiglu")
class SwiGLUStage(nn.Module):
    """down(silu(gate(x)) * up(x)); hidden = int(d * mult) rounded up to ``multiple_of``."""

    def __init__(self, model_dim: int, mlp_mult: float, multiple_of: int | None = None,
                 hidden_dim: int | None = None) -> None:
        super().__init__()
        hidden = hidden_dim or swiglu_hidden(model_dim, mlp_mult, multiple_of)
        self.gate = nn.Linear(model_dim, hidden, bias=False)
        self.up = nn.Linear(model_dim, hidden, bias=False)
        self.down = nn.Linear(hidden, model_dim, bias=False)
        for lin in (self.gate, self.up, self.down):
            nn.init.normal_(lin.weight, std=0.02)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), float(cfg["mlp_mult"]), cfg.get("multiple_of"), cfg.get("hidden_dim"))

    def forward(self, x: Tensor) -> Tensor:
        from .kernel_bridge import swiglu_mlp
        return swiglu_mlp(x, self.gate.weight, self.up.weight, self.down.weight)


@stage("geglu", "reglu", "solu")
class GLUStage(nn.Module):
    """Gated linear unit family; hidden width is always 8d/3 (rounded), independent of ``mlp_mult``."""

    def __init__(self, model_dim: int, mlp_mult: int = 4, multiple_of: int | None = None,
                 activation: str = "gelu") -> None:
        super().__init__()
        hidden = int(8 * model_dim / 3)
        if multiple_of:
            hidden = (hidden + multiple_of - 1) // multiple_of * multiple_of
        self.gate = nn.Linear(model_dim, hidden, bias=False)
        self.up = nn.Linear(model_dim, hidden, bias=False)
        self.down = nn.Linear(hidden, model_dim, bias=False)
        for lin in (self.gate, self.up, self.down):
            nn.init.normal_(lin.weight, std=0.02)
        self.activation = activation

    @classmethod
    def from_config(cls, cfg):
        act = cfg.get("activation") or {"geglu": "gelu", "reglu": "relu", "solu": "softmax"}.get(
            str(cfg.get("__module_type__", "geglu")), "gelu")
        return cls(int(cfg["model_dim"]), int(cfg.get("mlp_mult", 4)), cfg.get("multiple_of"), act)

    def forward(self, x: Tensor) -> Tensor:
        g = self.gate(x)
        if self.activation == "gelu":
            g = F.gelu(g)
        elif self.activation == "relu":
            g = F.relu(g)
        else:  # SoLU: x * softmax(x)
            g = g * torch.softmax(g.float(), dim=-1).to(g.dtype)
        return self.down(g * self.up(x))


@stage("mlp_relu2")
class MLPReluSquaredStage(nn.Module):
    def __init__(self, model_dim: int, mlp_mult: int) -> None:
        super().__init__()
        self.fc = nn.Linear(model_dim, mlp_mult * model_dim, bias=False)
        self.proj = nn.Linear(mlp_mult * model_dim, model_dim, bias=False)
        nn.init.normal_(self.fc.weight, std=0.02)
        nn.init.zeros_(self.proj.weight)

    @classmethod
    def from_config(cls, cfg):
        return cls(int(cfg["model_dim"]), int(cfg["mlp_mult"]))

    def forward(self, x: Tensor) -> Tensor:
        return self.proj(F.relu(self.fc(x)).square())
