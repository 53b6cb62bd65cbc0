"""Bridge between graph stages and the sm_100a kernel library.

Each function takes ordinary tensors and dispatches: CUDA + bf16 + supported shape ->
``torch.autograd.Function`` around the C-ABI kernels (forward and backward both native);
anything else -> the plain PyTorch formulation, which is also what the kernel tests use
as their fp32 oracle. ``NFN_B200_FORCE_TORCH=1`` disables the native path.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F
from torch import Tensor

_FORCE_TORCH = os.environ.get("NFN_B200_FORCE_TORCH", "") == "1"


def _native_ok(*tensors: Tensor) -> bool:
    if _FORCE_TORCH:
        return False
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.bfloat16:
            return False
    from ..ops import _lib
    return _lib.available()


def _autocast_bf16(*tensors):
    """Under CUDA bf16 autocast, cast floating CUDA tensors to bf16 (differentiably) so the
    native path applies to fp32-parameter modules, as torch's own autocast would do for matmuls."""
    if not (torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16):
        return tensors
    return tuple(t.to(torch.bfloat16) if (t is not None and t.is_cuda and t.is_floating_point()) else t
                 for t in tensors)


def _K():
    from ..ops import kernels
    return kernels


def _gemm():
    from ..ops.gemm import gemm
    return gemm


# ---------------------------------------------------------------------------- linear --
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, weight, bias):
        ctx.save_for_backward(x2d, weight)
        ctx.has_bias = bias is not None
        return _gemm()(x2d, weight, bias=bias)

    @staticmethod
    def backward(ctx, dy):
        x2d, weight = ctx.saved_tensors
        dy = dy.contiguous()
        gemm = _gemm()
        dx = gemm(dy, weight, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = gemm(dy, x2d, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    x, weight, bias = _autocast_bf16(x, weight, bias)
    if (_native_ok(x, weight, bias) and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0
            and weight.is_contiguous()):
        x2d = x.reshape(-1, x.shape[-1])
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        return _LinearFn.apply(x2d, weight, bias).reshape(*x.shape[:-1], weight.shape[0])
    return F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))


# ----------------------------------------------------------------------------- norms --
class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, weight, bias, eps, mode, centered):
        K = _K()
        y, mean, rstd = K.norm_forward(x2d, weight, bias, eps=eps, mode=mode, centered=centered)
        ctx.save_for_backward(x2d, weight, mean if mean is not None else rstd, rstd)
        ctx.mode, ctx.centered, ctx.has_w, ctx.has_b = mode, centered, weight is not None, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        K = _K()
        x2d, weight, mean, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        dx = K.norm_backward_dx(dy, x2d, weight if ctx.has_w else None, mean, rstd, mode=ctx.mode,
                                centered=ctx.centered)
        dw = db = None
        if ctx.has_w or ctx.has_b:
            C = x2d.shape[1]
            scratch = torch.empty(64 * 2 * C, device=x2d.device, dtype=torch.float32)
            dw = torch.empty(C, device=x2d.device, dtype=torch.bfloat16) if ctx.has_w else None
            db = torch.empty(C, device=x2d.device, dtype=torch.bfloat16) if ctx.has_b else None
            K.norm_backward_wb(dy, x2d, mean, rstd, dw, db, scratch, mode=ctx.mode)
        return dx, dw, db, None, None, None


def _norm_native(x, weight, bias, eps, mode, centered):
    C = x.shape[-1]
    x2d = x.reshape(-1, C)
    if not x2d.is_contiguous():
        x2d = x2d.contiguous()
    return _NormFn.apply(x2d, weight, bias, float(eps), mode, bool(centered)).reshape(x.shape)


def rms_norm(x: Tensor, weight: Tensor | None, eps: float, centered: bool = False,
             force_float32: bool = False) -> Tensor:
    if x.dtype == torch.bfloat16 and weight is not None and weight.dtype != x.dtype:
        weight = weight.to(x.dtype)
    if _native_ok(x, weight) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _norm_native(x, weight, None, eps, 1, centered)
    src = x.float() if force_float32 or x.dtype != torch.float32 else x
    y = src * torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.to(y.dtype)
        y = y * (1.0 + w if centered else w)
    return y.to(x.dtype)


def layer_norm(x: Tensor, weight: Tensor, bias: Tensor | None, eps: float) -> Tensor:
    if x.dtype == torch.bfloat16 and weight.dtype != x.dtype:
        weight = weight.to(x.dtype)
        bias = None if bias is None else bias.to(x.dtype)
    if _native_ok(x, weight, bias) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _norm_native(x, weight, bias, eps, 0, False)
    return F.layer_norm(x, (x.shape[-1],), weight.to(x.dtype), None if bias is None else bias.to(x.dtype), eps)


# ------------------------------------------------------------------------- attention --
class _AttentionFn(torch.autograd.Function):
    """q [B, Hq, T, D], k/v [B, Hkv, T, D] (bf16) -> [B, Hq, T, D]."""

    @staticmethod
    def forward(ctx, q, k, v, causal, window, scale, softcap=0.0, seq_ids=None):
        K = _K()
        B, Hq, T, D = q.shape
        Hkv = k.shape[1]
        # token-major packed views [B*T, H*D]
        qp = q.transpose(1, 2).reshape(B * T, Hq * D).contiguous()
        kp = k.transpose(1, 2).reshape(B * T, Hkv * D).contiguous()
        vp = v.transpose(1, 2).reshape(B * T, Hkv * D).contiguous()
        o, lse = K.attention_forward(qp, kp, vp, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D,
                                     causal=causal, window=window, scale=scale, softcap=softcap, seq_ids=seq_ids)
        ctx.save_for_backward(qp, kp, vp, o, lse)
        ctx.meta = (B, T, Hq, Hkv, D, causal, window, scale, softcap)
        ctx.seq_ids = seq_ids
        return o.view(B, T, Hq, D).transpose(1, 2)

    @staticmethod
    def backward(ctx, do):
        K = _K()
        qp, kp, vp, o, lse = ctx.saved_tensors
        B, T, Hq, Hkv, D, causal, window, scale, softcap = ctx.meta
        dop = do.transpose(1, 2).reshape(B * T, Hq * D).contiguous()
        dq, dk, dv = torch.empty_like(qp), torch.empty_like(kp), torch.empty_like(vp)
        K.attention_backward(dop, qp, kp, vp, o, lse, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D,
                             causal=causal, window=window, scale=scale, softcap=softcap, seq_ids=ctx.seq_ids,
                             dq=dq, dk=dk, dv=dv)
        return (dq.view(B, T, Hq, D).transpose(1, 2), dk.view(B, T, Hkv, D).transpose(1, 2),
                dv.view(B, T, Hkv, D).transpose(1, 2), None, None, None, None, None)


def segment_attention(q: Tensor, k: Tensor, v: Tensor, seq_ids: Tensor, *, causal: bool = False,
                      scale: float | None = None) -> Tensor:
    """Attention over packed sequences: q/k/v [B, H, T, D], ``seq_ids`` int [B, T]; a key is visible
    only to queries of its own segment. On the native path one kernel launch covers all segments
    (the flash kernels mask by sequence id and skip key blocks outside the visible range of a
    causal tile); head dims other than 64 / 128 are zero-padded up, which leaves scores and
    outputs unchanged. Elsewhere: scaled-dot-product attention under a block-diagonal mask."""
    q, k, v = _autocast_bf16(q, k, v)
    D = q.shape[-1]
    sc = float(scale if scale is not None else D ** -0.5)
    if _native_ok(q, k, v) and D <= 128 and q.shape[1] % k.shape[1] == 0 and q.shape[-2] == k.shape[-2]:
        Dp = 64 if D <= 64 else 128
        if Dp != D:
            q, k, v = (F.pad(t, (0, Dp - D)) for t in (q, k, v))
        ids = seq_ids.reshape(-1).to(torch.int32).contiguous()
        out = _AttentionFn.apply(q, k, v, bool(causal), 0, sc, 0.0, ids)
        return out[..., :D] if Dp != D else out
    same = seq_ids.unsqueeze(-1) == seq_ids.unsqueeze(-2)                      # [B, T, T]
    if causal:
        same = same & torch.ones(same.shape[-2:], dtype=torch.bool, device=same.device).tril()
    return F.scaled_dot_product_attention(q, k, v, attn_mask=same.unsqueeze(1), scale=sc,
                                          enable_gqa=q.size(1) != k.size(1))


def attention(q: Tensor, k: Tensor, v: Tensor, *, causal: bool = True, window: int = 0, dropout_p: float = 0.0,
              scale: float | None = None, math_path: bool = False) -> Tensor:
    q, k, v = _autocast_bf16(q, k, v)
    D = q.shape[-1]
    same_len = q.shape[-2] == k.shape[-2]
    if (_native_ok(q, k, v) and D in (64, 128) and dropout_p == 0.0 and same_len and not math_path
            and q.shape[1] % k.shape[1] == 0):
        return _AttentionFn.apply(q, k, v, bool(causal), int(window), float(scale or D ** -0.5), 0.0, None)
    if window and window > 0:
        from .stages_attention import sparse_attention_mask
        mask = sparse_attention_mask(q.size(-2), k.size(-2), is_causal=causal, window=window, num_sinks=0,
                                     block=None, compress_stride=None, device=q.device, dtype=q.dtype)
        return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=dropout_p, scale=scale,
                                              enable_gqa=q.size(1) != k.size(1))
    return F.scaled_dot_product_attention(q, k, v, dropout_p=dropout_p, is_causal=causal and same_len, scale=scale,
                                          enable_gqa=q.size(1) != k.size(1))


class _PackedAttentionFn(torch.autograd.Function):
    """Causal attention straight on packed rows [B * T, (Hq + 2 Hkv) * D] -> [B * T, Hq * D]:
    the kernels take q, k and v as strided views, and the backward pass writes dq, dk and dv
    into the three column ranges of one gradient buffer - no re-packing copies either way."""

    @staticmethod
    def forward(ctx, qkv, B, T, Hq, Hkv, D, causal, window, scale):
        K = _K()
        q, k, v = qkv[:, :Hq * D], qkv[:, Hq * D:(Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:(Hq + 2 * Hkv) * D]
        o, lse = K.attention_forward(q, k, v, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, causal=causal, window=window, scale=scale)
        ctx.save_for_backward(qkv, o, lse)
        ctx.meta = (B, T, Hq, Hkv, D, causal, window, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        K = _K()
        qkv, o, lse = ctx.saved_tensors
        B, T, Hq, Hkv, D, causal, window, scale = ctx.meta
        q, k, v = qkv[:, :Hq * D], qkv[:, Hq * D:(Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:(Hq + 2 * Hkv) * D]
        dqkv = torch.empty_like(qkv) if qkv.shape[1] == (Hq + 2 * Hkv) * D else torch.zeros_like(qkv)
        K.attention_backward(do.contiguous(), q, k, v, o, lse, B=B, T=T, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, causal=causal, window=window,
                             scale=scale, dq=dqkv[:, :Hq * D], dk=dqkv[:, Hq * D:(Hq + Hkv) * D], dv=dqkv[:, (Hq + Hkv) * D:(Hq + 2 * Hkv) * D])
        return dqkv, None, None, None, None, None, None, None, None


def attention_packed_qkv(qkv: Tensor, *, B: int, T: int, n_q_heads: int, n_kv_heads: int, head_dim: int, causal: bool = True,
                         window: int = 0, scale: float | None = None) -> Tensor:
    """Self-attention over packed QKV rows (row = b * T + t); returns token-major [B * T, Hq * D]."""
    Hq, Hkv, D = n_q_heads, n_kv_heads, head_dim
    if _native_ok(qkv) and qkv.dim() == 2 and qkv.stride(1) == 1 and D in (64, 128) and Hq % Hkv == 0:
        return _PackedAttentionFn.apply(qkv, B, T, Hq, Hkv, D, bool(causal), int(window), float(scale or D ** -0.5))
    q = qkv[:, :Hq * D].view(B, T, Hq, D).transpose(1, 2)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D).transpose(1, 2)
    v = qkv[:, (Hq + Hkv) * D:(Hq + 2 * Hkv) * D].view(B, T, Hkv, D).transpose(1, 2)
    return attention(q, k, v, causal=causal, window=window, scale=scale).transpose(1, 2).reshape(B * T, Hq * D)


# ------------------------------------------------------------------------------ loss --
class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits2d, targets, z_coef):
        K = _K()
        rows, V = logits2d.shape
        work = logits2d.clone()  # the kernel overwrites logits with gradients
        mean_loss, _ = K.cross_entropy(work, targets, vocab=V, cap=0.0, z_coef=z_coef, grad_scale=1.0 / rows,
                                       loss_scale=1.0 / rows)
        ctx.save_for_backward(work)
        return mean_loss.reshape(())

    @staticmethod
    def backward(ctx, dloss):
        (grad,) = ctx.saved_tensors
        return grad * dloss.to(grad.dtype), None, None


def token_cross_entropy(logits: Tensor, target_ids: Tensor, z_loss_coef: float = 0.0) -> Tensor:
    V = logits.size(-1)
    if _native_ok(logits) and V % 8 == 0 and logits.is_contiguous():
        return _CrossEntropyFn.apply(logits.reshape(-1, V), target_ids.reshape(-1).to(torch.int32).contiguous(),
                                     float(z_loss_coef))
    fl = logits.reshape(-1, V).float()
    ft = target_ids.reshape(-1).long()
    if z_loss_coef <= 0.0:
        return F.cross_entropy(fl, ft, reduction="mean")
    lse = torch.logsumexp(fl, dim=-1)
    tv = fl.gather(1, ft.unsqueeze(1)).squeeze(1)
    return (lse - tv).mean() + z_loss_coef * lse.pow(2).mean()


# ------------------------------------------------------------------------------ MLPs --
class _SwiGLUFn(torch.autograd.Function):
    """gate_up [rows, 2 F] (gate | up) -> silu(gate) * up [rows, F]."""

    @staticmethod
    def forward(ctx, gate_up, inter):
        from ..ops.infer import swiglu_forward
        ctx.save_for_backward(gate_up)
        ctx.inter = inter
        return swiglu_forward(gate_up, inter)

    @staticmethod
    def backward(ctx, dout):
        from ..ops.infer import swiglu_backward
        (gate_up,) = ctx.saved_tensors
        return swiglu_backward(gate_up, dout.contiguous(), ctx.inter), None


def swiglu(gate_up: Tensor, inter: int) -> Tensor:
    """SwiGLU over packed (gate | up) rows; native kernels for contiguous bf16 CUDA rows."""
    if _native_ok(gate_up) and gate_up.dim() == 2 and gate_up.is_contiguous() and inter % 8 == 0:
        return _SwiGLUFn.apply(gate_up, int(inter))
    return F.silu(gate_up[..., :inter]) * gate_up[..., inter:]


class _RopeFn(torch.autograd.Function):
    """Rotates the q and k heads of packed [B * T, (Hq + 2 Hkv) * D] rows in place (v untouched);
    the gradient is the inverse rotation."""

    @staticmethod
    def forward(ctx, qkv, T, n_q, n_kv, head_dim, cos, sin, convention):
        from ..ops.infer import rope_inplace
        rope_inplace(qkv, T=T, n_q_heads=n_q, n_kv_heads=n_kv, head_dim=head_dim, cos=cos, sin=sin, convention=convention)
        ctx.mark_dirty(qkv)
        ctx.meta = (T, n_q, n_kv, head_dim, convention)
        ctx.save_for_backward(cos, sin)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        from ..ops.infer import rope_inplace
        cos, sin = ctx.saved_tensors
        T, n_q, n_kv, head_dim, convention = ctx.meta
        d = dqkv.contiguous().clone()
        rope_inplace(d, T=T, n_q_heads=n_q, n_kv_heads=n_kv, head_dim=head_dim, cos=cos, sin=sin, convention=convention, backward=True)
        return d, None, None, None, None, None, None, None


def rope_packed_qkv(qkv: Tensor, *, T: int, n_q_heads: int, n_kv_heads: int, head_dim: int, cos: Tensor, sin: Tensor, convention: str = "hf") -> Tensor:
    """Rotary embedding on packed QKV rows (row r is position r % T). ``cos`` / ``sin``: fp32
    [>= T, head_dim / 2]. Native in-place kernel on bf16 CUDA rows, PyTorch otherwise."""
    if _native_ok(qkv) and qkv.dim() == 2 and qkv.is_contiguous() and cos.dtype == torch.float32:
        return _RopeFn.apply(qkv, T, n_q_heads, n_kv_heads, head_dim, cos, sin, convention)
    rows, hd, half = qkv.shape[0], head_dim, head_dim // 2
    sign = 1.0 if convention == "hf" else -1.0
    qk = qkv[:, :(n_q_heads + n_kv_heads) * hd].reshape(rows // T, T, n_q_heads + n_kv_heads, hd)
    c, s_ = cos[:T].to(qkv.dtype)[None, :, None], sin[:T].to(qkv.dtype)[None, :, None]
    a, b = qk[..., :half], qk[..., half:]
    rot = torch.cat((a * c - sign * b * s_, b * c + sign * a * s_), -1).reshape(rows, -1)
    return torch.cat((rot, qkv[:, (n_q_heads + n_kv_heads) * hd:]), -1)


def swiglu_mlp(x: Tensor, w_gate: Tensor, w_up: Tensor, w_down: Tensor) -> Tensor:
    g = linear(x, w_gate)
    u = linear(x, w_up)
    return linear(F.silu(g) * u, w_down)


def nf4_lora_linear(x: Tensor, packed: Tensor, absmax: Tensor, group_size: int, lora_a: Tensor, lora_b: Tensor,
                    scaling: float, bias: Tensor | None, dropout) -> Tensor:
    from .stages_linear import nf4_dequantize
    w = nf4_dequantize(packed, absmax, group_size).to(x.dtype)
    y = F.linear(x, w, None if bias is None else bias.to(x.dtype))
    upd = F.linear(F.linear(dropout(x), lora_a.to(x.dtype)), lora_b.to(x.dtype))
    return y + scaling * upd
