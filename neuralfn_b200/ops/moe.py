"""Mixture-of-experts feed-forward on the sm_100a kernels: router GEMM (fp32 logits) ->
top-k routing -> expert-sorted permutation -> grouped tcgen05 GEMM (gate|up) -> SwiGLU ->
grouped GEMM (down) -> weighted combine. No host synchronisation anywhere: the number of
live tiles is read by the grouped GEMM from device memory.

Weights: ``w_router`` [E, d], ``w_gate_up`` [E, 2F, d] (gate rows then up rows per expert),
``w_down`` [E, d, F], all bf16. Matches the math of the tensor-runtime stages
``router_topk`` + ``grouped_swiglu_experts`` (reference ``torch_backend.py`` MoE stages and
``kernels.cu:12612-12862``).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from . import _lib
from .gemm import gemm, gemm_grouped_k
from .infer import swiglu_forward

__all__ = ["MoEWorkspace", "moe_forward", "moe_reference", "moe_experts", "moe_experts_native_ok"]

GROUPED = 3


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _st():
    return c_void_p(_lib.stream_ptr())


class MoEWorkspace:
    """Buffers for up to ``max_tokens`` tokens (worst-case padded row capacity)."""

    def __init__(self, max_tokens: int, n_experts: int, top_k: int, d_model: int, d_ff: int, device) -> None:
        cap = (max_tokens * top_k + n_experts * 127 + 127) // 128 * 128
        self.capacity_rows, self.max_tiles = cap, cap // 128
        i32 = dict(dtype=torch.int32, device=device)
        self.logits = torch.empty(max_tokens, n_experts, dtype=torch.float32, device=device)
        self.topk_idx = torch.empty(max_tokens, top_k, **i32)
        self.topk_w = torch.empty(max_tokens, top_k, dtype=torch.float32, device=device)
        self.counts = torch.zeros(n_experts, **i32)
        self.offsets = torch.zeros(n_experts + 1, **i32)
        self.cursor = torch.zeros(n_experts, **i32)
        self.tile_expert = torch.zeros(self.max_tiles, **i32)
        self.plan = torch.zeros(2, **i32)
        self.row_of = torch.empty(max_tokens * top_k, **i32)
        bf = dict(dtype=torch.bfloat16, device=device)
        self.xs = torch.zeros(cap, d_model, **bf)
        self.h = torch.empty(cap, 2 * d_ff, **bf)
        self.a = torch.empty(cap, d_ff, **bf)
        self.ys = torch.empty(cap, d_model, **bf)


def _grouped_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ws: MoEWorkspace) -> None:
    from ..parallel.tp import GemmTpArgs
    E, N, K = w.shape
    args = GemmTpArgs()
    args.mode = GROUPED
    args.a, args.b, args.c = a.data_ptr(), w.data_ptr(), out.data_ptr()
    args.m, args.n, args.k = a.shape[0], N, K
    args.lda, args.ldb, args.ldc = a.stride(0), K, out.stride(0)
    args.tile_group, args.num_m_tiles_dev, args.groups = ws.tile_expert.data_ptr(), ws.plan.data_ptr(), E
    _lib.check(_lib.load().nfn_gemm_tp(ctypes.byref(args), _st()), "nfn_gemm_tp(grouped)")


def moe_forward(x: torch.Tensor, w_router: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, top_k: int, ws: MoEWorkspace, *,
                score_fn: str = "softmax", norm_topk: bool = True, route_scale: float = 1.0, resid: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """x bf16 [T, d] -> bf16 [T, d] (+ resid)."""
    T, d = x.shape
    E, F2, _ = w_gate_up.shape
    F = F2 // 2
    L = _lib.load()
    if E % 8:
        # the GEMM wants N in multiples of 8: pad the router with zero rows once (their logits are
        # never looked at - the routing kernel reads the first E columns only)
        key = (w_router.data_ptr(), w_router._version)
        if getattr(ws, "_router_key", None) != key:
            Ep = (E + 7) // 8 * 8
            ws._router_pad = torch.zeros(Ep, d, dtype=w_router.dtype, device=w_router.device)
            ws._router_pad[:E].copy_(w_router)
            ws._logits_pad = torch.empty(ws.logits.shape[0], Ep, dtype=torch.float32, device=w_router.device)
            ws._router_key = key
        gemm(x, ws._router_pad, out=ws._logits_pad[:T], out_dtype=torch.float32)
        logits = ws._logits_pad
    else:
        gemm(x, w_router, out=ws.logits[:T], out_dtype=torch.float32)
        logits = ws.logits
    ws.counts.zero_()
    _lib.check(L.nfn_moe_route(_p(logits), c_int(logits.stride(0)), c_int(T), c_int(E), c_int(top_k), c_int(1 if score_fn == "sigmoid" else 0),
                               c_int(int(norm_topk)), c_float(route_scale), _p(ws.topk_idx), _p(ws.topk_w), _p(ws.counts), _st()), "nfn_moe_route")
    _lib.check(L.nfn_moe_plan(_p(ws.counts), c_int(E), c_int(ws.max_tiles), _p(ws.offsets), _p(ws.cursor), _p(ws.tile_expert), _p(ws.plan), _st()),
               "nfn_moe_plan")
    _lib.check(L.nfn_moe_permute(_p(x), c_int(x.stride(0)), c_int(T), c_int(top_k), c_int(d), _p(ws.topk_idx), _p(ws.offsets), _p(ws.cursor),
                                 c_int(ws.capacity_rows), _p(ws.xs), _p(ws.row_of), _st()), "nfn_moe_permute")
    _grouped_gemm(ws.xs, w_gate_up, ws.h, ws)
    swiglu_forward(ws.h, F, out=ws.a)
    _grouped_gemm(ws.a, w_down, ws.ys, ws)
    out = torch.empty(T, d, dtype=torch.bfloat16, device=x.device) if out is None else out
    _lib.check(L.nfn_moe_combine(_p(ws.ys), c_int(d), c_int(T), c_int(top_k), _p(ws.row_of), _p(ws.topk_w), _p(resid),
                                 c_int(0 if resid is None else resid.stride(0)), _p(out), c_int(out.stride(0)), _st()), "nfn_moe_combine")
    return out


def moe_reference(x, w_router, w_gate_up, w_down, top_k: int, *, score_fn: str = "softmax", norm_topk: bool = True,
                  route_scale: float = 1.0, resid=None) -> torch.Tensor:
    """fp32 PyTorch oracle of ``moe_forward`` (dense loop over experts)."""
    xf = x.float()
    logits = xf @ w_router.float().T
    scores = torch.sigmoid(logits) if score_fn == "sigmoid" else torch.softmax(logits, -1)
    w, idx = scores.topk(top_k, dim=-1)
    if norm_topk:
        w = w / w.sum(-1, keepdim=True)
    w = w * route_scale
    F = w_gate_up.shape[1] // 2
    out = torch.zeros_like(xf)
    for e in range(w_gate_up.shape[0]):
        sel = (idx == e)
        rows = sel.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        h = xf[rows] @ w_gate_up[e].float().T
        a = torch.nn.functional.silu(h[:, :F]) * h[:, F:]
        y = a @ w_down[e].float().T
        out[rows] += y * (w[rows] * sel[rows]).sum(-1, keepdim=True)
    return out + (resid.float() if resid is not None else 0)


# --------------------------------------------------------------------------- training path --
class _MoEExpertsFn(torch.autograd.Function):
    """Dropless expert FFN with gradients. Inputs in the tensor-runtime layout: x [T, d] bf16,
    w1 / w3 [E, d, h] (gate / up), w2 [E, h, d], routing weights [T, k] (any float dtype) and
    indices [T, k] (int64). Forward: expert-sorted permutation -> grouped tcgen05 GEMM (gate|up)
    -> SwiGLU -> grouped GEMM (down) -> weighted combine. Backward: the same plan drives the
    grouped input-gradient GEMMs (the stored [E, K, N] weights are already the operand layout
    those need); weight gradients are one TN GEMM per expert over its row segment; routing
    weights get <expert output, upstream gradient>.

    Reference counterparts: ``moe_swiglu_forward/backward`` (``kernels.cu:12612-12862``), which
    loop per token over its k experts with dense weights and no permutation."""

    @staticmethod
    def forward(ctx, x, w1, w2, w3, weights, indices):
        T, d = x.shape
        E, _, h = w1.shape
        k = indices.shape[-1]
        L = _lib.load()
        ws = MoEWorkspace(T, E, k, d, h, x.device)
        ws.topk_idx.copy_(indices)
        ws.topk_w.copy_(weights)
        ws.counts.copy_(torch.bincount(indices.reshape(-1), minlength=E))
        w_gu = torch.cat([w1.transpose(1, 2), w3.transpose(1, 2)], 1).contiguous()  # [E, 2h, d]
        w_dn = w2.transpose(1, 2).contiguous()                                     # [E, d, h]
        _lib.check(L.nfn_moe_plan(_p(ws.counts), c_int(E), c_int(ws.max_tiles), _p(ws.offsets), _p(ws.cursor), _p(ws.tile_expert), _p(ws.plan), _st()),
                   "nfn_moe_plan")
        _lib.check(L.nfn_moe_permute(_p(x), c_int(x.stride(0)), c_int(T), c_int(k), c_int(d), _p(ws.topk_idx), _p(ws.offsets), _p(ws.cursor),
                                     c_int(ws.capacity_rows), _p(ws.xs), _p(ws.row_of), _st()), "nfn_moe_permute")
        _grouped_gemm(ws.xs, w_gu, ws.h, ws)
        swiglu_forward(ws.h, h, out=ws.a)
        _grouped_gemm(ws.a, w_dn, ws.ys, ws)
        out = torch.empty(T, d, dtype=torch.bfloat16, device=x.device)
        _lib.check(L.nfn_moe_combine(_p(ws.ys), c_int(d), c_int(T), c_int(k), _p(ws.row_of), _p(ws.topk_w), _p(None), c_int(0), _p(out),
                                     c_int(out.stride(0)), _st()), "nfn_moe_combine")
        ctx.ws, ctx.dims = ws, (T, d, E, h, k)
        ctx.save_for_backward(w1, w2, w3)
        ctx.w_dtype = weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        from .infer import swiglu_backward
        w1, w2, w3 = ctx.saved_tensors
        ws, (T, d, E, h, k) = ctx.ws, ctx.dims
        dout = dout.contiguous()
        rows = ws.row_of.long()                                         # [T * k] sorted row of every (token, slot)
        # routing-weight gradient and the upstream gradient of every sorted row
        ys_tk = ws.ys[rows].view(T, k, d)
        d_w = torch.einsum("tkd,td->tk", ys_tk.float(), dout.float())
        dys = torch.zeros_like(ws.ys)
        dys[rows] = (dout[:, None, :].float() * ws.topk_w[:, :, None]).to(torch.bfloat16).view(T * k, d)
        # input gradients through the two grouped GEMMs (weights as stored are the [E, N, K] operands)
        da = torch.empty_like(ws.a)
        _grouped_gemm(dys, w2.contiguous(), da, ws)                     # [cap, h] = dys @ w2[e]^T
        dh = swiglu_backward(ws.h, da, h)                               # [cap, 2h]
        dxs = torch.empty_like(ws.xs)
        _grouped_gemm(dh, torch.cat([w1, w3], 2).contiguous(), dxs, ws)  # [cap, d] = dh @ [w1 | w3][e]^T
        dx = dxs[rows].view(T, k, d).float().sum(1).to(torch.bfloat16)
        # weight gradients of all experts: three grouped contractions over the plan's padded row segments (pad rows of xs and
        # dys are zero, those of a and dh are finite), no host read of the counts
        dw1, dw2, dw3 = torch.empty_like(w1), torch.empty_like(w2), torch.empty_like(w3)
        gemm_grouped_k(ws.xs, dh[:, :h], ws.offsets, dw1)               # [E, d, h] = xs^T dh_gate
        gemm_grouped_k(ws.xs, dh[:, h:], ws.offsets, dw3)
        gemm_grouped_k(ws.a, dys, ws.offsets, dw2)                      # [E, h, d] = a^T dys
        ctx.ws = None
        return dx, dw1, dw2, dw3, d_w.to(ctx.w_dtype), None


def moe_experts_native_ok(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor, indices: torch.Tensor) -> bool:
    E, d, h = w1.shape
    return (x.is_cuda and x.dtype == torch.bfloat16 and w1.dtype == w2.dtype == w3.dtype == torch.bfloat16 and _lib.available()
            and d % 64 == 0 and h % 64 == 0 and E <= 256 and indices.shape[-1] <= 8 and x.shape[0] > 0)


def moe_experts(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Differentiable expert FFN on the native kernels (see ``_MoEExpertsFn``)."""
    return _MoEExpertsFn.apply(x.contiguous(), w1, w2, w3, weights, indices)
