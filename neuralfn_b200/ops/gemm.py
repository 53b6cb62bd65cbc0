"""BF16 GEMM family on tcgen05/TMEM with fused epilogues (Python front-end).

``gemm(a, b)`` computes ``opA @ opB^T`` where each operand is stored either
K-major (``[rows, K]``) or MN-major (``[K, rows]``); this gives the three linear
layer products without transposes:

* forward          ``y = x @ w.T``      -> ``gemm(x, w)``
* input gradient   ``dx = dy @ w``      -> ``gemm(dy, w, b_mn=True)``
* weight gradient  ``dw = dy.T @ x``    -> ``gemm(dy, x, a_mn=True, b_mn=True)``

Reference counterpart: the linear kernels and cuBLASLt call sites of
neuralfn/csrc/tile_cuda/kernels.cu:16746-17574.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

EPI_BIAS = 1 << 0
EPI_SAVE_PRE = 1 << 1
EPI_RESID = 1 << 2
EPI_DACT = 1 << 3
EPI_ACCUM = 1 << 4
EPI_OUT_F32 = 1 << 5
EPI_ACT_SHIFT = 8
ACT_IDS = {"none": 0, None: 0, "gelu_tanh": 1, "gelu": 1, "gelu_erf": 2, "silu": 3, "relu2": 4,
           "tanh_cap": 5, "relu": 6}


def _check2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with a contiguous last dimension, got "
                         f"shape={tuple(t.shape)} stride={t.stride()}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16")


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: torch.Tensor | None = None, act: str | None = None, act_param: float = 0.0,
         save_pre: torch.Tensor | None = None, resid: torch.Tensor | None = None,
         dact_pre: torch.Tensor | None = None, accum: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
         alpha: float = 1.0, workspace: torch.Tensor | None = None, split_k: int = 0) -> torch.Tensor:
    _check2d(a, "a")
    _check2d(b, "b")
    if a_mn:
        k, m = a.shape
    else:
        m, k = a.shape
    if b_mn:
        kb, n = b.shape
    else:
        n, kb = b.shape
    if kb != k:
        raise ValueError(f"contraction mismatch: {k} vs {kb}")
    if out is None:
        out = torch.empty((m, n), device=a.device, dtype=out_dtype)
    if out.shape != (m, n) or out.stride(1) != 1:
        raise ValueError("bad out tensor")
    flags = ACT_IDS[act] << EPI_ACT_SHIFT
    args = _lib.GemmArgs()
    args.a, args.b, args.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.m, args.n, args.k = m, n, k
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), out.stride(0)
    args.a_mn, args.b_mn = int(a_mn), int(b_mn)
    args.alpha, args.act_param = alpha, act_param
    if bias is not None:
        if bias.dtype != torch.bfloat16 or bias.numel() != n:
            raise ValueError("bias must be bf16 [N]")
        flags |= EPI_BIAS
        args.bias = bias.data_ptr()
    if save_pre is not None:
        flags |= EPI_SAVE_PRE
        args.aux_out, args.ld_aux_out = save_pre.data_ptr(), save_pre.stride(0)
    if resid is not None:
        _check2d(resid, "resid")
        flags |= EPI_RESID
        args.aux_in, args.ld_aux_in = resid.data_ptr(), resid.stride(0)
    if dact_pre is not None:
        _check2d(dact_pre, "dact_pre")
        flags |= EPI_DACT
        args.aux_in, args.ld_aux_in = dact_pre.data_ptr(), dact_pre.stride(0)
    if accum:
        flags |= EPI_ACCUM
    if out.dtype == torch.float32:
        flags |= EPI_OUT_F32
    elif out.dtype != torch.bfloat16:
        raise ValueError("out must be bf16 or fp32")
    args.flags = flags
    if workspace is not None:
        args.workspace = workspace.data_ptr()
        args.workspace_bytes = workspace.numel() * workspace.element_size()
        args.split_k = split_k
    else:
        args.split_k = 1
    rc = _lib.load().nfn_gemm_bf16(ctypes.byref(args), ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "nfn_gemm_bf16")
    return out


def gemm_grouped_k(a: torch.Tensor, b: torch.Tensor, group_rows: torch.Tensor, out: torch.Tensor, *, alpha: float = 1.0, accum: bool = False) -> torch.Tensor:
    """out[g] = alpha * a[r0:r1]^T @ b[r0:r1] with (r0, r1) = group_rows[g], group_rows[g + 1], for every group in ONE launch and
    without reading the offsets on the host: the weight gradients of all experts of an MoE layer over the expert-sorted token
    buffer. ``a`` [rows, M] and ``b`` [rows, N] bf16 (row pitch free, columns contiguous), ``group_rows`` int32 [G + 1] on the
    device, multiples of 64, with the padding rows of every group zero in at least one operand and finite in both;
    ``out`` [G, M, N] bf16 or fp32, contiguous in its last two dimensions. A group without rows gives zeros.

    The reference computes these per token inside ``moe_swiglu_backward`` (``kernels.cu:12700-12862``, atomics into dense
    weight gradients); here they are tcgen05 tiles over (group, m-tile, n-tile) whose K loop walks the group's rows."""
    _check2d(a, "a")
    _check2d(b, "b")
    rows, m = a.shape
    n = b.shape[1]
    G = group_rows.numel() - 1
    if b.shape[0] != rows or out.shape != (G, m, n) or out.stride(2) != 1 or out.stride(1) < n or group_rows.dtype != torch.int32:
        raise ValueError("gemm_grouped_k: a [rows, M], b [rows, N], group_rows int32 [G + 1], out [G, M, N]")
    flags = 0
    if accum:
        flags |= EPI_ACCUM
    if out.dtype == torch.float32:
        flags |= EPI_OUT_F32
    elif out.dtype != torch.bfloat16:
        raise ValueError("out must be bf16 or fp32")
    args = _lib.GemmArgs()
    args.a, args.b, args.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.m, args.n, args.k = m, n, rows
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), out.stride(1)
    args.a_mn, args.b_mn = 1, 1
    args.alpha, args.flags, args.split_k = alpha, flags, 1
    L = _lib.load()
    rc = L.nfn_gemm_grouped_k(ctypes.byref(args), ctypes.c_void_p(group_rows.data_ptr()), ctypes.c_int(G), ctypes.c_longlong(out.stride(0)),
                              ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "nfn_gemm_grouped_k")
    return out
