"""Expert-parallel MoE feed-forward for TRAINING on this framework's own peer-memory kernels: the token
rows, their gradients and the per-row scalars cross NVLink by pull kernels in both passes; the step
makes no library all-to-all.

    exch = PeerExchange(n_experts, top_k, model_dim, max_tokens, device, group)
    y = fused_expert_parallel_ffn(x, weights, indices, w1, w2, w3, exch)       # same math as parallel.ep_train

Forward on every rank: per-expert counts -> one kernel publishes them to every peer and waits for
theirs -> plan (where each (expert, source) segment sits in the owner's receive buffer, where this rank's
rows will be found again) -> sort rows by expert into the symmetric send buffer -> flag -> owners PULL
their segments -> grouped tcgen05 GEMMs + SwiGLU on the owned experts -> flag -> sources PULL-combine
their rows out of the owners' output buffers with the routing weights.

Backward takes the same route with the roles of the buffers swapped. The upstream gradient of every
(token, slot) is scattered to the send-buffer row its activation used (``nfn_moe_scatter_rows``), the
owners pull it, scale it by the routing weight they pulled in the forward pass (``nfn_moe_ep_pull_f32``),
run the grouped input-gradient GEMMs and per-expert weight-gradient products, and leave the row gradients
in the symmetric buffer where the sources pull-combine them. The routing-weight gradient <upstream,
expert output> is formed at the owner, one scalar per row, and read back by ``nfn_moe_ep_gather_f32``.

One small device-to-host read per call gives the number of received rows, which sizes the saved
activations (the NCCL path reads its split sizes the same way). CUDA bf16 only; ``parallel.ep_train``
is the portable path (gloo ranks in the CPU tests) and the oracle.

The reference has no expert parallelism (dense ``[E, d, h]`` experts on one GPU,
``neuralfn/csrc/tile_cuda/kernels.cu:12612-12862``); routing math as ``neuralfn/torch_backend.py:2795-2952``.
"""
from __future__ import annotations

from ctypes import c_int, c_void_p
from types import SimpleNamespace

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import kernels as K
from ..ops.gemm import gemm, gemm_grouped_k
from ..ops.infer import swiglu_backward, swiglu_forward
from ..ops.moe import _grouped_gemm
from .tp import _Symmetric

__all__ = ["PeerExchange", "fused_expert_parallel_ffn", "fused_exchange_ok"]


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _st():
    return c_void_p(_lib.stream_ptr())


def _arr(ptrs):
    return (c_void_p * len(ptrs))(*[c_void_p(int(p)) for p in ptrs])


class PeerExchange:
    """Symmetric buffers shared by every MoE layer of a model (the layers run one after another).

    ``capacity_factor`` bounds the rows one rank can receive: ``factor * max_tokens * top_k`` (+ tile
    padding). ``world`` (the default) can never overflow; a balanced router needs about 1. A call that
    would overflow raises before anything is pulled."""

    def __init__(self, n_experts: int, top_k: int, model_dim: int, max_tokens: int, device, group=None, *, capacity_factor: float | None = None) -> None:
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_experts % self.world or self.world > 8:
            raise ValueError("n_experts must be a multiple of the world size (at most 8 ranks)")
        if model_dim % 8:
            raise ValueError("model_dim must be a multiple of 8")
        self.E, self.El, self.k, self.d, self.T = n_experts, n_experts // self.world, top_k, model_dim, max_tokens
        self.device = torch.device(device)
        W = self.world
        factor = float(W if capacity_factor is None else capacity_factor)
        self.cap = (int(factor * max_tokens * top_k) + self.El * 127 + 127) // 128 * 128
        self.max_tiles = self.cap // 128
        sym = lambda n, dt: _Symmetric(n, dt, self.device, group, W)  # noqa: E731
        self.send = sym(max_tokens * top_k * model_dim, torch.bfloat16)   # rows sorted by expert (activations, then gradients)
        self.recv = sym(self.cap * model_dim, torch.bfloat16)             # owner side: expert outputs, then row gradients
        self.fsend = sym(max_tokens * top_k, torch.float32)               # routing weight of every sent row
        self.frecv = sym(self.cap, torch.float32)                         # owner side: <upstream, output> per row
        self.table = sym(W * n_experts, torch.int32)
        self.flags = sym(8 * W, torch.int32)
        self.epoch = 0
        self.ones = torch.ones(max_tokens, top_k, dtype=torch.float32, device=self.device)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if W > 1:
            dist.barrier(group)

    def barrier(self, slot: int) -> None:
        """Every rank has reached this point of the call (flag exchange on the stream, bounded wait)."""
        if self.world == 1:
            return
        K.peer_arrive(self.flags.ptrs, self.rank, self.world, slot, self.epoch)
        K.peer_wait(self.flags.t.data_ptr(), self.world, slot, self.epoch, timeout_s=10.0)


def fused_exchange_ok(x: torch.Tensor, w1: torch.Tensor) -> bool:
    _E, d, h = w1.shape
    return x.is_cuda and x.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and _lib.available() and d % 64 == 0 and h % 64 == 0


class _FusedEPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, w2, w3, weights, indices, ex: PeerExchange):
        L = _lib.load()
        T, d = x.shape
        El, _, F = w1.shape
        E, W, k = ex.E, ex.world, ex.k
        if T > ex.T or d != ex.d or indices.shape[-1] != k or El != ex.El:
            raise ValueError("batch does not fit the exchange buffers it was given")
        dev = x.device
        i32 = dict(dtype=torch.int32, device=dev)
        ex.epoch += 1
        idx = indices.to(torch.int32).contiguous()
        wts = weights.to(torch.float32).contiguous()
        counts = torch.bincount(idx.reshape(-1), minlength=E).to(torch.int32)
        src_off, cursor, recv_off = torch.zeros(E + 1, **i32), torch.zeros(E, **i32), torch.zeros(El + 1, **i32)
        seg_src, seg_dst, seg_rows = (torch.zeros(El * W, **i32) for _ in range(3))
        home_row, tile_expert, plan = torch.zeros(E, **i32), torch.zeros(ex.max_tiles, **i32), torch.zeros(2, **i32)
        row_of = torch.empty(T * k, **i32)
        _lib.check(L.nfn_moe_ep_exchange_counts(_p(counts), c_int(E), _arr(ex.table.ptrs), _arr(ex.flags.ptrs), c_int(ex.rank), c_int(W),
                                                c_int(ex.epoch), c_void_p(0), _st()), "nfn_moe_ep_exchange_counts")
        _lib.check(L.nfn_moe_ep_plan(_p(ex.table.t), c_int(E), c_int(W), c_int(ex.rank), c_int(ex.max_tiles), _p(src_off), _p(cursor), _p(recv_off),
                                     _p(seg_src), _p(seg_dst), _p(seg_rows), _p(home_row), _p(tile_expert), _p(plan), _st()), "nfn_moe_ep_plan")
        _lib.check(L.nfn_moe_permute(_p(x), c_int(x.stride(0)), c_int(T), c_int(k), c_int(d), _p(idx), _p(src_off), _p(cursor), c_int(ex.T * k),
                                     _p(ex.send.t), _p(row_of), _st()), "nfn_moe_permute")
        ex.fsend.t[row_of.long()] = wts.reshape(-1)
        ex.barrier(1)
        host = torch.cat([plan, recv_off, seg_rows]).cpu()                 # the one device-to-host read of the call
        n_rows = int(host[1])
        if n_rows > ex.cap:
            raise RuntimeError(f"{n_rows} rows arrive at rank {ex.rank} but the exchange holds {ex.cap}: raise capacity_factor")
        offs = host[2:2 + El + 1].tolist()
        per_expert = host[2 + El + 1:].view(El, W).sum(1).tolist()
        xs = torch.zeros(max(n_rows, 128), d, dtype=torch.bfloat16, device=dev)    # padding rows stay zero
        w_rows = torch.zeros(max(n_rows, 128), dtype=torch.float32, device=dev)
        seg = (seg_src, seg_dst, seg_rows)
        _lib.check(L.nfn_moe_ep_pull(_arr(ex.send.ptrs), _p(seg_src), _p(seg_dst), _p(seg_rows), c_int(El), c_int(W), c_int(d), c_int(xs.shape[0]),
                                     _p(xs), _st()), "nfn_moe_ep_pull")
        _lib.check(L.nfn_moe_ep_pull_f32(_arr(ex.fsend.ptrs), _p(seg_src), _p(seg_dst), _p(seg_rows), c_int(El), c_int(W), c_int(w_rows.shape[0]),
                                         _p(w_rows), _st()), "nfn_moe_ep_pull_f32")
        tiles = SimpleNamespace(tile_expert=tile_expert, plan=plan)
        w_gu = torch.cat([w1.transpose(1, 2), w3.transpose(1, 2)], 1).contiguous()   # [El, 2F, d]
        w_dn = w2.transpose(1, 2).contiguous()                                       # [El, d, F]
        h = torch.empty(xs.shape[0], 2 * F, dtype=torch.bfloat16, device=dev)
        a = torch.empty(xs.shape[0], F, dtype=torch.bfloat16, device=dev)
        ys = ex.recv.t[:xs.shape[0] * d].view(xs.shape[0], d)
        _grouped_gemm(xs, w_gu, h, tiles)
        swiglu_forward(h, F, out=a)
        _grouped_gemm(a, w_dn, ys, tiles)
        ex.barrier(2)
        out = torch.empty(T, d, dtype=torch.bfloat16, device=dev)
        _lib.check(L.nfn_moe_ep_combine(_arr(ex.recv.ptrs), c_int(d), c_int(T), c_int(k), c_int(E), c_int(W), _p(idx), _p(row_of), _p(src_off),
                                        _p(home_row), _p(wts), _p(None), c_int(0), _p(out), c_int(out.stride(0)), _st()), "nfn_moe_ep_combine")
        ys_keep = ys.clone()                     # the symmetric buffer is reused by the next layer
        ex.barrier(3)                            # nobody refills send / recv while a peer still reads them
        ctx.ex, ctx.tiles, ctx.seg, ctx.route = ex, tiles, seg, (idx, wts, row_of, src_off, home_row)
        ctx.dims, ctx.segments, ctx.w_dtype, ctx.recv_off = (T, d, F, n_rows), (offs, per_expert), weights.dtype, recv_off
        ctx.save_for_backward(w1, w2, w3, xs, h, a, ys_keep, w_rows)
        return out

    @staticmethod
    def backward(ctx, dout):
        L = _lib.load()
        w1, w2, w3, xs, h, a, ys, w_rows = ctx.saved_tensors
        ex, tiles, (seg_src, seg_dst, seg_rows) = ctx.ex, ctx.tiles, ctx.seg
        idx, wts, row_of, src_off, home_row = ctx.route
        (T, d, F, n_rows), (offs, per_expert) = ctx.dims, ctx.segments
        E, El, W, k, dev = ex.E, ex.El, ex.world, ex.k, dout.device
        dout = dout.contiguous()
        ex.epoch += 1
        _lib.check(L.nfn_moe_scatter_rows(_p(dout), c_int(dout.stride(0)), c_int(T), c_int(k), c_int(d), _p(row_of), c_int(ex.T * k), _p(ex.send.t),
                                          _st()), "nfn_moe_scatter_rows")
        ex.barrier(1)
        rows = xs.shape[0]
        dyo = torch.zeros(rows, d, dtype=torch.bfloat16, device=dev)      # padding rows zero: they add nothing to the weight gradients
        _lib.check(L.nfn_moe_ep_pull(_arr(ex.send.ptrs), _p(seg_src), _p(seg_dst), _p(seg_rows), c_int(El), c_int(W), c_int(d), c_int(rows), _p(dyo),
                                     _st()), "nfn_moe_ep_pull")
        torch.sum(dyo.float() * ys.float(), dim=1, out=ex.frecv.t[:rows])  # d(routing weight) of every row, read back by its source
        dys = (dyo.float() * w_rows[:, None]).to(torch.bfloat16)
        da = torch.empty(rows, F, dtype=torch.bfloat16, device=dev)
        _grouped_gemm(dys, w2.contiguous(), da, tiles)                     # [rows, F] = dys @ w2[e]^T
        dh = swiglu_backward(h, da, F)
        dxs = ex.recv.t[:rows * d].view(rows, d)
        _grouped_gemm(dh, torch.cat([w1, w3], 2).contiguous(), dxs, tiles)  # [rows, d] = dh @ [w1 | w3][e]^T
        ex.barrier(2)
        dx = torch.empty(T, d, dtype=torch.bfloat16, device=dev)
        _lib.check(L.nfn_moe_ep_combine(_arr(ex.recv.ptrs), c_int(d), c_int(T), c_int(k), c_int(E), c_int(W), _p(idx), _p(row_of), _p(src_off),
                                        _p(home_row), _p(ex.ones), _p(None), c_int(0), _p(dx), c_int(dx.stride(0)), _st()), "nfn_moe_ep_combine")
        d_w = torch.empty(T, k, dtype=torch.float32, device=dev)
        _lib.check(L.nfn_moe_ep_gather_f32(_arr(ex.frecv.ptrs), c_int(T), c_int(k), c_int(E), c_int(W), _p(idx), _p(row_of), _p(src_off), _p(home_row),
                                           _p(d_w), _st()), "nfn_moe_ep_gather_f32")
        # weight gradients stay with the owner: three grouped contractions over the received (128-row padded) segments; the
        # padding rows of xs and dys are zero, those of a and dh finite
        dw1, dw2, dw3 = torch.empty_like(w1), torch.empty_like(w2), torch.empty_like(w3)
        gemm_grouped_k(xs, dh[:, :F], ctx.recv_off, dw1)
        gemm_grouped_k(xs, dh[:, F:], ctx.recv_off, dw3)
        gemm_grouped_k(a, dys, ctx.recv_off, dw2)
        ex.barrier(3)
        return dx, dw1, dw2, dw3, d_w.to(ctx.w_dtype), None, None


def fused_expert_parallel_ffn(x: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor,
                              exchange: PeerExchange) -> torch.Tensor:
    """x [T, d] bf16, routing weights / indices [T, k], this rank's experts w1 / w3 [E / W, d, h] and w2 [E / W, h, d]."""
    return _FusedEPFn.apply(x.contiguous(), w1, w2, w3, weights, indices, exchange)
