"""Expert-parallel mixture-of-experts layer: experts split across the ranks of one NVSwitch
domain, tokens exchanged through peer memory by this framework's own kernels (no NCCL
all-to-all).

Per call, on one stream: router GEMM -> top-k routing -> publish per-expert counts to every
peer and wait for theirs (one kernel) -> plan (segment table, tile table) -> sort local
tokens by expert into a symmetric send buffer -> flag "send buffer ready" -> PULL the
segments of the locally owned experts from the peers' send buffers -> grouped tcgen05 GEMMs
with SwiGLU on the owned experts -> flag "outputs ready" -> PULL-combine: every source reads
its rows from the owners' output buffers and applies the routing weights -> flag "done".

With ``world == 1`` the same code runs without symmetric memory and equals ``ops.moe``.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import kernels as K
from ..ops.gemm import gemm
from ..ops.infer import swiglu_forward
from ..ops.moe import _grouped_gemm
from .tp import _Symmetric

__all__ = ["ExpertParallelMoE"]


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _st():
    return c_void_p(_lib.stream_ptr())


def _arr(ptrs):
    return (c_void_p * len(ptrs))(*[c_void_p(int(p)) for p in ptrs])


class ExpertParallelMoE:
    """Holds the buffers for up to ``max_tokens`` local tokens. ``w_gate_up`` [E_local, 2F, d] and
    ``w_down`` [E_local, d, F] are this rank's experts (global ids rank * E_local ...)."""

    def __init__(self, n_experts: int, top_k: int, d_model: int, d_ff: int, max_tokens: int, device, group=None) -> None:
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_experts % self.world or self.world > 8:
            raise ValueError("n_experts must be a multiple of the world size (at most 8 ranks)")
        self.E, self.El, self.k, self.d, self.F = n_experts, n_experts // self.world, top_k, d_model, d_ff
        self.device = torch.device(device)
        W, T = self.world, max_tokens
        self.max_tokens = T
        self.cap = (W * T * top_k + self.El * 127 + 127) // 128 * 128
        self.max_tiles = self.cap // 128
        i32 = dict(dtype=torch.int32, device=self.device)
        bf = dict(dtype=torch.bfloat16, device=self.device)
        sym = lambda n, dt: _Symmetric(n, dt, self.device, group, W)  # noqa: E731
        self.send = sym(T * top_k * d_model, torch.bfloat16)
        self.ys = sym(self.cap * d_model, torch.bfloat16)
        self.table = sym(W * n_experts, torch.int32)
        self.flags = sym(8 * W, torch.int32)  # slot 0: counts, 1: send ready, 2: outputs ready, 3: done
        self.logits = torch.empty(T, (n_experts + 7) // 8 * 8, dtype=torch.float32, device=self.device)
        self.topk_idx, self.topk_w = torch.empty(T, top_k, **i32), torch.empty(T, top_k, dtype=torch.float32, device=self.device)
        self.counts, self.src_off, self.cursor = torch.zeros(n_experts, **i32), torch.zeros(n_experts + 1, **i32), torch.zeros(n_experts, **i32)
        self.recv_off = torch.zeros(self.El + 1, **i32)
        self.seg_src, self.seg_dst, self.seg_rows = (torch.zeros(self.El * W, **i32) for _ in range(3))
        self.home_row = torch.zeros(n_experts, **i32)
        self.tile_expert, self.plan = torch.zeros(self.max_tiles, **i32), torch.zeros(2, **i32)
        self.row_of = torch.empty(T * top_k, **i32)
        self.xs, self.h, self.a = torch.zeros(self.cap, d_model, **bf), torch.empty(self.cap, 2 * d_ff, **bf), torch.empty(self.cap, d_ff, **bf)
        self.epoch = 0
        self._router_pad = None
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if W > 1:
            dist.barrier(group)

    def _barrier(self, slot: int) -> None:
        """Cross-rank flag exchange on the stream: everyone has reached this point of the call."""
        if self.world == 1:
            return
        K.peer_arrive(self.flags.ptrs, self.rank, self.world, slot, self.epoch)
        K.peer_wait(self.flags.t.data_ptr(), self.world, slot, self.epoch, timeout_s=10.0)

    def forward(self, x: torch.Tensor, w_router: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, *, score_fn: str = "softmax",
                norm_topk: bool = True, route_scale: float = 1.0, resid: torch.Tensor | None = None) -> torch.Tensor:
        T, d = x.shape
        if T > self.max_tokens:
            raise ValueError("more tokens than the layer was sized for")
        L, E, W, k = _lib.load(), self.E, self.world, self.k
        self.epoch += 1
        # the GEMM wants N in multiples of 8: pad the router once
        if E % 8:
            if self._router_pad is None or self._router_pad[1] != (w_router.data_ptr(), w_router._version):
                pad = torch.zeros(self.logits.shape[1], d, dtype=w_router.dtype, device=self.device)
                pad[:E].copy_(w_router)
                self._router_pad = (pad, (w_router.data_ptr(), w_router._version))
            w_router = self._router_pad[0]
        gemm(x, w_router, out=self.logits[:T, :w_router.shape[0]], out_dtype=torch.float32)
        self.counts.zero_()
        _lib.check(L.nfn_moe_route(_p(self.logits), c_int(self.logits.stride(0)), c_int(T), c_int(E), c_int(k), c_int(1 if score_fn == "sigmoid" else 0),
                                   c_int(int(norm_topk)), c_float(route_scale), _p(self.topk_idx), _p(self.topk_w), _p(self.counts), _st()), "nfn_moe_route")
        _lib.check(L.nfn_moe_ep_exchange_counts(_p(self.counts), c_int(E), _arr(self.table.ptrs), _arr(self.flags.ptrs), c_int(self.rank), c_int(W),
                                                c_int(self.epoch), c_void_p(0), _st()), "nfn_moe_ep_exchange_counts")
        _lib.check(L.nfn_moe_ep_plan(_p(self.table.t), c_int(E), c_int(W), c_int(self.rank), c_int(self.max_tiles), _p(self.src_off), _p(self.cursor),
                                     _p(self.recv_off), _p(self.seg_src), _p(self.seg_dst), _p(self.seg_rows), _p(self.home_row), _p(self.tile_expert),
                                     _p(self.plan), _st()), "nfn_moe_ep_plan")
        _lib.check(L.nfn_moe_permute(_p(x), c_int(x.stride(0)), c_int(T), c_int(k), c_int(d), _p(self.topk_idx), _p(self.src_off), _p(self.cursor),
                                     c_int(self.max_tokens * k), _p(self.send.t), _p(self.row_of), _st()), "nfn_moe_permute")
        self._barrier(1)
        _lib.check(L.nfn_moe_ep_pull(_arr(self.send.ptrs), _p(self.seg_src), _p(self.seg_dst), _p(self.seg_rows), c_int(self.El), c_int(W), c_int(d),
                                     c_int(self.cap), _p(self.xs), _st()), "nfn_moe_ep_pull")
        ws = self  # the grouped GEMM helper reads tile_expert / plan from its workspace argument
        _grouped_gemm(self.xs, w_gate_up, self.h, ws)
        swiglu_forward(self.h, self.F, out=self.a)
        _grouped_gemm(self.a, w_down, self.ys.t.view(self.cap, d), ws)
        self._barrier(2)
        out = torch.empty(T, d, dtype=torch.bfloat16, device=self.device)
        _lib.check(L.nfn_moe_ep_combine(_arr(self.ys.ptrs), c_int(d), c_int(T), c_int(k), c_int(E), c_int(W), _p(self.topk_idx), _p(self.row_of),
                                        _p(self.src_off), _p(self.home_row), _p(self.topk_w), _p(resid), c_int(0 if resid is None else resid.stride(0)),
                                        _p(out), c_int(out.stride(0)), _st()), "nfn_moe_ep_combine")
        self._barrier(3)  # nobody overwrites send / output buffers of the next call while a peer still reads these
        return out
