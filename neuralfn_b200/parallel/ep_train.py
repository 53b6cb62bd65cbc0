"""Expert-parallel MoE feed-forward for TRAINING: experts split across the ranks of a group, every
rank keeps its own tokens (data parallel outside the layer), gradients flow through the exchange.

    y = ExpertParallelFFN(...)(x [T, d], routing_weights [T, k], routing_indices [T, k])

Forward on every rank: sort the (token, slot) assignments by global expert id -> exchange the
per-expert counts -> all-to-all of the token rows to the ranks that own the experts -> local
dropless expert FFN (grouped tcgen05 GEMMs on CUDA, see ``ops.moe.moe_experts``; a PyTorch loop
on CPU) -> all-to-all back -> multiply by the routing weights and add into the token rows.
Backward is the mirror image: the all-to-all is its own adjoint with the split sizes swapped, so
row gradients travel to the owners, expert weight gradients stay local to the owner, and input /
routing-weight gradients come back with the rows.

The exchange here is ``torch.distributed.all_to_all_single`` (NCCL on GPUs, gloo in the CPU
tests); the forward-only serving path in ``parallel/ep.py`` is the one that moves rows by this
framework's own peer-memory kernels. Split sizes are data dependent, so each call reads one small
count tensor back to the host.

The reference has no expert parallelism: its MoE trainers keep dense ``[E, d, h]`` expert tensors
on one GPU (``kernels.cu:12612-12862``); the routing math (softmax / sigmoid scores, top-k,
renormalisation, density balance loss) is that of ``neuralfn/torch_backend.py:2795-2952``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..tensor.stages_moe import grouped_swiglu_experts

__all__ = ["ExpertParallelFFN", "expert_parallel_ffn", "all_to_all_rows"]


class _AllToAllRows(torch.autograd.Function):
    """rows [sum(send), d] -> [sum(recv), d]; the gradient takes the opposite route."""

    @staticmethod
    def forward(ctx, rows, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = rows.new_empty((sum(recv), rows.shape[1]))
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, dout):
        din = dout.new_empty((sum(ctx.send), dout.shape[1]))
        dist.all_to_all_single(din, dout.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv, group=ctx.group)
        return din, None, None, None


def all_to_all_rows(rows: torch.Tensor, send: list[int], recv: list[int], group=None) -> torch.Tensor:
    return _AllToAllRows.apply(rows, send, recv, group)


class ExpertParallelFFN(nn.Module):
    """SwiGLU experts ``w1 / w3 [E_local, d, h]`` (gate / up) and ``w2 [E_local, h, d]``; global
    expert e lives on rank ``e // E_local``."""

    def __init__(self, model_dim: int, hidden_dim: int, n_experts: int, group=None, *, device=None, dtype=None, seed: int = 0) -> None:
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_experts % self.world:
            raise ValueError(f"{n_experts} experts do not divide over {self.world} ranks")
        self.n_experts, self.local = n_experts, n_experts // self.world
        gen = torch.Generator().manual_seed(seed)
        full = [torch.randn(n_experts, *shape, generator=gen) * 0.02 for shape in ((model_dim, hidden_dim), (hidden_dim, model_dim), (model_dim, hidden_dim))]
        lo = self.rank * self.local
        self.w1, self.w2, self.w3 = (nn.Parameter(t[lo:lo + self.local].to(device=device, dtype=dtype).contiguous()) for t in full)

    @torch.no_grad()
    def load_full(self, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor) -> None:
        lo = self.rank * self.local
        for p, t in ((self.w1, w1), (self.w2, w2), (self.w3, w3)):
            p.copy_(t[lo:lo + self.local])

    def forward(self, x: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        return expert_parallel_ffn(x, weights, indices, self.w1, self.w2, self.w3, self.n_experts, self.group)


def expert_parallel_ffn(x: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor,
                        n_experts: int, group=None) -> torch.Tensor:
    """Functional form: ``w1 / w2 / w3`` are this rank's experts ``[n_experts / W, ...]``."""
    T, d = x.shape
    W = dist.get_world_size(group) if dist.is_initialized() else 1
    k, E, local = indices.shape[-1], n_experts, w1.shape[0]
    if local * W != E:
        raise ValueError(f"{local} local experts x {W} ranks != {E} experts")
    flat_e = indices.reshape(-1)
    order = torch.argsort(flat_e, stable=True)            # assignments sorted by global expert (hence by owner rank)
    token_of = order // k
    counts = torch.bincount(flat_e, minlength=E)          # [E] rows this rank sends to every expert
    if W > 1:
        theirs = torch.empty_like(counts)                 # [W * local]: rows every rank sends to MY experts, by source rank
        dist.all_to_all_single(theirs, counts, group=group)
        both = torch.stack([counts, theirs]).cpu()
        send = both[0].view(W, local).sum(1).tolist()
        recv_counts = both[1].view(W, local)
        recv = recv_counts.sum(1).tolist()
    else:
        recv_counts = counts.cpu().view(1, E)
        send = recv = [int(recv_counts.sum())]
    rows = x[token_of]
    got = all_to_all_rows(rows, send, recv, group) if W > 1 else rows
    # local expert id of every received row: per source rank the rows come sorted by expert
    local_id = torch.repeat_interleave(torch.arange(local).repeat(recv_counts.shape[0]), recv_counts.reshape(-1)).to(x.device)
    n = got.shape[0]
    if n:
        ones = torch.ones(n, 1, dtype=torch.float32, device=x.device)
        ys = grouped_swiglu_experts(got, w1, w2, w3, ones, local_id.view(n, 1))
    else:
        ys = got * (w1.sum() + w2.sum() + w3.sum()) * 0  # keeps the parameters in the graph
    back = all_to_all_rows(ys, recv, send, group) if W > 1 else ys
    wsorted = weights.reshape(-1)[order].unsqueeze(-1).to(back.dtype)
    out = torch.zeros(T, d, dtype=back.dtype, device=x.device)
    return out.index_add(0, token_of, back * wsorted)
