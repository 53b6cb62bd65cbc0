"""Tensor-parallel linears whose collective runs inside the GEMM kernel.

``TensorParallelContext`` owns the symmetric (peer-visible) buffers of one TP group:
gathered-activation buffers, reduce-scatter slot buffers, a control block of flags and a
device-resident epoch counter. ``column_linear`` is all-gather -> GEMM (sequence-sharded
input, column-sharded weight), ``row_linear`` is GEMM -> reduce-scatter (column-sharded
input, row... K-sharded weight; sequence-sharded output), ``gathered_weight_linear`` gathers
a row-sharded weight into the GEMM that consumes it (parameter sharding).

Each has three implementations selected by ``impl``:
  * ``"fused"``  one ``nfn_gemm_tp`` launch (peer memory, no NCCL call) - the product;
  * ``"nccl"``   NCCL all-gather / reduce-scatter around the plain tcgen05 GEMM - the baseline
                 the fused path is measured against;
  * ``"torch"``  torch.distributed + torch.matmul in fp32 (CPU / gloo tests, oracle).

The reference has no tensor parallelism (its TODO list names it, ``todo-kernels.md:133-145``);
the sharding conventions follow the usual Megatron column/row split so checkpoints of the
unsharded model load by slicing.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch
import torch.distributed as dist

from ..ops import _lib

__all__ = ["TensorParallelContext", "GemmTpArgs"]

AG_A, AG_B, RS = 0, 1, 2
_ACT = {None: 0, "none": 0, "gelu_tanh": 1, "gelu": 1, "gelu_erf": 2, "silu": 3, "relu2": 4}
EPI_BIAS, EPI_ACT_SHIFT = 1, 8


class GemmTpArgs(ctypes.Structure):
    _fields_ = [("mode", c_int), ("a", c_void_p), ("b", c_void_p), ("c", c_void_p),
                ("m", c_int), ("n", c_int), ("k", c_int), ("lda", c_int), ("ldb", c_int), ("ldc", c_int),
                ("flags", c_int), ("act_param", c_float), ("bias", c_void_p),
                ("rank", c_int), ("world", c_int), ("rows_per_rank", c_int),
                ("epoch", c_int), ("epoch_dev", c_void_p),
                ("peer_bufs", c_void_p * 8), ("ctrl_local", c_void_p), ("ctrl_peer", c_void_p * 8), ("ctrl_ints", c_int),
                ("out", c_void_p), ("ld_out", c_int), ("resid", c_void_p), ("ld_resid", c_int), ("n_copy", c_int),
                ("tile_group", c_void_p), ("num_m_tiles_dev", c_void_p), ("groups", c_int)]


class _Symmetric:
    """One tensor allocated identically on every rank plus the peers' addresses of it."""

    def __init__(self, numel: int, dtype, device, group, world: int) -> None:
        if world > 1 and device.type == "cuda":
            import torch.distributed._symmetric_memory as symm
            self.t = symm.empty(numel, dtype=dtype, device=device)
            self.t.zero_()
            self.handle = symm.rendezvous(self.t, (group or dist.group.WORLD).group_name)
            self.ptrs = list(self.handle.buffer_ptrs)
        else:
            self.t = torch.zeros(numel, dtype=dtype, device=device)
            self.handle = None
            self.ptrs = [self.t.data_ptr()]


class TensorParallelContext:
    CTRL_INTS = 2048

    def __init__(self, device, group=None, impl: str | None = None) -> None:
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ValueError("a tensor-parallel group spans at most the 8 GPUs of one NVSwitch domain")
        self.impl = impl or ("fused" if self.device.type == "cuda" else "torch")
        self._bufs: dict[tuple, _Symmetric] = {}
        self._parity: dict[tuple, int] = {}
        self.epoch = 0
        if self.impl == "fused":
            self.ctrl = _Symmetric(self.CTRL_INTS, torch.int32, self.device, group, self.world)
            self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._sync()

    def _sync(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)

    # ---- symmetric scratch, two of each (kind, shape) so consecutive calls never share one ----
    def _buffer(self, kind: str, numel: int) -> _Symmetric:
        key = (kind, numel)
        par = self._parity.get(key, 0)
        self._parity[key] = par ^ 1
        full = (kind, numel, par)
        if full not in self._bufs:
            self._bufs[full] = _Symmetric(numel, torch.bfloat16, self.device, self.group, self.world)
            self._sync()
        return self._bufs[full]

    def gather_buffer(self, rows_local: int, K: int) -> tuple[torch.Tensor, "_Symmetric"]:
        """Symmetric [world * rows_local, K] buffer and the view of this rank's own rows:
        produce the activation straight into the view, then call ``column_linear(buffer=...)``."""
        sym = self._buffer("ag", self.world * rows_local * K)
        full = sym.t.view(self.world * rows_local, K)
        return full[self.rank * rows_local:(self.rank + 1) * rows_local], sym

    def _next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def _launch(self, mode: int, a, b, c, m, n, k, rows_per_rank, peer_ptrs, *, bias=None, act=None, out=None, resid=None,
                n_copy: int = 0) -> None:
        args = GemmTpArgs()
        args.mode = mode
        args.a, args.b, args.c = a.data_ptr(), b.data_ptr(), (0 if c is None else c.data_ptr())
        args.m, args.n, args.k = m, n, k
        args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), (n if c is None else c.stride(0))
        args.flags = (EPI_BIAS if bias is not None else 0) | (_ACT[act] << EPI_ACT_SHIFT)
        args.act_param = 0.0
        args.bias = 0 if bias is None else bias.data_ptr()
        args.rank, args.world, args.rows_per_rank = self.rank, self.world, rows_per_rank
        args.epoch, args.epoch_dev = self._next_epoch(), self.epoch_dev.data_ptr()
        for r in range(self.world):
            args.peer_bufs[r] = peer_ptrs[r]
            args.ctrl_peer[r] = self.ctrl.ptrs[r]
        args.ctrl_local = self.ctrl.t.data_ptr()
        args.ctrl_ints = self.CTRL_INTS
        if out is not None:
            args.out, args.ld_out = out.data_ptr(), out.stride(0)
        if resid is not None:
            args.resid, args.ld_resid = resid.data_ptr(), resid.stride(0)
        args.n_copy = n_copy
        _lib.check(_lib.load().nfn_gemm_tp(ctypes.byref(args), c_void_p(_lib.stream_ptr())), "nfn_gemm_tp")

    # ------------------------------------------------------------------ all-gather -> GEMM --
    def column_linear(self, x_local: torch.Tensor, weight: torch.Tensor, bias=None, act=None, *, buffer=None, n_copy: int = 0,
                      return_gathered: bool = False):
        """x_local [rows, K] (this rank's sequence shard), weight [N_local, K] -> [world * rows, N_local].
        Pass ``buffer`` (from ``gather_buffer``) when x_local already lives in its slot. With
        ``return_gathered`` the result is (y, gathered x [world * rows, K]); on the fused path that
        is a view of the symmetric buffer, valid until the second next call with the same shape."""
        rows, K = x_local.shape
        N = weight.shape[0]
        M = rows * self.world
        if self.impl == "torch":
            xs = [torch.empty_like(x_local) for _ in range(self.world)]
            if self.world > 1:
                dist.all_gather(xs, x_local.contiguous(), group=self.group)
            else:
                xs = [x_local]
            xg = torch.cat(xs)
            y = xg.float() @ weight.float().T
            y = y + bias.float() if bias is not None else y
            y = _act_torch(y, act).to(x_local.dtype)
            return (y, xg) if return_gathered else y
        from ..ops.gemm import gemm
        if self.impl == "nccl":
            xg = torch.empty(M, K, dtype=x_local.dtype, device=x_local.device)
            if self.world > 1:
                dist.all_gather_into_tensor(xg, x_local.contiguous(), group=self.group)
            else:
                xg.copy_(x_local)
            y = gemm(xg, weight, bias=bias, act=act)
            return (y, xg) if return_gathered else y
        if buffer is None:
            view, buffer = self.gather_buffer(rows, K)
            view.copy_(x_local)
        xg = buffer.t.view(M, K)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
        self._launch(AG_A, xg, weight, out, M, N, K, rows, buffer.ptrs, bias=bias, act=act, n_copy=n_copy)
        return (out, xg) if return_gathered else out

    # ------------------------------------------------ weight all-gather -> GEMM (sharded params) --
    def gathered_weight_linear(self, x: torch.Tensor, weight_local: torch.Tensor, bias=None, act=None, n_copy: int = 0):
        """x [M, K] (replicated or local batch), weight_local [N / world, K] (this rank's row shard
        of the full weight) -> [M, N]."""
        M, K = x.shape
        rows = weight_local.shape[0]
        N = rows * self.world
        if self.impl in ("torch", "nccl"):
            ws = [torch.empty_like(weight_local) for _ in range(self.world)]
            if self.world > 1:
                dist.all_gather(ws, weight_local.contiguous(), group=self.group)
            else:
                ws = [weight_local]
            w = torch.cat(ws)
            if self.impl == "nccl":
                from ..ops.gemm import gemm
                return gemm(x, w, bias=bias, act=act)
            y = x.float() @ w.float().T
            y = y + bias.float() if bias is not None else y
            return _act_torch(y, act).to(x.dtype)
        sym = self._buffer("agw", N * K)
        wg = sym.t.view(N, K)
        wg[self.rank * rows:(self.rank + 1) * rows].copy_(weight_local)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
        self._launch(AG_B, x, wg, out, M, N, K, rows, sym.ptrs, bias=bias, act=act, n_copy=n_copy)
        return out

    # -------------------------------------------------------------- GEMM -> reduce-scatter --
    def row_linear(self, x: torch.Tensor, weight: torch.Tensor, bias=None, resid=None):
        """x [M, K_local], weight [N, K_local] -> this rank's [M / world, N] rows of
        sum_r x_r W_r^T (+ bias + resid, resid being this rank's [M / world, N] rows)."""
        M, K = x.shape
        N = weight.shape[0]
        rows = M // self.world
        if self.impl == "torch":
            y = x.float() @ weight.float().T
            if self.world > 1:
                dist.all_reduce(y, group=self.group)
            y = y[self.rank * rows:(self.rank + 1) * rows]
            y = y + bias.float() if bias is not None else y
            y = y + resid.float() if resid is not None else y
            return y.to(x.dtype)
        if self.impl == "nccl":
            from ..ops.gemm import gemm
            part = gemm(x, weight)
            out = torch.empty(rows, N, dtype=part.dtype, device=part.device)
            if self.world > 1:
                dist.reduce_scatter_tensor(out, part, group=self.group)
            else:
                out.copy_(part)
            if bias is not None:
                out += bias
            if resid is not None:
                out += resid
            return out
        sym = self._buffer("rs", self.world * rows * N)
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=self.device)
        self._launch(RS, x, weight, None, M, N, K, rows, sym.ptrs, bias=bias, out=out, resid=resid)
        return out

    # ------------------------------------------- decode: all-reduce + residual + RMS norm --
    def partial_buffer(self, rows: int, n: int) -> tuple[torch.Tensor, "_Symmetric"]:
        """Symmetric [rows, n] bf16 buffer for a rank's partial projection output (two
        alternate). Write the partial into it, then call ``allreduce_resid_norm``."""
        sym = self._buffer("ar", rows * n)
        return sym.t.view(rows, n), sym

    def allreduce_resid_norm(self, partial: torch.Tensor, sym: "_Symmetric | None", *, bias=None, resid=None, norm_weight=None,
                             eps: float = 1e-6, centered: bool = False, use_multicast: bool = True, post_weight=None,
                             post_eps: float = 1e-6):
        """sum over ranks of ``partial`` (+ bias + resid, resid updated in place), then RMS
        norm with ``norm_weight`` when given. With ``post_weight`` (sandwich-norm blocks) the summed
        rows are RMS-normalised with it before they join the residual stream. Returns the bf16
        [rows, n] result."""
        rows, n = partial.shape
        if self.impl != "fused":
            y = partial.float().clone()
            if self.world > 1:
                dist.all_reduce(y, group=self.group)
            y = y + bias.float() if bias is not None else y
            if post_weight is not None:
                pw = post_weight.float()
                y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + post_eps) * (1 + pw if centered else pw)
            if resid is not None:
                y = y + resid.float()
                resid.copy_(y.to(resid.dtype))
                y = resid.float()
            if norm_weight is not None:
                w = norm_weight.float()
                y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * (1 + w if centered else w)
            return y.to(partial.dtype)
        assert sym is not None and partial.data_ptr() == sym.t.data_ptr(), "partial must be the symmetric partial_buffer"
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=self.device)
        ptr_arr = (c_void_p * 8)(*sym.ptrs)
        ctrl_arr = (c_void_p * 8)(*[p + 4 * 1024 for p in self.ctrl.ptrs])  # second half of the control block
        mc = 0
        if use_multicast and sym.handle is not None:
            mc = int(getattr(sym.handle, "multicast_ptr", 0) or 0)
        rc = _lib.load().nfn_allreduce_sandwich_norm(
            ptr_arr, c_void_p(mc), c_void_p(self.ctrl.t.data_ptr() + 4 * 1024), ctrl_arr, c_int(self.rank), c_int(self.world),
            c_int(self._next_epoch()), c_void_p(self.epoch_dev.data_ptr()), c_int(rows), c_int(n), c_int(partial.stride(0)),
            c_void_p(0 if bias is None else bias.data_ptr()), c_void_p(0 if post_weight is None else post_weight.data_ptr()),
            c_float(post_eps), c_void_p(0 if resid is None else resid.data_ptr()),
            c_int(0 if resid is None else resid.stride(0)), c_void_p(0 if norm_weight is None else norm_weight.data_ptr()),
            c_float(eps), c_int(int(centered)), c_void_p(out.data_ptr()), c_int(out.stride(0)), c_void_p(_lib.stream_ptr()))
        _lib.check(rc, "nfn_allreduce_resid_norm")
        return out

    def advance_epoch_on_device(self, by: int = 1) -> None:
        """For CUDA-graph replays: bump the device-side epoch base by the number of fused
        calls the captured graph contains."""
        from ..ops import kernels as K
        K.counter_add(self.epoch_dev, by)


def _act_torch(y: torch.Tensor, act) -> torch.Tensor:
    import torch.nn.functional as F
    if act in (None, "none"):
        return y
    if act in ("gelu", "gelu_tanh"):
        return F.gelu(y, approximate="tanh")
    if act == "gelu_erf":
        return F.gelu(y)
    if act == "silu":
        return F.silu(y)
    if act == "relu2":
        return F.relu(y).square()
    raise ValueError(f"unknown activation {act!r}")
