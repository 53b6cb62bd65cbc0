"""Python front-ends of the inference-side kernels: rotary embedding, fused QK-norm + RoPE,
argmax / sampling, split-KV decode attention, K-quant / NF4 dequantisation and the
quantised skinny product. Same conventions as ``ops.kernels``: CUDA tensors in, current
stream, no synchronisation.
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from . import _lib

_bf16 = torch.bfloat16

__all__ = ["rope_tables", "rope_inplace", "qk_norm_rope_forward", "argmax_rows", "argmax_merge", "sample_rows",
           "DecodeAttentionWorkspace", "decode_attention", "BlockAttentionWorkspace", "block_attention", "kv_commit_layers",
           "dequant_kquant", "dequant_nf4", "kquant_gemv", "gemm_kquant", "NF4LoRALinear", "QTYPE_NF4", "quant_block_bytes"]


def _p(t) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _st() -> c_void_p:
    return c_void_p(_lib.stream_ptr())


def rope_tables(max_pos: int, rot_dim: int, base: float = 10000.0, *, inv_freq: torch.Tensor | None = None,
                device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables [max_pos, rot_dim/2]; pass ``inv_freq`` for scaled variants."""
    if inv_freq is None:
        inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv_freq.double().cpu())
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


def _sign(convention) -> float:
    if convention in ("hf", 1, 1.0):
        return 1.0
    if convention in ("legacy", -1, -1.0):
        return -1.0
    raise ValueError("rotary convention must be 'legacy' or 'hf'")


def rope_inplace(qkv, *, T: int, n_q_heads: int, n_kv_heads: int, head_dim: int, cos, sin, convention="legacy",
                 rot_dim: int | None = None, positions=None, q_scale: float = 1.0, backward: bool = False) -> None:
    """Rotates the q and k heads of packed bf16 rows in place. ``backward=True`` applies the
    inverse rotation (the gradient of the forward call; q_scale is applied again)."""
    assert qkv.dtype == _bf16 and qkv.dim() == 2 and qkv.stride(1) == 1
    rot_dim = head_dim if rot_dim is None else rot_dim
    sign = _sign(convention) * (-1.0 if backward else 1.0)
    rc = _lib.load().nfn_rope_inplace(_p(qkv), c_int(qkv.stride(0)), c_longlong(qkv.shape[0]), c_int(T), c_int(n_q_heads),
                                      c_int(n_kv_heads), c_int(head_dim), c_int(rot_dim), _p(cos), _p(sin), _p(positions),
                                      c_int(cos.shape[0]), c_float(sign), c_float(q_scale), _st())
    _lib.check(rc, "nfn_rope_inplace")


def qk_norm_rope_forward(qkv, *, T: int, n_q_heads: int, n_kv_heads: int, head_dim: int, cos, sin, convention="legacy",
                         q_weight=None, k_weight=None, positions=None, eps: float = 1e-6, q_scale: float = 1.0, rstd=None):
    rc = _lib.load().nfn_qk_norm_rope_forward(_p(qkv), c_int(qkv.stride(0)), c_longlong(qkv.shape[0]), c_int(T), c_int(n_q_heads),
                                              c_int(n_kv_heads), c_int(head_dim), _p(q_weight), _p(k_weight), _p(cos), _p(sin),
                                              _p(positions), c_int(cos.shape[0]), c_float(_sign(convention)), c_float(eps),
                                              c_float(q_scale), _p(rstd), _st())
    _lib.check(rc, "nfn_qk_norm_rope_forward")
    return rstd


def argmax_rows(logits, *, index_offset: int = 0, workspace=None, return_values: bool = False):
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype in (_bf16, torch.float32)
    rows, V = logits.shape
    idx = torch.empty(rows, dtype=torch.int32, device=logits.device)
    val = torch.empty(rows, dtype=torch.float32, device=logits.device) if return_values else None
    if workspace is None:
        workspace = torch.empty(rows * 64 * 8, dtype=torch.uint8, device=logits.device)
    rc = _lib.load().nfn_argmax_rows(_p(logits), c_int(logits.dtype == torch.float32), c_longlong(logits.stride(0)), c_int(rows),
                                     c_int(V), _p(idx), _p(val), _p(workspace), c_longlong(workspace.numel()), c_int(index_offset), _st())
    _lib.check(rc, "nfn_argmax_rows")
    return (idx, val) if return_values else idx


def argmax_merge(vals, idx):
    world, rows = vals.shape
    out = torch.empty(rows, dtype=torch.int32, device=vals.device)
    rc = _lib.load().nfn_argmax_merge(_p(vals), _p(idx), c_int(world), c_int(rows), _p(out), _p(None), _st())
    _lib.check(rc, "nfn_argmax_merge")
    return out


def sample_rows(logits, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0, offset: int = 0,
                offset_dev=None, row_params=None, index_offset: int = 0, return_logprob: bool = False):
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype in (_bf16, torch.float32)
    rows, V = logits.shape
    idx = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lp = torch.empty(rows, dtype=torch.float32, device=logits.device) if return_logprob else None
    rc = _lib.load().nfn_sample_rows(_p(logits), c_int(logits.dtype == torch.float32), c_longlong(logits.stride(0)), c_int(rows),
                                     c_int(V), _p(idx), _p(lp), c_float(temperature), c_int(top_k), c_float(top_p), _p(row_params),
                                     c_ulonglong(seed), c_ulonglong(offset), _p(offset_dev), c_int(index_offset), _st())
    _lib.check(rc, "nfn_sample_rows")
    return (idx, lp) if return_logprob else idx


class DecodeAttentionWorkspace:
    """Zero-initialised scratch for ``decode_attention`` (tickets + per-split partials)."""

    def __init__(self, B: int, n_q_heads: int, n_kv_heads: int, head_dim: int, device, max_splits: int = 64) -> None:
        n = _lib.load().nfn_decode_attention_workspace_bytes
        n.restype = c_longlong
        nbytes = n(c_int(B), c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(max_splits))
        if nbytes <= 0:
            raise ValueError("bad decode attention geometry")
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)


def decode_attention_set_impl(impl: str) -> str:
    """Selects the decode-attention kernel: ``"mma"`` (tensor-core, default) or ``"simt"``. Returns the previous one."""
    if impl not in ("mma", "simt"):
        raise ValueError("impl is 'mma' or 'simt'")
    old = _lib.load().nfn_decode_attention_set_impl(c_int(1 if impl == "mma" else 0))
    return "mma" if old else "simt"


def decode_attention(qkv, k_cache, v_cache, lengths, *, n_q_heads: int, n_kv_heads: int, head_dim: int, workspace: DecodeAttentionWorkspace,
                     cos=None, sin=None, convention="hf", qk_norm: bool = False, q_norm_weight=None, k_norm_weight=None,
                     eps: float = 1e-6, scale: float | None = None, splits: int = 0, out=None):
    """qkv bf16 [B, >= (Hq+2Hkv)*D]; caches bf16 [B, Hkv, cap, D]; lengths int32 [B] (counting
    the new token). Appends the new k/v and returns bf16 [B, Hq*D]."""
    B = qkv.shape[0]
    assert k_cache.dtype == _bf16 and k_cache.dim() == 4 and k_cache.shape == v_cache.shape and k_cache[0].is_contiguous()
    assert k_cache.stride(0) == v_cache.stride(0) and lengths.dtype == torch.int32
    cap = k_cache.shape[2]
    out = torch.empty(B, n_q_heads * head_dim, dtype=_bf16, device=qkv.device) if out is None else out
    scale = head_dim ** -0.5 if scale is None else scale
    rc = _lib.load().nfn_decode_attention(
        _p(qkv), c_int(qkv.stride(0)), _p(k_cache), _p(v_cache), c_longlong(k_cache.stride(0)), _p(lengths), _p(out), c_int(B),
        c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(cap), _p(q_norm_weight), _p(k_norm_weight), c_int(int(qk_norm)),
        c_float(eps), _p(cos), _p(sin), c_int(0 if cos is None else cos.shape[0]), c_float(_sign(convention) if cos is not None else 0.0),
        c_float(scale), _p(workspace.buf), c_longlong(workspace.buf.numel()), c_int(splits), _st())
    _lib.check(rc, "nfn_decode_attention")
    return out


class BlockAttentionWorkspace:
    """Zero-initialised scratch for ``block_attention`` (tickets + per-split partials)."""

    def __init__(self, B: int, rows: int, n_q_heads: int, n_kv_heads: int, head_dim: int, device, max_splits: int = 16) -> None:
        n = _lib.load().nfn_block_attention_workspace_bytes
        n.restype = c_longlong
        nbytes = n(c_int(B), c_int(rows), c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(max_splits))
        if nbytes <= 0:
            raise ValueError("bad block attention geometry")
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)


def block_attention(qkv, k_cache, v_cache, lengths, *, rows: int, n_q_heads: int, n_kv_heads: int, head_dim: int,
                    workspace: BlockAttentionWorkspace, window: int = 0, causal: bool = True, n_rows=None, stage_k=None, stage_v=None,
                    scale: float | None = None, splits: int = 0, out=None):
    """``rows`` new rows per sequence against the cached keys plus the block itself; the caches are
    not written. qkv bf16 [B*rows, >= (Hq+2Hkv)*D] (norm / rotary applied); caches bf16
    [B, Hkv, cap, D]; lengths int32 [B] = tokens already cached. Returns bf16 [B*rows, Hq*D]."""
    B = k_cache.shape[0]
    assert qkv.shape[0] == B * rows and k_cache.dtype == _bf16 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert lengths.dtype == torch.int32 and (n_rows is None or n_rows.dtype == torch.int32)
    cap = k_cache.shape[2]
    out = torch.empty(B * rows, n_q_heads * head_dim, dtype=_bf16, device=qkv.device) if out is None else out
    scale = head_dim ** -0.5 if scale is None else scale
    rc = _lib.load().nfn_block_attention(
        _p(qkv), c_int(qkv.stride(0)), _p(k_cache), _p(v_cache), _p(lengths), _p(n_rows), _p(out), c_int(out.stride(0)), _p(stage_k),
        _p(stage_v), c_int(B), c_int(rows), c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(cap), c_int(window),
        c_int(int(causal)), c_float(scale), _p(workspace.buf), c_longlong(workspace.buf.numel()), c_int(splits), _st())
    _lib.check(rc, "nfn_block_attention")
    return out


def kv_commit_layers(stage_k: list, stage_v: list, k_caches: list, v_caches: list, lengths, accepted, *, rows: int) -> None:
    """Appends the first ``accepted[b]`` staged rows of every layer to that layer's cache
    (ring rows ``position % cap``). One launch for all layers."""
    dev = lengths.device
    B, Hkv, _, D = k_caches[0].shape
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)  # noqa: E731
    caps = torch.tensor([t.shape[2] for t in k_caches], dtype=torch.int32, device=dev)
    sk, sv, kc, vc = ptrs(stage_k), ptrs(stage_v), ptrs(k_caches), ptrs(v_caches)
    rc = _lib.load().nfn_kv_commit_layers(_p(sk), _p(sv), _p(kc), _p(vc), _p(caps), _p(lengths), _p(accepted), c_int(len(k_caches)),
                                          c_int(B), c_int(rows), c_int(Hkv), c_int(D), _st())
    _lib.check(rc, "nfn_kv_commit_layers")
    torch.cuda.current_stream().synchronize()  # the pointer tables above must outlive the launch


def sigmoid_gate_inplace(att: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """att[r, :] *= sigmoid(gate[r, :]) (bf16 row views of equal width; row strides free)."""
    rc = _lib.load().nfn_sigmoid_gate_inplace(_p(att), c_int(att.stride(0)), _p(gate), c_int(gate.stride(0)), c_longlong(att.shape[0]),
                                              c_int(att.shape[1]), _st())
    _lib.check(rc, "nfn_sigmoid_gate_inplace")
    return att


def rmsnorm_residual(x: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor | None, *, eps: float, centered: bool = False, out=None):
    """out = resid + rms_norm(x) * weight (``(1 + weight)`` when centered); contiguous [rows, C] bf16. ``out`` may alias ``resid``."""
    out = torch.empty_like(x) if out is None else out
    rc = _lib.load().nfn_rmsnorm_residual(_p(x), _p(weight), _p(resid), _p(out), c_longlong(x.shape[0]), c_int(x.shape[1]), c_float(eps),
                                          c_int(int(centered)), _st())
    _lib.check(rc, "nfn_rmsnorm_residual")
    return out


def kv_cache_write(qkv: torch.Tensor, k_cache_slot: torch.Tensor, v_cache_slot: torch.Tensor, *, n_q_heads: int, n_kv_heads: int,
                   head_dim: int, pos0: int = 0) -> None:
    """Writes the k and v heads of ``qkv`` rows (one sequence, positions pos0 ...) into one slot's caches
    [Hkv, cap, D]; positions wrap modulo cap (ring caches of sliding-window layers)."""
    rc = _lib.load().nfn_kv_cache_write(_p(qkv), c_int(qkv.stride(0)), _p(k_cache_slot), _p(v_cache_slot), c_int(qkv.shape[0]),
                                        c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(k_cache_slot.shape[1]), c_int(pos0), _st())
    _lib.check(rc, "nfn_kv_cache_write")


def swiglu_forward(gate_up: torch.Tensor, inter: int, out=None) -> torch.Tensor:
    """gate_up bf16 [rows, 2 * inter] (gate | up) -> silu(gate) * up, bf16 [rows, inter]."""
    rows = gate_up.shape[0]
    out = torch.empty(rows, inter, dtype=_bf16, device=gate_up.device) if out is None else out
    rc = _lib.load().nfn_swiglu_forward(_p(gate_up), c_int(gate_up.stride(0)), _p(out), c_int(out.stride(0)), c_longlong(rows),
                                        c_int(inter), _st())
    _lib.check(rc, "nfn_swiglu_forward")
    return out


def swiglu_backward(gate_up: torch.Tensor, dout: torch.Tensor, inter: int, out=None) -> torch.Tensor:
    rows = gate_up.shape[0]
    out = torch.empty_like(gate_up) if out is None else out
    rc = _lib.load().nfn_swiglu_backward(_p(gate_up), c_int(gate_up.stride(0)), _p(dout), c_int(dout.stride(0)), _p(out),
                                         c_int(out.stride(0)), c_longlong(rows), c_int(inter), _st())
    _lib.check(rc, "nfn_swiglu_backward")
    return out


def quant_block_bytes(qtype: int) -> int:
    return int(_lib.load().nfn_quant_block_bytes(c_int(qtype)))


def dequant_kquant(qtype: int, blocks: torch.Tensor, out=None) -> torch.Tensor:
    """blocks: uint8 tensor holding whole super-blocks -> bf16 [n_blocks * 256]."""
    assert blocks.dtype == torch.uint8 and blocks.is_contiguous()
    nb = blocks.numel() // quant_block_bytes(qtype)
    out = torch.empty(nb * 256, dtype=_bf16, device=blocks.device) if out is None else out
    _lib.check(_lib.load().nfn_dequant_kquant(c_int(qtype), _p(blocks), c_longlong(nb), _p(out), _st()), "nfn_dequant_kquant")
    return out


def dequant_nf4(codes: torch.Tensor, absmax: torch.Tensor, group: int = 64, out=None) -> torch.Tensor:
    n = codes.numel() * 2
    out = torch.empty(n, dtype=_bf16, device=codes.device) if out is None else out
    _lib.check(_lib.load().nfn_dequant_nf4(_p(codes), _p(absmax), c_longlong(n), c_int(group), _p(out), _st()), "nfn_dequant_nf4")
    return out


def kquant_gemv(qtype: int, w: torch.Tensor, x: torch.Tensor, N: int, *, w_gate_pair: torch.Tensor | None = None, bias=None,
                resid=None, out=None) -> torch.Tensor:
    """y[b, n] = W[n] . x[b] for quantised W (uint8 [N * K/256 * block_bytes]); with
    ``w_gate_pair`` the result is silu(W x) * (W_pair x). x: bf16 [B <= 8, K]."""
    assert x.dtype == _bf16 and x.dim() == 2 and x.stride(1) == 1
    B, K = x.shape
    assert w.numel() == N * (K // 256) * quant_block_bytes(qtype), "weight size does not match N x K"
    out = torch.empty(B, N, dtype=_bf16, device=x.device) if out is None else out
    rc = _lib.load().nfn_kquant_gemv(c_int(qtype), _p(w), _p(w_gate_pair), _p(x), c_int(x.stride(0)), _p(out), c_int(out.stride(0)),
                                     _p(bias), _p(resid), c_int(0 if resid is None else resid.stride(0)), c_int(B), c_int(N), c_int(K), _st())
    _lib.check(rc, "nfn_kquant_gemv")
    return out


def gemm_kquant(qtype: int, x: torch.Tensor, w: torch.Tensor, N: int, *, bias=None, act: str | None = None, resid=None, out=None,
                alpha: float = 1.0) -> torch.Tensor:
    """Prefill product ``x @ dequant(W)^T`` with the dequantisation fused into the GEMM's operand
    pipeline. x: bf16 [M, K] (K a multiple of 256); w: uint8, N rows of K / 256 super-blocks."""
    from .gemm import ACT_IDS, EPI_ACT_SHIFT, EPI_BIAS, EPI_RESID
    assert x.dtype == _bf16 and x.dim() == 2 and x.stride(1) == 1
    M, K = x.shape
    assert w.numel() == N * (K // 256) * quant_block_bytes(qtype), "weight size does not match N x K"
    out = torch.empty(M, N, dtype=_bf16, device=x.device) if out is None else out
    a = _lib.GemmArgs()
    a.a, a.b, a.c = x.data_ptr(), w.data_ptr(), out.data_ptr()
    a.m, a.n, a.k = M, N, K
    a.lda, a.ldb, a.ldc = x.stride(0), K, out.stride(0)
    a.flags = ACT_IDS[act] << EPI_ACT_SHIFT
    a.alpha, a.split_k = alpha, 1
    if bias is not None:
        a.bias, a.flags = bias.data_ptr(), a.flags | EPI_BIAS
    if resid is not None:
        a.aux_in, a.ld_aux_in, a.flags = resid.data_ptr(), resid.stride(0), a.flags | EPI_RESID
    import ctypes
    rc = _lib.load().nfn_gemm_kquant(c_int(qtype), ctypes.byref(a), _st())
    _lib.check(rc, "nfn_gemm_kquant")
    return out


QTYPE_NF4 = 100


class NF4LoRALinear:
    """A frozen NF4 base weight [N, K] (codes + per-64 absmax) with a trainable rank-r adapter:
    ``y = x W^T + (alpha / r) * (x A^T) B^T``. Forward is one tiny GEMM (x A^T, 64 padded columns)
    plus ONE fused launch that decodes the NF4 tiles inside the GEMM pipeline and accumulates the
    adapter as an extra k-block. Backward returns dX, dA, dB; the base weight is decoded to a
    transient bf16 matrix for dX = dY W (the decode-in-pipeline kernel covers K-major products only).

    Reference counterparts: ``tile_ops.h:19-27``, ``muse_glimmer_native_train.cpp:3324-3419``,
    ``torch_backend.py:990-1097``."""

    def __init__(self, codes: torch.Tensor, absmax: torch.Tensor, N: int, K: int, lora_a: torch.Tensor, lora_b: torch.Tensor, alpha: float = 16.0):
        r = lora_a.shape[0]
        assert codes.dtype == torch.uint8 and codes.numel() == N * K // 2 and absmax.numel() == N * K // 64 and absmax.dtype == torch.float32
        assert lora_a.shape == (r, K) and lora_b.shape == (N, r) and r <= 64 and K % 64 == 0 and N % 8 == 0
        self.codes, self.absmax, self.N, self.K, self.r, self.scale = codes, absmax, N, K, r, alpha / r
        self.a, self.b = lora_a, lora_b
        dev = codes.device
        self._a_pad = torch.zeros(64, K, dtype=_bf16, device=dev)
        self._b_pad = torch.zeros(N, 64, dtype=_bf16, device=dev)
        self.refresh_adapter()

    def refresh_adapter(self) -> None:
        """Call after an optimizer step on ``a`` / ``b``."""
        self._a_pad[:self.r].copy_(self.a)
        self._b_pad[:, :self.r].copy_(self.b)

    def forward(self, x: torch.Tensor, bias=None, out=None) -> torch.Tensor:
        import ctypes

        from .gemm import EPI_BIAS, gemm
        assert x.dtype == _bf16 and x.dim() == 2 and x.shape[1] == self.K and x.stride(1) == 1
        M = x.shape[0]
        t = gemm(x, self._a_pad, alpha=self.scale)  # [M, 64]: scale * x A^T, zero beyond column r
        out = torch.empty(M, self.N, dtype=_bf16, device=x.device) if out is None else out
        a = _lib.GemmArgs()
        a.a, a.b, a.c = x.data_ptr(), self.codes.data_ptr(), out.data_ptr()
        a.m, a.n, a.k = M, self.N, self.K
        a.lda, a.ldb, a.ldc = x.stride(0), self.K, out.stride(0)
        a.alpha, a.split_k, a.flags = 1.0, 1, 0
        if bias is not None:
            a.bias, a.flags = bias.data_ptr(), EPI_BIAS
        rc = _lib.load().nfn_gemm_quant_lora(c_int(QTYPE_NF4), ctypes.byref(a), _p(self.absmax), _p(t), c_int(t.stride(0)), _p(self._b_pad),
                                             c_int(self._b_pad.stride(0)), _st())
        _lib.check(rc, "nfn_gemm_quant_lora")
        self._saved_t = t
        return out

    def backward(self, x: torch.Tensor, dy: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(dX bf16 [M, K], dA fp32 [r, K], dB fp32 [N, r]) for the last forward's input ``x``."""
        from .gemm import gemm
        w = dequant_nf4(self.codes, self.absmax).view(self.N, self.K)
        u = gemm(dy, self._b_pad, b_mn=True, alpha=self.scale)       # [M, 64] = scale * dY B
        dx = gemm(dy, w, b_mn=True)                                   # dY W
        dx = gemm(u, self._a_pad, b_mn=True, resid=dx)                # + u A
        da = gemm(u, x, a_mn=True, b_mn=True, out_dtype=torch.float32)[:self.r]        # u^T x
        db = gemm(dy, self._saved_t, a_mn=True, b_mn=True, out_dtype=torch.float32)[:, :self.r]  # dY^T (scale x A^T)
        return dx, da, db
