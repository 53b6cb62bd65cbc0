"""Python front-ends of the non-GEMM kernels in ``libnfn_b200_kernels.so``.

All functions take CUDA tensors, launch on the current stream and return/modify
tensors; none of them synchronises. Argument checking lives here (shape, dtype,
contiguity) so the C side only sees validated raw pointers.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p, c_int, c_float, c_longlong, c_double

import torch

from . import _lib

_bf16 = torch.bfloat16


def _p(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _st() -> c_void_p:
    return c_void_p(_lib.stream_ptr())


def _need(t: torch.Tensor, dtype, name: str) -> None:
    if t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"{name}: expected contiguous {dtype}, got {t.dtype} stride={t.stride()}")


# --------------------------------------------------------------------- norms --
NORM_LAYER, NORM_RMS = 0, 1


def norm_forward(x, weight, bias, *, eps: float, mode: int, centered: bool = False,
                 out=None, mean=None, rstd=None):
    """x: bf16 [rows, C]. Returns (y, mean, rstd); stats are fp32 [rows]."""
    _need(x, _bf16, "x")
    rows, C = x.shape
    y = torch.empty_like(x) if out is None else out
    if mean is None and mode == NORM_LAYER:
        mean = torch.empty(rows, device=x.device, dtype=torch.float32)
    if rstd is None:
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
    rc = _lib.load().nfn_norm_forward(_p(x), _p(weight), _p(bias), _p(y), _p(mean), _p(rstd),
                                      c_int(rows), c_int(C), c_float(eps), c_int(mode),
                                      c_int(int(centered)), _st())
    _lib.check(rc, "nfn_norm_forward")
    return y, mean, rstd


def norm_backward_dx(dy, x, weight, mean, rstd, *, mode: int, centered: bool = False,
                     dresid=None, out=None):
    _need(dy, _bf16, "dy")
    _need(x, _bf16, "x")
    rows, C = x.shape
    dx = torch.empty_like(x) if out is None else out
    rc = _lib.load().nfn_norm_backward_dx(_p(dy), _p(x), _p(weight), _p(mean), _p(rstd), _p(dresid),
                                          _p(dx), c_int(rows), c_int(C), c_int(mode),
                                          c_int(int(centered)), _st())
    _lib.check(rc, "nfn_norm_backward_dx")
    return dx


def norm_backward_wb(dy, x, mean, rstd, dweight, dbias, scratch, *, mode: int, accumulate: bool = False):
    """dweight/dbias: bf16 [C] (either may be None). scratch: fp32 >= 64*2*C."""
    rows, C = x.shape
    if scratch.numel() < 64 * 2 * C:
        raise ValueError("norm_backward_wb: scratch too small")
    rc = _lib.load().nfn_norm_backward_wb(_p(dy), _p(x), _p(mean), _p(rstd), _p(dweight), _p(dbias),
                                          _p(scratch), c_int(rows), c_int(C), c_int(mode),
                                          c_int(int(accumulate)), _st())
    _lib.check(rc, "nfn_norm_backward_wb")


def norm_fused_rows() -> int:
    return int(_lib.load().nfn_norm_fused_rows())


def norm_backward(dy, x, weight, mean, rstd, dweight, dbias, scratch, *, mode: int, centered: bool = False, dresid=None, out=None,
                  accumulate: bool = False, dx_colsum=None):
    """dx (returned), dweight and dbias (bf16 [C], either may be None) in one pass over dy and x.
    ``dx_colsum`` (bf16 [C], optional) receives the column sum of dx: the bias gradient of the
    linear layer whose output is the residual stream this norm reads.
    scratch: fp32 with at least ``norm_fused_rows() * 3 * C`` entries."""
    _need(dy, _bf16, "dy")
    _need(x, _bf16, "x")
    rows, C = x.shape
    if scratch.numel() < norm_fused_rows() * 3 * C:
        raise ValueError("norm_backward: scratch too small")
    dx = torch.empty_like(x) if out is None else out
    rc = _lib.load().nfn_norm_backward_ex(_p(dy), _p(x), _p(weight), _p(mean), _p(rstd), _p(dresid), _p(dx), _p(dweight), _p(dbias),
                                          _p(dx_colsum), _p(scratch), c_int(rows), c_int(C), c_int(mode), c_int(int(centered)),
                                          c_int(int(accumulate)), _st())
    _lib.check(rc, "nfn_norm_backward_ex")
    return dx


def colsum(dy, out, scratch, *, accumulate: bool = False):
    """out[c] = sum_r dy[r, c]; dy bf16 [rows, C] (row stride allowed), out bf16 [C]."""
    rows, C = dy.shape
    if dy.stride(1) != 1 or scratch.numel() < 64 * C:
        raise ValueError("colsum: bad operands")
    rc = _lib.load().nfn_colsum(_p(dy), c_int(dy.stride(0)), _p(out), _p(scratch), c_int(rows),
                                c_int(C), c_int(int(accumulate)), _st())
    _lib.check(rc, "nfn_colsum")
    return out


def qk_norm_forward(qkv, n_q_heads: int, n_kv_heads: int, head_dim: int, *, eps: float = 1e-6,
                    q_scale: float = 1.0, rstd=None):
    """In place on the q and k head groups of packed ``qkv`` rows (q | k | v)."""
    tokens, ld = qkv.shape
    if rstd is None:
        rstd = torch.empty(tokens, n_q_heads + n_kv_heads, device=qkv.device, dtype=torch.float32)
    rc = _lib.load().nfn_qk_norm_forward(_p(qkv), _p(rstd), c_int(tokens), c_int(n_q_heads),
                                         c_int(n_kv_heads), c_int(head_dim), c_int(qkv.stride(0)),
                                         c_float(eps), c_float(q_scale), _st())
    _lib.check(rc, "nfn_qk_norm_forward")
    return rstd


def qk_norm_backward(dqkv, qkv_normed, rstd, n_q_heads: int, n_kv_heads: int, head_dim: int, *,
                     q_scale: float = 1.0):
    tokens = dqkv.shape[0]
    rc = _lib.load().nfn_qk_norm_backward(_p(dqkv), _p(qkv_normed), _p(rstd), c_int(tokens),
                                          c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim),
                                          c_int(dqkv.stride(0)), c_float(q_scale), _st())
    _lib.check(rc, "nfn_qk_norm_backward")


# ----------------------------------------------------------------- dropout --
def dropout_apply(x, out, p: float, *, seed: int, stream_id: int, step=None, accumulate: bool = False):
    """out (+)= mask * x / (1 - p); the mask is a function of (seed, stream_id, step[0], row, column) and is never stored: the same
    call reproduces it. x / out bf16 [rows, width] views with free row strides; ``step`` an int64 device tensor or None."""
    from ctypes import c_ulonglong
    rc = _lib.load().nfn_dropout_apply(_p(x), c_int(x.stride(0)), _p(out), c_int(out.stride(0)), c_longlong(x.shape[0]), c_int(x.shape[1]),
                                       c_float(float(p)), c_ulonglong(int(seed) & (2**64 - 1)), c_int(int(stream_id)), _p(step),
                                       c_int(int(accumulate)), _st())
    _lib.check(rc, "nfn_dropout_apply")
    return out


# ------------------------------------------------------------ gated attention --
def sigmoid_gate_forward(att, gate, out):
    """out = att * sigmoid(gate); bf16 [rows, width] views with free row strides."""
    rc = _lib.load().nfn_sigmoid_gate_forward(_p(att), c_int(att.stride(0)), _p(gate), c_int(gate.stride(0)), _p(out), c_int(out.stride(0)),
                                              c_longlong(att.shape[0]), c_int(att.shape[1]), _st())
    _lib.check(rc, "nfn_sigmoid_gate_forward")
    return out


def sigmoid_gate_backward(dout, att, gate, datt, dgate):
    """d(att) = dout * sigmoid(gate); d(gate) = dout * att * sigmoid'(gate)."""
    rc = _lib.load().nfn_sigmoid_gate_backward(_p(dout), c_int(dout.stride(0)), _p(att), c_int(att.stride(0)), _p(gate), c_int(gate.stride(0)),
                                               _p(datt), c_int(datt.stride(0)), _p(dgate), c_int(dgate.stride(0)),
                                               c_longlong(att.shape[0]), c_int(att.shape[1]), _st())
    _lib.check(rc, "nfn_sigmoid_gate_backward")


# ---------------------------------------------------- differential attention glue --
def diff_partials() -> int:
    return int(_lib.load().nfn_diff_partials())


def diff_q_expand(q, q2, n_heads: int, head_dim: int):
    """q: bf16 [tokens, >= H*D] view -> q2 [tokens, 2*H*D]: pseudo-head 2h keeps the first half of head h, 2h+1 the second."""
    rc = _lib.load().nfn_diff_q_expand(_p(q), c_int(q.stride(0)), _p(q2), c_longlong(q.shape[0]), c_int(n_heads), c_int(head_dim), _st())
    _lib.check(rc, "nfn_diff_q_expand")


def diff_q_collapse(dq2, dq, n_heads: int, head_dim: int):
    rc = _lib.load().nfn_diff_q_collapse(_p(dq2), _p(dq), c_int(dq.stride(0)), c_longlong(dq.shape[0]), c_int(n_heads), c_int(head_dim), _st())
    _lib.check(rc, "nfn_diff_q_collapse")


def diff_combine(a, lam, out_scale: float, eps: float, out, rstd, n_heads: int, head_dim: int):
    """out = rms_norm(a1 - lambda * a2) * out_scale over each head; a: [tokens, 2*H*D], lam: bf16 (element 0)."""
    rc = _lib.load().nfn_diff_combine(_p(a), _p(lam), c_float(out_scale), c_float(eps), _p(out), _p(rstd), c_longlong(a.shape[0]),
                                      c_int(n_heads), c_int(head_dim), _st())
    _lib.check(rc, "nfn_diff_combine")


def diff_combine_backward(dout, a, lam, out_scale: float, rstd, da, partial, dlam, n_heads: int, head_dim: int):
    rc = _lib.load().nfn_diff_combine_backward(_p(dout), _p(a), _p(lam), c_float(out_scale), _p(rstd), _p(da), _p(partial), _p(dlam),
                                               c_longlong(a.shape[0]), c_int(n_heads), c_int(head_dim), _st())
    _lib.check(rc, "nfn_diff_combine_backward")


# ----------------------------------------------------------------- attention --
class AttentionArgs(ctypes.Structure):
    """Mirror of ``nfn_attention_args`` (csrc/kernels/nfn_kernels.h)."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("o", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("B", c_int), ("T", c_int), ("Hq", c_int), ("Hkv", c_int), ("D", c_int),
        ("ld_q", c_int), ("ld_k", c_int), ("ld_v", c_int), ("ld_o", c_int),
        ("causal", c_int), ("window", c_int),
        ("scale", c_float), ("softcap", c_float),
        ("seq_ids", ctypes.c_void_p),
        ("gate", ctypes.c_void_p), ("ld_gate", c_int),
        ("d_o", ctypes.c_void_p), ("ld_do", c_int),
        ("delta", ctypes.c_void_p),
        ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p),
        ("ld_dq", c_int), ("ld_dk", c_int), ("ld_dv", c_int),
    ]


def _ptr(t):
    return None if t is None else t.data_ptr()


def _attention_args(q, k, v, o, lse, B, T, n_q_heads, n_kv_heads, head_dim, causal, window, scale, softcap, seq_ids, gate):
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dtype != _bf16 or t.stride(1) != 1 or t.shape[0] != B * T:
            raise ValueError(f"attention: bad {name}")
    if seq_ids is not None and (seq_ids.dtype != torch.int32 or seq_ids.numel() != B * T or not seq_ids.is_contiguous()):
        raise ValueError("attention: seq_ids must be contiguous int32 [B*T]")
    if gate is not None and (gate.dtype != _bf16 or gate.stride(1) != 1 or gate.shape[0] != B * T):
        raise ValueError("attention: bad gate")
    a = AttentionArgs()
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(o), _ptr(lse)
    a.B, a.T, a.Hq, a.Hkv, a.D = B, T, n_q_heads, n_kv_heads, head_dim
    a.ld_q, a.ld_k, a.ld_v, a.ld_o = q.stride(0), k.stride(0), v.stride(0), (o.stride(0) if o is not None else 0)
    a.causal, a.window = int(causal), int(window)
    a.scale, a.softcap = float(head_dim ** -0.5 if scale is None else scale), float(softcap)
    a.seq_ids = _ptr(seq_ids)
    a.gate, a.ld_gate = _ptr(gate), (gate.stride(0) if gate is not None else 0)
    return a


def attention_forward(q, k, v, *, B: int, T: int, n_q_heads: int, n_kv_heads: int, head_dim: int,
                      causal: bool = True, window: int = 0, scale: float | None = None,
                      softcap: float = 0.0, seq_ids=None, gate=None, out=None, lse=None, need_lse: bool = True):
    """q: bf16 [B*T, >= Hq*D] view (row stride free), k/v: [B*T, >= Hkv*D] views.
    ``seq_ids`` (int32 [B*T]): packed sequences, a key is visible only inside the query's own
    sequence. ``softcap`` c > 0: scores become c * tanh(s * scale / c). ``gate`` (bf16 [B*T, Hq*D]):
    the output is multiplied by sigmoid(gate). Returns (o [B*T, Hq*D], lse [B, Hq, T])."""
    o = torch.empty(B * T, n_q_heads * head_dim, device=q.device, dtype=_bf16) if out is None else out
    if lse is None and need_lse:
        lse = torch.empty(B, n_q_heads, T, device=q.device, dtype=torch.float32)
    a = _attention_args(q, k, v, o, lse, B, T, n_q_heads, n_kv_heads, head_dim, causal, window, scale, softcap, seq_ids, gate)
    rc = _lib.load().nfn_attention_forward_ex(ctypes.byref(a), _st())
    _lib.check(rc, "nfn_attention_forward_ex")
    return o, lse


def attention_backward(do, q, k, v, o, lse, *, B: int, T: int, n_q_heads: int, n_kv_heads: int,
                       head_dim: int, causal: bool = True, window: int = 0, scale: float | None = None,
                       softcap: float = 0.0, seq_ids=None, dq, dk, dv, delta=None, dq_accum=None):
    """Gradients of attention (of the ungated output). dq/dk/dv are bf16 [B*T, *] views (row
    stride free). ``delta``: fp32 [B, Hq, T] scratch. ``dq_accum`` (fp32 [B*T, Hq*D]) is only
    needed by the first-generation kernels (``nfn_attention_set_impl(1)``)."""
    if delta is None:
        delta = torch.empty(B, n_q_heads, T, device=q.device, dtype=torch.float32)
    lib = _lib.load()
    if dq_accum is not None and softcap == 0.0 and seq_ids is None:
        # same call for both kernel generations: the library picks by nfn_attention_set_impl
        sc = head_dim ** -0.5 if scale is None else scale
        rc = lib.nfn_attention_backward(
            _p(do), _p(q), _p(k), _p(v), _p(o), _p(lse), _p(delta), _p(dq_accum), _p(dq), _p(dk), _p(dv),
            c_int(B), c_int(T), c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim),
            c_int(do.stride(0)), c_int(q.stride(0)), c_int(k.stride(0)), c_int(v.stride(0)),
            c_int(o.stride(0)), c_int(dq.stride(0)), c_int(dk.stride(0)), c_int(dv.stride(0)),
            c_int(int(causal)), c_int(window), c_float(sc), _st())
        _lib.check(rc, "nfn_attention_backward")
        return dq, dk, dv
    a = _attention_args(q, k, v, o, lse, B, T, n_q_heads, n_kv_heads, head_dim, causal, window, scale, softcap, seq_ids, None)
    a.d_o, a.ld_do, a.delta = do.data_ptr(), do.stride(0), delta.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.ld_dq, a.ld_dk, a.ld_dv = dq.stride(0), dk.stride(0), dv.stride(0)
    rc = lib.nfn_attention_backward_ex(ctypes.byref(a), _st())
    _lib.check(rc, "nfn_attention_backward_ex")
    return dq, dk, dv


# ---------------------------------------------------------------------- loss --
def cross_entropy(logits, targets, *, vocab: int, cap: float = 0.0, z_coef: float = 0.0,
                  grad_scale: float = 1.0, loss_scale: float = 1.0, row_scale=None,
                  write_grad: bool = True, row_loss=None, row_lse=None, mean_loss=None):
    """logits: bf16 [rows, ld] (soft-capped already when cap > 0); overwritten with
    d(loss)/d(logits) * grad_scale when ``write_grad``. targets: int32 [rows]."""
    _need(logits, _bf16, "logits")
    _need(targets, torch.int32, "targets")
    rows, ld = logits.shape
    dev = logits.device
    if row_loss is None:
        row_loss = torch.empty(rows, device=dev, dtype=torch.float32)
    if mean_loss is None:
        mean_loss = torch.empty(1, device=dev, dtype=torch.float32)
    rc = _lib.load().nfn_cross_entropy(_p(logits), _p(targets), _p(row_scale), _p(row_loss), _p(row_lse),
                                       _p(mean_loss), c_int(rows), c_int(vocab), c_int(ld), c_float(cap),
                                       c_float(z_coef), c_float(grad_scale), c_float(loss_scale),
                                       c_int(int(write_grad)), _st())
    _lib.check(rc, "nfn_cross_entropy")
    return mean_loss, row_loss


# ----------------------------------------------------------------- embedding --
def embedding_forward(tokens, wte, wpe, *, T: int, out=None):
    _need(tokens, torch.int32, "tokens")
    n = tokens.numel()
    vocab, C = wte.shape
    out = torch.empty(n, C, device=wte.device, dtype=_bf16) if out is None else out
    rc = _lib.load().nfn_embedding_forward(_p(tokens), _p(wte), _p(wpe), _p(out), c_int(n), c_int(T),
                                           c_int(C), c_int(vocab), _st())
    _lib.check(rc, "nfn_embedding_forward")
    return out


def sort_tokens(tokens, sorted_out=None, order_out=None):
    """Stable sort of a batch's token ids: (ids ascending [int32], row each came from [int64]). Equal tokens keep their row order,
    which is what makes ``embedding_backward`` sum them in the same order on every run. With the two output buffers nothing the
    caller keeps is allocated (safe inside a captured graph)."""
    flat = tokens.reshape(-1)
    if sorted_out is None:
        return torch.sort(flat, stable=True)
    torch.sort(flat, stable=True, out=(sorted_out, order_out))
    return sorted_out, order_out


def embedding_backward(dout, tokens, dwte, dwpe, *, B: int, T: int, accumulate_wpe: bool = False, sorted_tokens=None, order=None):
    """Adds the token-embedding gradient onto ``dwte`` (and writes ``dwpe``). With ``sorted_tokens`` / ``order`` (``sort_tokens`` of the
    batch, e.g. prepared when the batch was uploaded) rows of equal tokens are summed in row order by one block each: bitwise
    reproducible. Without them the sort happens here."""
    C = dout.shape[1]
    vocab = dwte.shape[0] if dwte is not None else 0
    L = _lib.load()
    if dwpe is not None:
        rc = L.nfn_embedding_backward(_p(dout), _p(tokens), _p(None), _p(dwpe), c_int(B), c_int(T), c_int(C), c_int(vocab),
                                      c_int(int(accumulate_wpe)), _st())
        _lib.check(rc, "nfn_embedding_backward")
    if dwte is not None:
        if sorted_tokens is None or order is None:
            sorted_tokens, order = sort_tokens(tokens)
        rc = L.nfn_embedding_backward_sorted(_p(dout), _p(sorted_tokens), _p(order), _p(dwte), c_int(B * T), c_int(C), c_int(vocab), _st())
        _lib.check(rc, "nfn_embedding_backward_sorted")


# ----------------------------------------------------------------- optimizer --
HP_LR, HP_BETA1, HP_BETA2, HP_EPS, HP_WD, HP_BC1, HP_BC2, HP_GRAD_SCALE, HP_MAX_NORM = range(9)
HYPER_SIZE = 16


def optim_max_partials() -> int:
    return int(_lib.load().nfn_optim_max_partials())


def grad_clip_scale(grad, partial, hyper, clip):
    rc = _lib.load().nfn_grad_clip_scale(_p(grad), c_longlong(grad.numel()), _p(partial), _p(hyper),
                                         _p(clip), _st())
    _lib.check(rc, "nfn_grad_clip_scale")


def adamw_flat(master, m, v, grad, param, n_decay: int, hyper, clip):
    rc = _lib.load().nfn_adamw_flat(_p(master), _p(m), _p(v), _p(grad), _p(param),
                                    c_longlong(master.numel()), c_longlong(n_decay), _p(hyper),
                                    _p(clip), _st())
    _lib.check(rc, "nfn_adamw_flat")


def _ptr_array(ptrs):
    arr = (c_void_p * len(ptrs))(*[c_void_p(int(p)) for p in ptrs])
    return arr


def counter_add(counter, value: int = 1):
    """counter (int32 device tensor)[0] += value, on the stream."""
    rc = _lib.load().nfn_counter_add(_p(counter), c_int(value), _st())
    _lib.check(rc, "nfn_counter_add")


def peer_arrive(peer_flag_ptrs, rank: int, world: int, slot: int, epoch: int, epoch_dev=None):
    rc = _lib.load().nfn_peer_arrive(_ptr_array(peer_flag_ptrs), c_int(rank), c_int(world), c_int(slot),
                                     c_int(epoch), _p(epoch_dev), _st())
    _lib.check(rc, "nfn_peer_arrive")


def peer_wait(my_flags_ptr: int, world: int, slot: int, epoch: int, timeout_s: float = 2.0, epoch_dev=None):
    rc = _lib.load().nfn_peer_wait(c_void_p(my_flags_ptr), c_int(world), c_int(slot), c_int(epoch),
                                   _p(epoch_dev), c_double(timeout_s), _st())
    _lib.check(rc, "nfn_peer_wait")


def dp_reduce(peer_grad_ptrs, rank: int, world: int, lo: int, n: int, gshard, partial):
    rc = _lib.load().nfn_dp_reduce(_ptr_array(peer_grad_ptrs), c_int(rank), c_int(world), c_longlong(lo),
                                   c_longlong(n), _p(gshard), _p(partial), _st())
    _lib.check(rc, "nfn_dp_reduce")


def dp_relay_blocks() -> int:
    return int(_lib.load().nfn_dp_relay_blocks())


def dp_reduce_relay(peer_grad_ptrs, peer_gshard_ptrs, rank: int, world: int, lo: int, n: int, shard: int, partial,
                    accumulate: bool, background: bool = False):
    """Bucketed reduce of flat elements [lo, lo + n): this rank sums its 1/world slice of the bucket
    over all peers and stores the fp32 sums into the owners' reduced-gradient shards."""
    rc = _lib.load().nfn_dp_reduce_relay(_ptr_array(peer_grad_ptrs), _ptr_array(peer_gshard_ptrs), c_int(rank), c_int(world),
                                         c_longlong(lo), c_longlong(n), c_longlong(shard), _p(partial),
                                         c_int(int(accumulate)), c_int(int(background)), _st())
    _lib.check(rc, "nfn_dp_reduce_relay")


def dp_norm_publish_n(partial, npartial: int, peer_slot_ptrs, rank: int, world: int, epoch: int, epoch_dev=None):
    rc = _lib.load().nfn_dp_norm_publish_n(_p(partial), c_int(npartial), _ptr_array(peer_slot_ptrs),
                                           c_int(rank), c_int(world), c_int(epoch), _p(epoch_dev), _st())
    _lib.check(rc, "nfn_dp_norm_publish_n")


def dp_norm_publish(partial, shard_n: int, peer_slot_ptrs, rank: int, world: int, epoch: int, epoch_dev=None):
    rc = _lib.load().nfn_dp_norm_publish(_p(partial), c_longlong(shard_n), _ptr_array(peer_slot_ptrs),
                                         c_int(rank), c_int(world), c_int(epoch), _p(epoch_dev), _st())
    _lib.check(rc, "nfn_dp_norm_publish")


def dp_norm_collect(my_slots_ptr: int, world: int, epoch: int, hyper, clip, timeout_s: float = 2.0,
                    epoch_dev=None):
    rc = _lib.load().nfn_dp_norm_collect(c_void_p(my_slots_ptr), c_int(world), c_int(epoch), _p(epoch_dev),
                                         _p(hyper), _p(clip), c_double(timeout_s), _st())
    _lib.check(rc, "nfn_dp_norm_collect")


def dp_adamw(master, m, v, gshard, peer_param_ptrs, rank: int, world: int, lo: int, n: int,
             n_decay_global: int, hyper, clip):
    rc = _lib.load().nfn_dp_adamw(_p(master), _p(m), _p(v), _p(gshard), _ptr_array(peer_param_ptrs),
                                  c_int(rank), c_int(world), c_longlong(lo), c_longlong(n),
                                  c_longlong(n_decay_global), _p(hyper), _p(clip), _st())
    _lib.check(rc, "nfn_dp_adamw")
