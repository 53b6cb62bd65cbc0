"""Kernel registry and coverage report: which operations have a native sm_100a kernel in this
library, under which exported symbol, for which dtypes, and what each falls back to.

``KERNELS`` is the catalogue; ``coverage_report()`` checks every entry against the loaded
library (symbol present or not) and returns one row per operation with a status:
``native`` (hand-written kernel, symbol found), ``missing`` (catalogued but the library on disk
lacks the symbol - a stale build), or ``torch`` (no kernel; the tensor runtime uses PyTorch).

Behavioural counterpart: the reference's kernel registry and coverage report
(``neuralfn/tile_cuda/registry.py:43-175, 922-946``; statuses tile / torch_fallback /
host_only / delegated / planned and its dtype matrix).
"""
from __future__ import annotations

from dataclasses import dataclass

__all__ = ["KernelEntry", "KERNELS", "coverage_report", "coverage_summary"]


@dataclass(frozen=True)
class KernelEntry:
    op: str
    symbol: str | None          # exported C symbol; None = no native kernel
    dtypes: tuple[str, ...]
    tensor_core: bool = False   # issues tcgen05.mma
    fused: str = ""             # what the kernel folds in
    fallback: str = "torch"


def _k(op, symbol, dtypes=("bf16",), tc=False, fused="", fallback="torch") -> KernelEntry:
    return KernelEntry(op, symbol, tuple(dtypes), tc, fused, fallback)


KERNELS: tuple[KernelEntry, ...] = (
    _k("gemm", "nfn_gemm_bf16", ("bf16", "fp32-out"), True, "bias, GELU/SiLU/ReLU^2/tanh-cap, residual, dGELU, accumulate, split-K"),
    _k("gemm, grouped contraction (expert weight gradients)", "nfn_gemm_grouped_k", ("bf16", "fp32-out"), True, "per-group K ranges read on the device, accumulate"),
    _k("gemm_kquant", "nfn_gemm_kquant", ("q4_k", "q5_k", "q6_k"), True, "dequantisation inside the operand pipeline + GEMM epilogues"),
    _k("gemm_nf4_lora", "nfn_gemm_quant_lora", ("nf4",), True, "NF4 decode + LoRA branch as an extra k-block"),
    _k("gemm_allgather / reduce_scatter / grouped", "nfn_gemm_tp", ("bf16",), True, "peer-memory all-gather or reduce-scatter inside the GEMM; grouped MoE GEMM"),
    _k("attention_forward", "nfn_attention_forward", ("bf16",), True, "causal / window / GQA, log-sum-exp"),
    _k("attention_backward", "nfn_attention_backward", ("bf16",), True, "dQ dK dV, delta pre-pass"),
    _k("block_attention", "nfn_block_attention", ("bf16",), True, "cache prefix + block, staging of block K/V, split-KV merge"),
    _k("decode_attention", "nfn_decode_attention", ("bf16",), False, "QK-norm, RoPE, cache append, split-KV merge"),
    _k("turboquant_attention", "nfn_turboquant_attention", ("tq-3.5",), False, "attention on compressed records"),
    _k("turboquant_encode", "nfn_turboquant_encode", ("tq-3.5",)),
    _k("kv_commit", "nfn_kv_commit_layers"), _k("kv_cache_write", "nfn_kv_cache_write"),
    _k("layernorm / rmsnorm forward", "nfn_norm_forward", ("bf16",), False, "centred scale"),
    _k("norm backward dx", "nfn_norm_backward_dx"), _k("norm backward dw db", "nfn_norm_backward_wb"),
    _k("rmsnorm + residual", "nfn_rmsnorm_residual"), _k("qk_norm", "nfn_qk_norm_forward"), _k("qk_norm backward", "nfn_qk_norm_backward"),
    _k("rope", "nfn_rope_inplace"), _k("qk_norm + rope", "nfn_qk_norm_rope_forward"),
    _k("cross_entropy", "nfn_cross_entropy", ("bf16",), False, "soft-cap derivative, z-loss, in-place gradient"),
    _k("embedding forward", "nfn_embedding_forward"), _k("embedding backward", "nfn_embedding_backward"), _k("embedding backward, sorted tokens (deterministic)", "nfn_embedding_backward_sorted"),
    _k("embedding + positions", "nfn_embedding_positions"), _k("swiglu", "nfn_swiglu_forward"), _k("swiglu backward", "nfn_swiglu_backward"),
    _k("dropout (counter-based, adapter branch)", "nfn_dropout_apply"), _k("sigmoid gate", "nfn_sigmoid_gate_inplace"), _k("bias gradient (column sum)", "nfn_colsum"),
    _k("adamw (flat, clip on device)", "nfn_adamw_flat", ("fp32 master", "bf16 params")), _k("grad clip scale", "nfn_grad_clip_scale"),
    _k("grad accumulate", "nfn_grad_accumulate"),
    _k("dp reduce + sharded adamw + all-gather", "nfn_dp_adamw", ("bf16", "fp32"), False, "peer loads, owner update, parameter push"),
    _k("all-reduce + residual + rmsnorm", "nfn_allreduce_resid_norm", ("bf16",), False, "peer loads or multimem.ld_reduce"),
    _k("argmax", "nfn_argmax_rows"), _k("sampling (top-k / top-p / Gumbel)", "nfn_sample_rows"),
    _k("dequant k-quant", "nfn_dequant_kquant", ("q4_k", "q5_k", "q6_k")), _k("dequant nf4", "nfn_dequant_nf4", ("nf4",)),
    _k("quantised gemv", "nfn_kquant_gemv", ("q4_k", "q5_k", "q6_k"), False, "SwiGLU pair, bias, residual"),
    _k("moe route / plan / permute / combine", "nfn_moe_route"), _k("moe expert-parallel pull", "nfn_moe_ep_pull"),
    # operations the tensor runtime still runs through PyTorch
    _k("conv / pooling stages", None), _k("ssm scan (mamba stages)", None), _k("diffusion noise schedule", None),
    _k("fp8 / nvfp4 / mxfp4 linear", None, ("fp8", "fp4")),
)


def coverage_report() -> list[dict]:
    from . import _lib
    lib = _lib.load() if _lib.available() else None
    rows = []
    for k in KERNELS:
        if k.symbol is None:
            status = "torch"
        elif lib is None:
            status = "unbuilt"
        else:
            status = "native" if hasattr(lib, k.symbol) else "missing"
        rows.append({"op": k.op, "symbol": k.symbol, "status": status, "dtypes": list(k.dtypes), "tensor_core": k.tensor_core,
                     "fused": k.fused, "fallback": k.fallback})
    return rows


def coverage_summary() -> dict:
    rows = coverage_report()
    out: dict = {"total": len(rows)}
    for r in rows:
        out[r["status"]] = out.get(r["status"], 0) + 1
    out["tensor_core_kernels"] = sum(1 for r in rows if r["tensor_core"] and r["status"] == "native")
    return out
