"""Python API of the resident inference engine (``csrc/engine``): weights, KV caches and
activations stay on the GPU; Python passes token ids in and gets token ids back.

    eng = ResidentEngine(EngineConfig.gpt2(cfg, max_batch=8))
    eng.load_dense_checkpoint("model_00001000.bin")      # or eng.load_named_tensors(...)
    out = eng.generate([[15496, 11], [40]], max_new_tokens=32, sampling=Sampling(temperature=0.8, top_p=0.95))

``generate`` is a continuous-batching loop: prompts are prefetched into free slots as
earlier sequences finish, and every decode step advances all live slots at once.
Counterpart of the reference's ``_native_inference`` module and its Python wrapper
(``csrc/native_gpt2/resident_binding.cpp``, ``neuralfn/native_inference.py``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, fields
from typing import Iterable, Sequence

import torch

from ..ops import _lib

__all__ = ["EngineConfig", "Sampling", "ResidentEngine", "resident_inference_abi_version", "resident_inference_capabilities"]


class _CConfig(C.Structure):
    _fields_ = [("family", C.c_int), ("n_layer", C.c_int), ("d_model", C.c_int), ("n_head", C.c_int), ("n_kv_head", C.c_int),
                ("head_dim", C.c_int), ("d_ff", C.c_int), ("vocab", C.c_int), ("padded_vocab", C.c_int), ("max_seq", C.c_int),
                ("max_batch", C.c_int), ("qk_norm", C.c_int), ("rope_hf", C.c_int), ("rope_theta", C.c_float),
                ("norm_eps", C.c_float), ("qk_norm_eps", C.c_float), ("logit_softcap", C.c_float), ("tie_embeddings", C.c_int),
                ("window", C.c_int), ("global_every", C.c_int), ("embed_scale", C.c_float), ("use_cuda_graph", C.c_int),
                ("gated_attention", C.c_int), ("sandwich_norms", C.c_int), ("centered_norms", C.c_int), ("embed_norm", C.c_int),
                ("rope_local_only", C.c_int), ("q_scale", C.c_float), ("output_multiplier", C.c_float), ("post_norm_eps", C.c_float),
                ("mlp_activation", C.c_int), ("kv_cache_mode", C.c_int)]


class _CSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("seed", C.c_uint64)]


@dataclass
class Sampling:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    def c(self) -> _CSampling:
        return _CSampling(self.temperature, self.top_k, self.top_p, self.seed)


@dataclass
class EngineConfig:
    family: int = 0                # 0 GPT-2 style, 1 Llama style
    n_layer: int = 12
    d_model: int = 768
    n_head: int = 12
    n_kv_head: int = 12
    head_dim: int = 64
    d_ff: int = 3072
    vocab: int = 50257
    padded_vocab: int = 50304
    max_seq: int = 1024
    max_batch: int = 8
    qk_norm: int = 0               # 0 none, 1 weightless, 2 weighted
    rope_hf: int = 1
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    qk_norm_eps: float = 1e-6
    logit_softcap: float = 0.0
    tie_embeddings: int = 1
    window: int = 0
    global_every: int = 0
    embed_scale: float = 1.0
    use_cuda_graph: int = 1
    # Glimmer-style blocks (family 1): gated attention output, sandwich norms with (1 + w) scales,
    # weightless embedding norm, rotary embedding on sliding-window layers only, query scale,
    # logit multiplier
    gated_attention: int = 0
    sandwich_norms: int = 0
    centered_norms: int = 0
    embed_norm: int = 0
    rope_local_only: int = 0
    q_scale: float = 0.0
    output_multiplier: float = 0.0
    post_norm_eps: float = 0.0
    mlp_activation: int = 0       # GPT-2 family: epilogue id of the MLP activation (0 = tanh GELU); see MLP_ACTIVATION_IDS
    kv_cache_mode: int = 0        # 0: bf16 K / V rows; 1: TurboQuant 3.5-bit records (decode only: no verification blocks)

    MLP_ACTIVATION_IDS = {"gelu": 1, "silu": 3, "relu2": 4, "relu": 6}

    @classmethod
    def gpt2(cls, cfg, max_batch: int = 8, *, activation: str | None = None, **kw) -> "EngineConfig":
        """From a ``models.gpt2.GPT2Config``. ``activation``: the one a mixture-of-activations checkpoint selected
        (``checkpoint.dense.read_moa_sidecar``); default: the configuration's own."""
        kw.setdefault("mlp_activation", cls.MLP_ACTIVATION_IDS[activation or getattr(cfg, "mlp_activation", "gelu")])
        return cls(family=0, n_layer=cfg.n_layer, d_model=cfg.d_model, n_head=cfg.n_head, n_kv_head=cfg.n_head,
                   head_dim=cfg.head_dim, d_ff=cfg.mlp_mult * cfg.d_model, vocab=cfg.vocab_size, padded_vocab=cfg.padded_vocab,
                   max_seq=cfg.max_seq_len, max_batch=max_batch, qk_norm=1 if cfg.qk_norm else 0, norm_eps=cfg.ln_eps,
                   qk_norm_eps=cfg.qk_norm_eps, logit_softcap=cfg.logit_softcap, tie_embeddings=1, **kw)

    @classmethod
    def glimmer(cls, *, n_layer: int, d_model: int, n_head: int, n_kv_head: int, head_dim: int, d_ff: int, vocab: int, max_seq: int,
                window: int, max_batch: int = 8, logit_softcap: float = 20.0, **kw) -> "EngineConfig":
        """Muse-Glimmer block layout: every 4th layer global without position signal, the others
        sliding-window with rotary embedding (theta 5e5), weightless per-head QK norm with query scale
        3.87, gated attention, centered sandwich norms, output multiplier 0.19611613513818404."""
        base = dict(family=1, n_layer=n_layer, d_model=d_model, n_head=n_head, n_kv_head=n_kv_head, head_dim=head_dim, d_ff=d_ff,
                    vocab=vocab, padded_vocab=(vocab + 127) // 128 * 128, max_seq=max_seq, max_batch=max_batch, qk_norm=1, rope_hf=1,
                    rope_theta=5.0e5, norm_eps=1e-5, qk_norm_eps=1e-6, logit_softcap=logit_softcap, tie_embeddings=0, window=window,
                    global_every=4, gated_attention=1, sandwich_norms=1, centered_norms=1, embed_norm=1, rope_local_only=1,
                    q_scale=3.87, output_multiplier=0.19611613513818404, post_norm_eps=1e-8)
        base.update(kw)
        return cls(**base)

    def c(self) -> _CConfig:
        return _CConfig(*[getattr(self, f.name) for f in fields(self)])


def _api():
    L = _lib.load()
    if getattr(L, "_engine_ready", False):
        return L
    vp, ip = C.c_void_p, C.c_int
    L.nfn_engine_last_error.restype = C.c_char_p
    L.nfn_engine_create.restype, L.nfn_engine_create.argtypes = vp, [C.POINTER(_CConfig), ip]
    L.nfn_engine_destroy.restype, L.nfn_engine_destroy.argtypes = None, [vp]
    L.nfn_engine_set_tensor.argtypes = [vp, C.c_char_p, vp, C.c_longlong]
    L.nfn_engine_set_tensor_kquant.argtypes = [vp, C.c_char_p, ip, vp, C.c_longlong, C.c_longlong]
    L.nfn_engine_expected_tensors.argtypes = [vp, C.c_char_p, ip]
    L.nfn_engine_load_dense_v5.argtypes = [vp, C.c_char_p]
    L.nfn_engine_finalize.argtypes = [vp]
    L.nfn_engine_set_turboquant.argtypes = [vp, vp]
    L.nfn_engine_device_bytes.restype, L.nfn_engine_device_bytes.argtypes = C.c_longlong, [vp]
    L.nfn_engine_prefill.argtypes = [vp, ip, vp, ip, C.POINTER(_CSampling), vp]
    L.nfn_engine_decode.argtypes = [vp, vp, vp, C.POINTER(_CSampling), vp, vp]
    L.nfn_engine_release.argtypes = [vp, ip]
    L.nfn_engine_slot_length.argtypes = [vp, ip]
    L.nfn_engine_last_logits.argtypes = [vp, ip, vp]
    L.nfn_engine_launches.restype, L.nfn_engine_launches.argtypes = C.c_longlong, [vp]
    L.nfn_engine_enable_verify.argtypes = [vp, ip]
    L.nfn_engine_verify.argtypes = [vp, vp, vp, ip, vp]
    L.nfn_engine_verify_logits.argtypes = [vp, ip, ip, vp]
    L.nfn_engine_commit.argtypes = [vp, vp]
    L.nfn_engine_truncate.argtypes = [vp, ip, ip]
    L.nfn_engine_fork.argtypes = [vp, ip, ip, ip]
    L.nfn_engine_prefill_rows.argtypes = [vp, ip, vp, ip, ip, C.POINTER(_CSampling), vp]
    L.nfn_engine_enable_taps.argtypes = [vp, vp, ip]
    L.nfn_engine_read_taps.argtypes = [vp, ip, ip, ip, vp, ip]
    L._engine_ready = True
    return L


def resident_inference_abi_version() -> int:
    return int(_api().nfn_engine_abi_version())


def resident_inference_capabilities() -> dict:
    return {"abi_version": resident_inference_abi_version(), "families": ["gpt2", "llama"], "kv_cache": "bf16",
            "hybrid_local_global": True, "qk_norm": True, "rope": ["hf", "legacy"], "continuous_batching": True,
            "cuda_graph_decode": True, "on_device_sampling": ["greedy", "temperature", "top_k", "top_p"],
            # projection weights may stay resident in K-quant blocks (``set_tensor_kquant``: quantised GEMV for up to eight rows,
            # decode-then-GEMM beyond); NF4 checkpoints are dequantised at load time; there is no int8-activation MMQ path
            "block_verification": True, "hidden_state_taps": True, "gpt2_mlp_activations": sorted(EngineConfig.MLP_ACTIVATION_IDS),
            "kv_cache_modes": ["bf16", "turboquant-3.5 (decode only)"], "quantized_weights": ["Q4_K", "Q5_K", "Q6_K"], "weight_dtypes": ["bf16", "k-quant projections (set_tensor_kquant)"],
            "dequantised_at_load": ["NF4"]}


class EngineError(RuntimeError):
    pass


class ResidentEngine:
    def __init__(self, config: EngineConfig, device: int = 0, *, turboquant_profile: str = "mse-3.5", turboquant_seed: int = 0) -> None:
        self.config = config
        self.device = int(device)
        self._L = _api()
        cc = config.c()
        self._h = self._L.nfn_engine_create(C.byref(cc), device)
        if not self._h:
            raise EngineError(self._err())
        self._finalized = False
        if config.kv_cache_mode == 1:
            self._set_turboquant(turboquant_profile, turboquant_seed)

    def _set_turboquant(self, profile: str, seed: int) -> None:
        """``kv_cache_mode`` 1: the codec of ``quant.turboquant`` (deterministic rotation / projection, Lloyd-Max centroids, the
        default outlier channel set) lives on the device for the engine's life; K / V are kept as its records."""
        from ..quant.turboquant import TurboQuantCodec, default_outlier_indices
        hd = self.config.head_dim
        self.turboquant = TurboQuantCodec(hd, profile=profile, seed=seed, outlier_indices=default_outlier_indices(hd))
        self._tq_tensors = t = self.turboquant.device_tables(torch.device("cuda", self.device))

        class _Tables(C.Structure):
            _fields_ = [("rotation", C.c_void_p), ("projection", C.c_void_p), ("centroids", C.c_void_p), ("key_fields", C.c_void_p),
                        ("value_fields", C.c_void_p), ("D", C.c_int), ("qjl", C.c_int), ("key_rec_bytes", C.c_int), ("value_rec_bytes", C.c_int)]
        self._tq_c = _Tables(t["rotation"].data_ptr(), t["projection"].data_ptr(), t["centroids"].data_ptr(), t["key_fields"].data_ptr(),
                             t["value_fields"].data_ptr(), hd, int(profile == "qjl-3.5"), self.turboquant.key_layout.record_bytes,
                             self.turboquant.value_layout.record_bytes)
        self._check(self._L.nfn_engine_set_turboquant(self._h, C.cast(C.byref(self._tq_c), C.c_void_p)))

    @property
    def kv_bytes_per_token(self) -> int:
        """Cache bytes one token occupies in a global (full-context) layer."""
        c = self.config
        if c.kv_cache_mode == 1:
            return c.n_kv_head * (self.turboquant.key_layout.record_bytes + self.turboquant.value_layout.record_bytes)
        return 2 * c.n_kv_head * c.head_dim * 2

    def _err(self) -> str:
        return (self._L.nfn_engine_last_error() or b"").decode("utf-8", "replace")

    def _check(self, rc: int) -> None:
        if rc < 0:
            raise EngineError(self._err())

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._L.nfn_engine_destroy(self._h)
            self._h = None

    __del__ = close

    # ---- weights --------------------------------------------------------------------------
    def expected_tensors(self) -> dict[str, int]:
        n = self._L.nfn_engine_expected_tensors(self._h, None, 0)
        buf = C.create_string_buffer(n + 1)
        self._L.nfn_engine_expected_tensors(self._h, buf, n + 1)
        return {a: int(b) for a, b in (line.split() for line in buf.value.decode().splitlines())}

    def set_tensor(self, name: str, t: torch.Tensor) -> None:
        t = t.detach().to("cpu", torch.bfloat16).contiguous()
        self._check(self._L.nfn_engine_set_tensor(self._h, name.encode(), t.data_ptr(), t.numel()))

    QTYPES = {"Q4_K": 12, "Q5_K": 13, "Q6_K": 14}

    def set_tensor_kquant(self, name: str, qtype: int | str, blocks: torch.Tensor) -> None:
        """Keeps projection weight ``name`` resident in its K-quant blocks (uint8, rows of K / 256 super-blocks back to back - the
        GGUF layout). Decode-sized products (up to eight rows) read the blocks directly; larger ones decode the tensor into one
        shared bf16 scratch buffer first. Embeddings, norms and biases stay bf16.

        Reference counterpart: the K-quant resident weights of ``resident_glimmer_cuda.cpp`` (``weight_precision k-quant-*``)."""
        from ..ops.infer import quant_block_bytes
        q = self.QTYPES[qtype] if isinstance(qtype, str) else int(qtype)
        b = blocks.detach().to("cpu", torch.uint8).contiguous().reshape(-1)
        numel = b.numel() // quant_block_bytes(q) * 256
        self._check(self._L.nfn_engine_set_tensor_kquant(self._h, name.encode(), q, b.data_ptr(), b.numel(), numel))

    def load_named_tensors(self, tensors: dict[str, torch.Tensor], quantized: dict[str, tuple] | None = None) -> None:
        """``quantized``: name -> (qtype, uint8 blocks) for projection weights that stay in K-quant form; those names need no
        entry in ``tensors``."""
        quantized = quantized or {}
        for name, (qtype, blocks) in quantized.items():
            self.set_tensor_kquant(name, qtype, blocks)
        for name, numel in self.expected_tensors().items():
            if name in quantized:
                continue
            if name not in tensors:
                raise EngineError(f"missing tensor {name!r}")
            t = tensors[name]
            if name in ("wte", "tok_embeddings", "lm_head") and t.numel() < numel:  # pad the vocabulary rows
                pad = torch.zeros(numel // t.shape[1] - t.shape[0], t.shape[1], dtype=t.dtype)
                t = torch.cat([t.cpu(), pad])
            self.set_tensor(name, t)
        self.finalize()

    def load_dense_checkpoint(self, path) -> None:
        self._check(self._L.nfn_engine_load_dense_v5(self._h, str(path).encode()))
        self.finalize()

    def load_hf_llama_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        """Hugging Face Llama / Qwen3-style names -> the engine's fused layout (q|k|v rows
        concatenated, gate|up rows concatenated)."""
        c = self.config
        out = {"tok_embeddings": sd["model.embed_tokens.weight"], "norm": sd["model.norm.weight"]}
        if not c.tie_embeddings:
            out["lm_head"] = sd["lm_head.weight"]
        for l in range(c.n_layer):
            p = f"model.layers.{l}."
            out[f"layers.{l}.attn_norm"] = sd[p + "input_layernorm.weight"]
            out[f"layers.{l}.wqkv"] = torch.cat([sd[p + f"self_attn.{n}_proj.weight"] for n in "qkv"])
            if c.qk_norm == 2:
                out[f"layers.{l}.q_norm"] = sd[p + "self_attn.q_norm.weight"]
                out[f"layers.{l}.k_norm"] = sd[p + "self_attn.k_norm.weight"]
            out[f"layers.{l}.wo"] = sd[p + "self_attn.o_proj.weight"]
            out[f"layers.{l}.ffn_norm"] = sd[p + "post_attention_layernorm.weight"]
            out[f"layers.{l}.w_gate_up"] = torch.cat([sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"]])
            out[f"layers.{l}.w_down"] = sd[p + "mlp.down_proj.weight"]
        self.load_named_tensors(out)

    def finalize(self) -> None:
        self._check(self._L.nfn_engine_finalize(self._h))
        self._finalized = True

    @property
    def device_bytes(self) -> int:
        return int(self._L.nfn_engine_device_bytes(self._h))

    @property
    def launches(self) -> int:
        return int(self._L.nfn_engine_launches(self._h))

    # ---- stepping --------------------------------------------------------------------------
    def prefill(self, slot: int, tokens: Sequence[int], sampling: Sampling | None = None) -> int:
        arr = (C.c_int32 * len(tokens))(*tokens)
        out = C.c_int32(0)
        s = (sampling or Sampling()).c()
        self._check(self._L.nfn_engine_prefill(self._h, slot, C.cast(arr, C.c_void_p), len(tokens), C.byref(s), C.cast(C.byref(out), C.c_void_p)))
        return int(out.value)

    def prefill_rows(self, slot: int, rows: torch.Tensor, sampling: Sampling | None = None) -> int:
        """Runs a prompt given as its layer-0 input rows (bf16 [n, d_model], host or this engine's device): token embeddings
        after the embedding norm, media placeholders replaced by projected media features (``serving.multimodal``)."""
        if rows.dim() != 2 or rows.shape[1] != self.config.d_model or rows.dtype != torch.bfloat16:
            raise EngineError("prefill_rows wants a bf16 [n, d_model] tensor")
        rows = rows.contiguous()
        out = C.c_int32(0)
        s = (sampling or Sampling()).c()
        self._check(self._L.nfn_engine_prefill_rows(self._h, slot, C.c_void_p(rows.data_ptr()), rows.shape[0], int(rows.is_cuda), C.byref(s),
                                                    C.cast(C.byref(out), C.c_void_p)))
        return int(out.value)

    def decode(self, tokens_in: dict[int, int], sampling: Sampling | None = None, per_slot: dict[int, Sampling] | None = None) -> dict[int, int]:
        B = self.config.max_batch
        tok = (C.c_int32 * B)()
        act = (C.c_uint8 * B)()
        for slot, t in tokens_in.items():
            tok[slot], act[slot] = t, 1
        s = (sampling or Sampling()).c()
        ps = None
        if per_slot:
            ps = (_CSampling * B)(*[(per_slot.get(b) or sampling or Sampling()).c() for b in range(B)])
        out = (C.c_int32 * B)()
        self._check(self._L.nfn_engine_decode(self._h, C.cast(tok, C.c_void_p), C.cast(act, C.c_void_p), C.byref(s),
                                              C.cast(ps, C.c_void_p) if ps is not None else None, C.cast(out, C.c_void_p)))
        return {slot: int(out[slot]) for slot in tokens_in}

    def release(self, slot: int) -> None:
        self._check(self._L.nfn_engine_release(self._h, slot))

    def slot_length(self, slot: int) -> int:
        return int(self._L.nfn_engine_slot_length(self._h, slot))

    def last_logits(self, slot: int) -> torch.Tensor:
        out = torch.empty(self.config.vocab, dtype=torch.float32)
        self._check(self._L.nfn_engine_last_logits(self._h, slot, out.data_ptr()))
        return out

    # ---- hidden-state taps (context of a block-diffusion draft) ---------------------------------
    def enable_taps(self, layers: Sequence[int]) -> None:
        """Keep the residual stream after each listed layer (0-based) for every cached position. Call before the first decode step."""
        arr = (C.c_int32 * len(layers))(*[int(l) for l in layers])
        self._check(self._L.nfn_engine_enable_taps(self._h, C.cast(arr, C.c_void_p), len(layers)))
        self.tap_layers = tuple(int(l) for l in layers)

    def read_taps(self, slot: int, pos0: int, n: int, *, device: bool = True):
        """bf16 [n, taps * d_model] for positions [pos0, pos0 + n) of ``slot`` (a CUDA tensor, or a host tensor with ``device=False``)."""
        import torch
        width = len(getattr(self, "tap_layers", ())) * self.config.d_model
        if not width:
            raise RuntimeError("taps are not enabled on this engine")
        out = torch.empty(n, width, dtype=torch.bfloat16, device=torch.device("cuda", self.device) if device else "cpu")
        self._check(self._L.nfn_engine_read_taps(self._h, slot, pos0, n, C.c_void_p(out.data_ptr()), int(device)))
        return out

    # ---- block verification / session operations ----------------------------------------------
    def enable_verify(self, max_rows: int = 17) -> None:
        """Allocates the staging buffers for ``verify`` / ``commit`` (once)."""
        self._check(self._L.nfn_engine_enable_verify(self._h, max_rows))
        self._verify_rows = max(max_rows, getattr(self, "_verify_rows", 0))

    def verify(self, blocks: dict[int, Sequence[int]]) -> dict[int, list[int]]:
        """Runs each slot's token block at the slot's current position without touching its KV
        cache. Returns, per slot, the most likely successor after every block row."""
        if not getattr(self, "_verify_rows", 0):
            self.enable_verify()
        B = self.config.max_batch
        rows = max(len(v) for v in blocks.values())
        tok = (C.c_int32 * (B * rows))()
        live = (C.c_int32 * B)()
        for slot, ids in blocks.items():
            live[slot] = len(ids)
            for r, t in enumerate(ids):
                tok[slot * rows + r] = t
        out = (C.c_int32 * (B * rows))()
        self._check(self._L.nfn_engine_verify(self._h, C.cast(tok, C.c_void_p), C.cast(live, C.c_void_p), rows, C.cast(out, C.c_void_p)))
        self._last_verify_rows = rows
        return {slot: [int(out[slot * rows + r]) for r in range(len(ids))] for slot, ids in blocks.items()}

    def verify_logits(self, slot: int, row: int) -> torch.Tensor:
        out = torch.empty(self.config.vocab, dtype=torch.float32)
        self._check(self._L.nfn_engine_verify_logits(self._h, slot, row, out.data_ptr()))
        return out

    def commit(self, accepted: dict[int, int]) -> None:
        """Appends the first ``accepted[slot]`` rows of the last ``verify`` to the caches."""
        acc = (C.c_int32 * self.config.max_batch)()
        for slot, n in accepted.items():
            acc[slot] = n
        self._check(self._L.nfn_engine_commit(self._h, C.cast(acc, C.c_void_p)))

    def append(self, slot: int, tokens: Sequence[int], chunk: int | None = None) -> int:
        """Extends a slot that already holds tokens (``prefill`` only starts at position 0).
        Returns the most likely next token."""
        if not getattr(self, "_verify_rows", 0):
            self.enable_verify()
        chunk = min(chunk or self._verify_rows, self._verify_rows)
        nxt = -1
        for i in range(0, len(tokens), chunk):
            part = list(tokens[i:i + chunk])
            nxt = self.verify({slot: part})[slot][-1]
            self.commit({slot: len(part)})
        return nxt

    def truncate(self, slot: int, n: int) -> None:
        self._check(self._L.nfn_engine_truncate(self._h, slot, n))

    def fork(self, src_slot: int, dst_slot: int, n: int | None = None) -> None:
        self._check(self._L.nfn_engine_fork(self._h, src_slot, dst_slot, self.slot_length(src_slot) if n is None else n))

    def generate(self, prompts: Iterable[Sequence[int]], max_new_tokens: int = 32, sampling: Sampling | None = None,
                 eos_token: int | None = None) -> list[list[int]]:
        """Continuous batching over ``max_batch`` slots; returns the generated ids per prompt."""
        prompts = [list(p) for p in prompts]
        results: list[list[int]] = [[] for _ in prompts]
        pending = list(range(len(prompts)))[::-1]
        live: dict[int, int] = {}       # slot -> prompt index
        last: dict[int, int] = {}       # slot -> token to feed next
        free = list(range(self.config.max_batch))[::-1]
        sampling = sampling or Sampling()

        def finished(idx: int, tok: int) -> bool:
            return len(results[idx]) >= max_new_tokens or (eos_token is not None and tok == eos_token)

        while pending or live:
            while pending and free:
                idx, slot = pending.pop(), free.pop()
                tok = self.prefill(slot, prompts[idx], sampling)
                results[idx].append(tok)
                if finished(idx, tok) or len(prompts[idx]) + 1 >= self.config.max_seq:
                    self.release(slot)
                    free.append(slot)
                else:
                    live[slot], last[slot] = idx, tok
            if not live:
                continue
            nxt = self.decode({slot: last[slot] for slot in live}, sampling)
            for slot, tok in nxt.items():
                idx = live[slot]
                results[idx].append(tok)
                last[slot] = tok
                if finished(idx, tok) or self.slot_length(slot) + 1 >= self.config.max_seq:
                    self.release(slot)
                    free.append(slot)
                    del live[slot], last[slot]
        return results
