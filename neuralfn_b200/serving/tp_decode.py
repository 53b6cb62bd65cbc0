"""Tensor-parallel Llama inference across the GPUs of one NVSwitch domain: sharded weights and
KV cache, prefill through the fused all-gather→GEMM / GEMM→reduce-scatter kernels, decode with
one fused all-reduce + residual + RMS-norm kernel after each row-parallel projection.

Per rank: H / W query heads and Hkv / W key-value heads of every layer (so the KV cache is
split W ways too), d_ff / W hidden units, V / W rows of the LM head. A decode step for B rows:

    h = norm(x)                                  (first layer only; later ones come fused)
    per layer:  qkv = h Wqkv_l^T                 local GEMM            [B, (Hq_l + 2 Hkv_l) D]
                a   = decode_attention(qkv)      rotary + append + attention on the local heads
                p   = a Wo_l^T                   local GEMM into a symmetric partial buffer
                h   = allreduce(p) + x -> x, RMS norm(ffn_norm)        ONE kernel over peer memory
                g   = swiglu(h Wgu_l^T);  p = g Wdown_l^T
                h   = allreduce(p) + x -> x, RMS norm(next attn_norm / final norm)
    logits_l = h Whead_l^T; local arg-max (value, global index); the W candidates are gathered
    and merged, every rank ends up with the same next token.

The whole step can be captured in a CUDA graph (``use_graph=True``): the fused kernels take
their epoch from a device counter that a tiny kernel advances at the start of every replay.
On CPU (gloo ranks) every operation falls back to PyTorch; that is what the parity tests run.

The reference serves on one GPU (``csrc/native_gpt2/resident_infer.cpp``); its north-star
configuration asks for the same model split over eight.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..models.llama import LlamaConfig
from ..parallel.tp import TensorParallelContext
from ..parallel.tp_llama import shard_llama_params

__all__ = ["TPLlamaDecoder", "random_full_params"]


def random_full_params(cfg: LlamaConfig, seed: int) -> dict[str, torch.Tensor]:
    """An unsharded random model on the host (tests: the same on every rank, and the oracle's input)."""
    from ..models.gpt2 import FlatLayout
    from ..models.llama import init_llama_params_, llama_param_specs
    layout = FlatLayout(llama_param_specs(cfg))
    flat = torch.zeros(layout.n_total)
    init_llama_params_(cfg, layout, flat, seed)
    return {k: v.clone() for k, v in layout.views(flat).items()}


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class TPLlamaDecoder:
    def __init__(self, cfg: LlamaConfig, tp: TensorParallelContext, *, max_batch: int, max_seq: int, full_params: dict | None = None,
                 seed: int = 1234, use_graph: bool = False) -> None:
        W = tp.world
        if cfg.n_head % W or cfg.n_kv_head % W or cfg.d_ff % W or cfg.padded_vocab % (8 * W):
            raise ValueError("heads, d_ff and the padded vocabulary must divide by the TP size")
        if cfg.tie_embeddings or cfg.qk_norm or cfg.logit_softcap > 0 or cfg.window:
            raise ValueError("the tensor-parallel decoder covers the plain Llama block")
        self.cfg, self.tp, self.B, self.cap = cfg, tp, max_batch, max_seq
        dev = self.dev = tp.device
        self.cuda = dev.type == "cuda"
        self.dtype = torch.bfloat16 if self.cuda else torch.float32
        self.Hq, self.Hkv, self.Fl, self.Vl = cfg.n_head // W, cfg.n_kv_head // W, cfg.d_ff // W, cfg.padded_vocab // W
        hd, C = cfg.head_dim, cfg.d_model
        if full_params is not None:
            sh = shard_llama_params(cfg, full_params, tp.rank, W)
            to = lambda t: t.to(dev, self.dtype).contiguous()
            # the decoder keeps the embedding table whole (one row gather per token) and shards the head by vocabulary rows
            self.embed = to(full_params["tok_embeddings"])
            self.head = to(full_params["lm_head"][tp.rank * self.Vl:(tp.rank + 1) * self.Vl])
            self.norm = to(sh["norm"])
            self.layers = [{k: to(sh[f"layers.{l}.{k}"]) for k in ("attn_norm", "wqkv", "wo", "ffn_norm", "w_gate_up", "w_down")}
                           for l in range(cfg.n_layer)]
        else:
            self._random_shards(seed)
        self.k_cache = [torch.zeros(max_batch, self.Hkv, max_seq, hd, dtype=self.dtype, device=dev) for _ in range(cfg.n_layer)]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]
        self.lengths = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        from ..ops.infer import rope_tables
        self.cos, self.sin = rope_tables(max_seq, hd, cfg.rope_theta, device=dev)
        self.x = torch.zeros(max_batch, C, dtype=self.dtype, device=dev)        # residual stream of the decode step
        self.tokens = torch.zeros(max_batch, dtype=torch.int64, device=dev)
        self.last_logits: torch.Tensor | None = None
        self.sampling: tuple | None = None   # (temperature, top_k, top_p, seed); None = greedy
        self._draws = 0
        self.use_graph = bool(use_graph and self.cuda)
        self._graph = None
        self._graph_ok = True   # cleared once a library collective ran on this group (see prefill)
        self._fused_calls_per_step = 2 * cfg.n_layer + (1 if W > 1 else 0)  # two per layer + the candidate exchange
        if self.cuda:
            from ..ops.infer import DecodeAttentionWorkspace
            self._ws = DecodeAttentionWorkspace(max_batch, self.Hq, self.Hkv, hd, dev)
            self._gemm_ws = torch.empty(32 << 20, dtype=torch.uint8, device=dev)  # split-K partials of the skinny products

    @classmethod
    def from_hf_directory(cls, directory, tp: TensorParallelContext, *, max_batch: int, max_seq: int, use_graph: bool = False) -> "TPLlamaDecoder":
        """Loads a Hugging Face Llama checkpoint directory (``config.json`` + safetensors, sharded
        or not) and keeps this rank's shards. Every rank reads the files; only its slices go to
        the device."""
        from ..checkpoint.safetensors_io import load_hf_llama_directory
        ec, tensors = load_hf_llama_directory(directory, max_batch=max_batch, max_seq=max_seq)
        if ec.tie_embeddings:
            tensors["lm_head"] = tensors["tok_embeddings"]
        cfg = LlamaConfig(n_layer=ec.n_layer, n_head=ec.n_head, n_kv_head=ec.n_kv_head, d_model=ec.d_model, d_ff=ec.d_ff, vocab_size=ec.vocab,
                          max_seq_len=max_seq, rope_theta=ec.rope_theta, rope_convention="hf", norm_eps=ec.norm_eps, head_dim_override=ec.head_dim,
                          vocab_pad_to=8 * tp.world)
        pad = cfg.padded_vocab - tensors["tok_embeddings"].shape[0]
        if pad > 0:  # the decoder wants the vocabulary divisible by 8 x world
            for k in ("tok_embeddings", "lm_head"):
                tensors[k] = torch.cat([tensors[k], torch.zeros(pad, ec.d_model, dtype=tensors[k].dtype)], 0)
        return cls(cfg, tp, max_batch=max_batch, max_seq=max_seq, full_params=tensors, use_graph=use_graph)

    def _random_shards(self, seed: int) -> None:
        """Random weights drawn shard by shard on the device (benchmarks): replicated tensors from
        a stream every rank shares, shards from one keyed by the rank."""
        cfg, dev, hd, C = self.cfg, self.dev, self.cfg.head_dim, self.cfg.d_model
        shared = torch.Generator(device=dev).manual_seed(seed)
        own = torch.Generator(device=dev).manual_seed(seed * 7919 + 1 + self.tp.rank)

        def rnd(shape, gen, std=0.02):
            return torch.empty(shape, dtype=torch.float32, device=dev).normal_(0.0, std, generator=gen).to(self.dtype)

        self.embed = rnd((cfg.padded_vocab, C), shared)
        self.head = rnd((self.Vl, C), own)
        self.norm = torch.ones(C, dtype=self.dtype, device=dev)
        rs = 0.02 / (2 * cfg.n_layer) ** 0.5
        self.layers = [{"attn_norm": torch.ones(C, dtype=self.dtype, device=dev), "ffn_norm": torch.ones(C, dtype=self.dtype, device=dev),
                        "wqkv": rnd(((self.Hq + 2 * self.Hkv) * hd, C), own), "wo": rnd((C, self.Hq * hd), own, rs),
                        "w_gate_up": rnd((2 * self.Fl, C), own), "w_down": rnd((C, self.Fl), own, rs)} for _ in range(cfg.n_layer)]

    # ------------------------------------------------------------------ local building blocks --
    def _mm(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if self.cuda:
            from ..ops.gemm import gemm
            return gemm(x, w, out=out, workspace=self._gemm_ws if x.shape[0] <= 128 else None)
        y = x @ w.T
        if out is not None:
            out.copy_(y)
            return out
        return y

    def _attend_one(self, qkv: torch.Tensor, l: int) -> torch.Tensor:
        """New-token attention for every row: rotary at position length - 1, append, attend."""
        cfg, hd = self.cfg, self.cfg.head_dim
        if self.cuda:
            from ..ops.infer import decode_attention
            return decode_attention(qkv, self.k_cache[l], self.v_cache[l], self.lengths, n_q_heads=self.Hq, n_kv_heads=self.Hkv, head_dim=hd,
                                    workspace=self._ws, cos=self.cos, sin=self.sin, convention=cfg.rope_convention)
        B = qkv.shape[0]
        pos = (self.lengths[:B] - 1).long()
        cos, sin = self.cos[pos][:, None], self.sin[pos][:, None]
        sign = 1.0 if cfg.rope_convention == "hf" else -1.0

        def rot(t):
            a, b = t[..., :hd // 2], t[..., hd // 2:]
            return torch.cat((a * cos - sign * b * sin, b * cos + sign * a * sin), -1)

        q = rot(qkv[:, :self.Hq * hd].view(B, self.Hq, hd))
        k = rot(qkv[:, self.Hq * hd:(self.Hq + self.Hkv) * hd].view(B, self.Hkv, hd))
        v = qkv[:, (self.Hq + self.Hkv) * hd:].view(B, self.Hkv, hd)
        rows = torch.arange(B)
        self.k_cache[l][rows, :, pos] = k
        self.v_cache[l][rows, :, pos] = v
        rep = self.Hq // self.Hkv
        kk = self.k_cache[l][:B].repeat_interleave(rep, 1)
        vv = self.v_cache[l][:B].repeat_interleave(rep, 1)
        s = torch.einsum("bhd,bhtd->bht", q, kk) * hd ** -0.5
        s = s.masked_fill(torch.arange(self.cap)[None, None, :] >= self.lengths[:B, None, None], float("-inf"))
        return torch.einsum("bht,bhtd->bhd", s.softmax(-1), vv).reshape(B, self.Hq * hd)

    def _reduce(self, partial: torch.Tensor, sym, norm_weight: torch.Tensor) -> torch.Tensor:
        return self.tp.allreduce_resid_norm(partial, sym, resid=self.x[:partial.shape[0]], norm_weight=norm_weight, eps=self.cfg.norm_eps)

    def _partial(self, B: int):
        if self.tp.impl == "fused":
            return self.tp.partial_buffer(B, self.cfg.d_model)
        return torch.empty(B, self.cfg.d_model, dtype=self.dtype, device=self.dev), None

    def _pick(self, h: torch.Tensor) -> torch.Tensor:
        """Greedy next token from the normalised hidden rows: local head slice, local arg-max,
        gather of the W candidates, merge."""
        logits = self._mm(h, self.head)
        self.last_logits = logits
        off, W = self.tp.rank * self.Vl, self.tp.world
        if self.tp.rank == W - 1 and self.cfg.padded_vocab != self.cfg.vocab_size:
            logits[:, self.cfg.vocab_size - off:] = -30000.0
        if self.sampling is not None:
            return self._sample(logits)
        val, idx = logits.float().max(-1)
        idx = idx + off
        if W == 1:
            return idx
        if self.tp.impl == "fused":
            # Exchange the candidates through the fused all-reduce kernel (no NCCL call, so the step
            # stays capturable and free of library collectives): every rank fills its own four
            # columns of a zero [B, 4 W] row - the value (already a bf16 number) and the index as
            # three base-128 digits, each exact in bf16 - and the sum over ranks is the gather.
            cols = max(8, 4 * W)
            cand, sym = self.tp.partial_buffer(logits.shape[0], cols)
            cand.zero_()
            mine = torch.stack([val, (idx % 128).float(), ((idx // 128) % 128).float(), (idx // 16384).float()], -1)
            cand[:, 4 * self.tp.rank:4 * self.tp.rank + 4] = mine.to(cand.dtype)
            allc = self.tp.allreduce_resid_norm(cand, sym)[:, :4 * W].float().view(-1, W, 4)
            vals = allc[..., 0]
            ids = allc[..., 1] + 128.0 * allc[..., 2] + 16384.0 * allc[..., 3]
            best = vals.argmax(1, keepdim=True)  # the first (lowest-rank) maximum wins, as an arg-max over the full row would pick
            return ids.gather(1, best).squeeze(1).long()
        mine = torch.stack([val, idx.float()], -1).contiguous()  # indices below 2^24 are exact in fp32
        allc = torch.empty(W, *mine.shape, dtype=mine.dtype, device=mine.device)
        dist.all_gather_into_tensor(allc, mine, group=self.tp.group) if self.cuda else \
            allc.copy_(torch.stack(self._gather_list(mine)))
        best = allc[..., 0].argmax(0)
        return allc[..., 1].gather(0, best[None]).squeeze(0).long()

    def set_sampling(self, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> None:
        """``temperature == 0`` selects greedy decoding (the default). With sampling every rank gathers
        the full logit rows and draws with the same counter-based generator, so all ranks pick the
        same token without exchanging it. A captured decode graph is dropped and captured again."""
        self.sampling = None if temperature <= 0 else (float(temperature), int(top_k), float(top_p), int(seed))
        self._graph = None
        self._draws = 0
        if self.cuda:
            self._draw_ctr = torch.zeros(1, dtype=torch.int64, device=self.dev)

    def _sample(self, logits: torch.Tensor) -> torch.Tensor:
        temperature, top_k, top_p, seed = self.sampling
        W, B = self.tp.world, logits.shape[0]
        if W > 1:
            allg = torch.empty(W, B, self.Vl, dtype=logits.dtype, device=logits.device)
            if self.cuda:
                dist.all_gather_into_tensor(allg, logits.contiguous(), group=self.tp.group)
            else:
                allg.copy_(torch.stack(self._gather_list(logits.contiguous())))
            full = allg.permute(1, 0, 2).reshape(B, W * self.Vl).contiguous()
        else:
            full = logits
        if self.cuda:
            from ..ops.infer import sample_rows
            tok = sample_rows(full, temperature=temperature, top_k=top_k, top_p=top_p, seed=seed, offset_dev=self._draw_ctr).long()
            self._draw_ctr += 1  # a device-side counter, so replays of a captured step draw fresh numbers
            return tok
        z = full.float() / temperature
        if top_k > 0:
            kth = z.topk(min(top_k, z.shape[-1]), -1).values[:, -1:]
            z = z.masked_fill(z < kth, float("-inf"))
        p = z.softmax(-1)
        if top_p < 1.0:
            sp, si = p.sort(-1, descending=True)
            keep = sp.cumsum(-1) - sp < top_p
            p = torch.zeros_like(p).scatter(-1, si, sp * keep)
            p = p / p.sum(-1, keepdim=True)
        gen = torch.Generator().manual_seed(seed * 1000003 + self._draws)
        self._draws += 1
        return torch.multinomial(p, 1, generator=gen).squeeze(-1)

    def _gather_list(self, t: torch.Tensor) -> list[torch.Tensor]:
        parts = [torch.empty_like(t) for _ in range(self.tp.world)]
        dist.all_gather(parts, t, group=self.tp.group)
        return parts

    # ----------------------------------------------------------------------------- prefill --
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, T] (B = max_batch rows, the same on every rank; B x T divisible by W).
        Fills the caches and returns the first generated token of every row."""
        cfg, tp, hd = self.cfg, self.tp, self.cfg.head_dim
        B, T = tokens.shape
        M, W = B * T, tp.world
        if B != self.B or T > self.cap or M % W:
            raise ValueError("prefill wants max_batch rows, T <= max_seq and B x T divisible by the TP size")
        rows, lo = M // W, tp.rank * (M // W)
        if tp.impl == "fused" and rows % 128:
            # the fused collective GEMMs work on 128-row tiles per rank: short prompts take the NCCL
            # collectives around the plain GEMM for this one pass (decode steps are unaffected)
            tp.impl = "nccl"
            # library collectives have now been issued on this communicator: decode steps stay eager
            # (capturing after NCCL traffic aborted in a 2-GPU run; with the fused prefill it does not)
            self._graph_ok = W == 1
            try:
                return self.prefill(tokens)
            finally:
                tp.impl = "fused"
        x = self.embed[tokens.reshape(-1)[lo:lo + rows].long()]
        for l, p in enumerate(self.layers):
            qkv = tp.column_linear(_rms(x, p["attn_norm"], cfg.norm_eps), p["wqkv"])
            if self.cuda:
                from ..ops import kernels as K
                from ..ops.infer import rope_inplace
                rope_inplace(qkv, T=T, n_q_heads=self.Hq, n_kv_heads=self.Hkv, head_dim=hd, cos=self.cos, sin=self.sin, convention=cfg.rope_convention)
                q, k, v = qkv[:, :self.Hq * hd], qkv[:, self.Hq * hd:(self.Hq + self.Hkv) * hd], qkv[:, (self.Hq + self.Hkv) * hd:]
                a, _ = K.attention_forward(q.contiguous(), k.contiguous(), v.contiguous(), B=B, T=T, n_q_heads=self.Hq, n_kv_heads=self.Hkv,
                                           head_dim=hd, causal=True, window=0, scale=hd ** -0.5)
                k4, v4 = k.reshape(B, T, self.Hkv, hd), v.reshape(B, T, self.Hkv, hd)
            else:
                sign = 1.0 if cfg.rope_convention == "hf" else -1.0
                cos, sin = self.cos[:T][None, :, None], self.sin[:T][None, :, None]

                def rot(t):
                    a_, b_ = t[..., :hd // 2], t[..., hd // 2:]
                    return torch.cat((a_ * cos - sign * b_ * sin, b_ * cos + sign * a_ * sin), -1)

                q4 = rot(qkv[:, :self.Hq * hd].view(B, T, self.Hq, hd))
                k4 = rot(qkv[:, self.Hq * hd:(self.Hq + self.Hkv) * hd].view(B, T, self.Hkv, hd))
                v4 = qkv[:, (self.Hq + self.Hkv) * hd:].view(B, T, self.Hkv, hd)
                a = F.scaled_dot_product_attention(q4.transpose(1, 2), k4.transpose(1, 2), v4.transpose(1, 2), is_causal=True,
                                                   enable_gqa=True).transpose(1, 2).reshape(M, self.Hq * hd)
            self.k_cache[l][:, :, :T] = k4.transpose(1, 2)
            self.v_cache[l][:, :, :T] = v4.transpose(1, 2)
            x = tp.row_linear(a, p["wo"], resid=x)
            gu = tp.column_linear(_rms(x, p["ffn_norm"], cfg.norm_eps), p["w_gate_up"])
            x = tp.row_linear(F.silu(gu[:, :self.Fl]) * gu[:, self.Fl:], p["w_down"], resid=x)
        if W > 1:
            full = torch.empty(M, cfg.d_model, dtype=x.dtype, device=x.device)
            if self.cuda:
                dist.all_gather_into_tensor(full, x.contiguous(), group=tp.group)
            else:
                full.copy_(torch.cat(self._gather_list(x.contiguous())))
        else:
            full = x
        last = full.view(B, T, -1)[:, -1]
        self.lengths.fill_(T)
        nxt = self._pick(_rms(last, self.norm, cfg.norm_eps))
        self.tokens.copy_(nxt)
        return nxt.clone()

    # ------------------------------------------------------------------------------ decode --
    def _step_body(self) -> None:
        """Consumes ``self.tokens`` (appends them at ``lengths``) and leaves the next ones there."""
        cfg, B = self.cfg, self.B
        self.lengths += 1
        self.x.copy_(self.embed[self.tokens])
        h = _rms(self.x, self.layers[0]["attn_norm"], cfg.norm_eps)
        for l, p in enumerate(self.layers):
            a = self._attend_one(self._mm(h, p["wqkv"]), l)
            part, sym = self._partial(B)
            h = self._reduce(self._mm(a, p["wo"], out=part), sym, p["ffn_norm"])
            gu = self._mm(h, p["w_gate_up"])
            if self.cuda:
                from ..ops.infer import swiglu_forward
                g = swiglu_forward(gu, self.Fl)
            else:
                g = F.silu(gu[:, :self.Fl]) * gu[:, self.Fl:]
            part, sym = self._partial(B)
            nxt_norm = self.layers[l + 1]["attn_norm"] if l + 1 < cfg.n_layer else self.norm
            h = self._reduce(self._mm(g, p["w_down"], out=part), sym, nxt_norm)
        self.tokens.copy_(self._pick(h))

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """One decode step for all rows; returns the new tokens [B]."""
        if not self.use_graph or self.sampling is not None or not self._graph_ok:  # NCCL traffic is kept out of graphs
            self._step_body()
            return self.tokens.clone()
        if self._graph is None:
            # warm up outside capture (allocates the symmetric buffers, loads kernels), then capture
            # once; the warm-up step is a real step, so its token is returned
            self._step_body()
            torch.cuda.synchronize(self.dev)
            out = self.tokens.clone()
            self._capture()
            return out
        self.tp.advance_epoch_on_device(self._fused_calls_per_step)
        self._graph.replay()
        return self.tokens.clone()

    def _capture(self) -> None:
        """Captures one step. The captured launches carry the host epochs of the capture pass;
        replays add the device-side base, advanced by one step's worth before every replay."""
        saved = (self.lengths.clone(), self.tokens.clone(), self.x.clone(), [k.clone() for k in self.k_cache], [v.clone() for v in self.v_cache])
        stream = torch.cuda.Stream(self.dev)
        stream.wait_stream(torch.cuda.current_stream(self.dev))
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                self._step_body()
        torch.cuda.current_stream(self.dev).wait_stream(stream)
        # capturing executes nothing, but the host epoch advanced as if one step had run: move the
        # device base back by that step so the first replay lands on the epochs the peers expect
        self.tp.advance_epoch_on_device(-self._fused_calls_per_step)
        self.lengths.copy_(saved[0]); self.tokens.copy_(saved[1]); self.x.copy_(saved[2])
        for dst, src in zip(self.k_cache, saved[3]):
            dst.copy_(src)
        for dst, src in zip(self.v_cache, saved[4]):
            dst.copy_(src)
        self._graph = g

    def close(self) -> None:
        """Drops the captured graph (call before tearing the process group down)."""
        self._graph = None
        if self.cuda:
            torch.cuda.synchronize(self.dev)

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        out = [self.prefill(prompt)]
        for _ in range(max_new_tokens - 1):
            out.append(self.step())
        return torch.stack(out, 1)
