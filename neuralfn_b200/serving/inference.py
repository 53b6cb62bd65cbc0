"""Session-level inference API on top of the resident engine: load an artifact, open sessions
(one engine slot each), prefill / decode with events, truncate / reset / fork / cancel, and
speculative decoding against any proposer.

Speculative step (greedy and sampled): the session keeps one *pending* token - emitted to the
caller but not yet in the KV cache. A step verifies ``[pending] + proposals`` in one batched
pass that leaves the cache untouched, accepts the longest agreeing prefix, commits exactly
those rows, and emits the accepted proposals plus one token chosen by the target itself (the
correction at the first disagreement, or a bonus token when everything agreed). That token
becomes the next pending token, so a correction is never run through the model on its own.
Greedy mode reproduces plain greedy decoding token for token; sampled mode uses rejection
sampling (accept x with probability min(1, p(x)/q(x)), otherwise draw from the normalised
residual max(p - q, 0)), which leaves the output distribution exactly the target's.

Behavioural counterpart: ``neuralfn/native_inference.py`` (GenerationConfig :121-183,
KVCacheConfig :187-251, NativeModelLoadConfig :255-334, NativeInferenceModel :1780-2452,
NativeInferenceSession :2454-3058, ``_decode_speculative`` :2757) and the block transaction of
``resident_glimmer.cpp:2503-2925``.
"""
from __future__ import annotations

import json
import math
import threading
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Callable, Protocol, Sequence

import torch

from .chat import IncrementalTokenDecoder, TextCodec, TokenIdTextCodec, load_text_codec
from .engine import EngineConfig, ResidentEngine, Sampling, resident_inference_abi_version

__all__ = ["InferenceError", "NativeInferenceCapabilities", "GenerationConfig", "KVCacheConfig", "NativeModelLoadConfig", "GenerationEvent",
           "GenerationResult", "Proposer", "NGramProposer", "DraftEngineProposer", "DFlashProposer", "target_embed_and_head", "NativeInferenceModel", "NativeInferenceSession",
           "MANIFEST_NAME", "write_artifact"]

MANIFEST_NAME = "native-execution-manifest.json"
MANIFEST_SCHEMA = "neuralfn_b200.native_execution.v1"


class InferenceError(RuntimeError):
    pass


@dataclass(frozen=True)
class NativeInferenceCapabilities:
    native_inference: bool = True
    resident_inference: bool = True
    lossless_kv_cache: bool = True
    turboquant_kv_cache: bool = False
    function_tools: bool = False
    structured_output: bool = True
    session_state_kinds: tuple[str, ...] = ("tokens",)
    resident_inference_abi: int = 1
    session_prefix_fork: bool = True
    speculative_decoding: bool = True
    dflash_cuda: bool = False
    vision: bool = False
    native_lora: bool = False

    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        d["session_state_kinds"] = list(self.session_state_kinds)
        return d


@dataclass(frozen=True)
class GenerationConfig:
    """One decode request. A temperature of exactly 0 selects strict greedy decoding."""
    max_new_tokens: int = 1
    temperature: float = 0.8
    top_k: int | None = None
    top_p: float = 1.0
    seed: int | None = None
    stop_token_ids: tuple[int, ...] = ()

    def __post_init__(self) -> None:
        if isinstance(self.max_new_tokens, bool) or not isinstance(self.max_new_tokens, int) or self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be an integer >= 0")
        t = float(self.temperature)
        if not math.isfinite(t) or t < 0.0:
            raise ValueError("temperature must be a finite number >= 0")
        object.__setattr__(self, "temperature", t)
        if self.top_k is not None and (isinstance(self.top_k, bool) or not isinstance(self.top_k, int) or self.top_k < 0):
            raise ValueError("top_k must be a non-negative integer or None")
        p = float(self.top_p)
        if not math.isfinite(p) or not 0.0 < p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        object.__setattr__(self, "top_p", p)
        if self.seed is not None and (isinstance(self.seed, bool) or not isinstance(self.seed, int)):
            raise TypeError("seed must be an integer or None")
        object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))

    @property
    def strict_model_compute(self) -> bool:
        return self.temperature == 0.0

    def sampling(self) -> Sampling:
        return Sampling(temperature=self.temperature, top_k=self.top_k or 0, top_p=self.top_p, seed=self.seed or 0)


@dataclass(frozen=True)
class KVCacheConfig:
    mode: str = "auto"                 # auto | off | full | turboquant
    turboquant_profile: str = "mse-3.5"
    cuda_device: int = 0

    def __post_init__(self) -> None:
        if self.mode not in ("auto", "off", "full", "turboquant"):
            raise ValueError("kv cache mode must be auto, off, full or turboquant")
        if self.turboquant_profile not in ("mse-3.5", "qjl-3.5"):
            raise ValueError("turboquant profile must be mse-3.5 or qjl-3.5")


@dataclass(frozen=True)
class NativeModelLoadConfig:
    weight_precision: str = "auto"     # auto | bf16 | k-quant-dynamic | k-quant-17gb
    runtime: str = "auto"              # auto | native-cuda
    cuda_device: int = 0
    vram_reserve_bytes: int | None = None
    context_tokens: int | None = None
    session_count: int = 1
    companion_checkpoints: tuple[str, ...] = ()
    speculative_decoding: str = "auto"  # off | auto | required

    def __post_init__(self) -> None:
        if self.weight_precision not in ("auto", "bf16", "k-quant-dynamic", "k-quant-17gb"):
            raise ValueError("unknown weight_precision")
        if self.runtime not in ("auto", "native-cuda"):
            raise ValueError("runtime must be auto or native-cuda (this framework has no CPU inference runtime)")
        if self.speculative_decoding not in ("off", "auto", "required"):
            raise ValueError("speculative_decoding must be off, auto or required")
        if self.session_count < 1:
            raise ValueError("session_count must be >= 1")


@dataclass(frozen=True)
class GenerationEvent:
    token_id: int
    index: int
    position: int
    text: str = ""
    finish_reason: str | None = None
    committed: bool = True
    kind: str = "token"


@dataclass(frozen=True)
class GenerationResult:
    token_ids: tuple[int, ...]
    text: str
    finish_reason: str
    prompt_tokens: int
    completion_tokens: int
    events: tuple[GenerationEvent, ...] = ()
    cancelled: bool = False
    speculative_proposed_tokens: int = 0
    speculative_accepted_tokens: int = 0
    speculative_rejected_tokens: int = 0
    speculative_target_rows: int = 0
    speculative_assistant_blocks: int = 0
    compute_policy: dict | None = None   # inference_policy.compute_policy_payload of the generation


# ------------------------------------------------------------------------------- proposers


class Proposer(Protocol):
    """``propose(history, k)`` returns up to k token ids that may follow ``history`` (which
    ends with the pending token) and, optionally, the probability the proposer gave each."""

    def propose(self, history: Sequence[int], k: int) -> tuple[list[int], list[float] | None]: ...

    def reset(self) -> None: ...


class NGramProposer:
    """Prompt lookup: finds the most recent earlier occurrence of the last ``n`` tokens and
    proposes what followed it. Needs no second model; effective on repetitive text."""

    def __init__(self, max_ngram: int = 4, min_ngram: int = 1) -> None:
        self.max_ngram, self.min_ngram = max_ngram, min_ngram

    def reset(self) -> None:
        pass

    def propose(self, history: Sequence[int], k: int) -> tuple[list[int], list[float] | None]:
        h = list(history)
        for n in range(min(self.max_ngram, len(h) - 1), self.min_ngram - 1, -1):
            tail = h[-n:]
            for start in range(len(h) - n - 1, -1, -1):
                if h[start:start + n] == tail:
                    follow = h[start + n:start + n + k]
                    if follow:
                        return follow, None
        return [], None


class DraftEngineProposer:
    """A second (smaller) resident engine decodes ``k`` greedy tokens as the proposal. The draft
    keeps its own slot in step with the target's history (truncate + append after a rejection)."""

    def __init__(self, draft: ResidentEngine, slot: int = 0) -> None:
        self.draft, self.slot = draft, slot
        self._have: list[int] = []  # tokens in the draft's cache

    def reset(self) -> None:
        self.draft.release(self.slot)
        self._have = []

    def propose(self, history: Sequence[int], k: int) -> tuple[list[int], list[float] | None]:
        h = [int(t) for t in history]
        ctx, tok = h[:-1], h[-1]
        d, slot = self.draft, self.slot
        common = 0
        while common < min(len(self._have), len(ctx)) and self._have[common] == ctx[common]:
            common += 1
        if common < len(self._have):  # the draft ran ahead on tokens the target rejected
            try:
                d.truncate(slot, common)
                self._have = self._have[:common]
            except Exception:
                d.release(slot)
                self._have = []
        missing = ctx[len(self._have):]
        if missing:
            if self._have:
                d.append(slot, missing)
            else:
                d.prefill(slot, missing)
            self._have = list(ctx)
        out: list[int] = []
        room = d.config.max_seq - 2 - len(self._have)
        for _ in range(max(0, min(k, room))):
            fed = tok
            tok = d.decode({slot: fed})[slot] if self._have else d.prefill(slot, [fed])
            self._have.append(fed)
            out.append(int(tok))
        return out, None


# ----------------------------------------------------------------------------------- model


class DFlashProposer:
    """Block-diffusion draft on the target's own hidden states: the resident engine keeps the residual
    stream after the draft's tap layers for every cached position (``ResidentEngine.enable_taps``); one
    call reads the last ``context_window`` positions of the slot, runs the draft over the block
    [pending token, mask, mask, ...] (bidirectional inside the block, context on the taps) and maps the
    block's hidden states through the target's final norm and head. Block slot i proposes the token at
    distance i from the pending one, so a single draft pass yields ``block_size - 1`` proposals, which
    the engine then verifies in one batched pass.

    ``draft``: a ``tensor.dflash.DFlashDraftModel`` (trained by ``DFlashDistillationTrainer`` or loaded from its
    exported assistant file); ``embed`` [vocab, d] and ``head(hidden) -> logits`` are the target's embedding
    table and its final norm + LM head on the engine's device. Proposals are the draft's arg-max (a point-mass
    proposal distribution: rejection sampling then accepts with the target's own probability).

    Reference: the assistant path of ``neuralfn/csrc/native_gpt2/resident_glimmer_assistant.cpp:1295-1352`` (tap
    context + block through the draft, shared target head) and ``resident_glimmer.cpp:2503-2925`` (propose /
    verify / commit loop)."""

    def __init__(self, engine: ResidentEngine, slot: int, draft, embed: torch.Tensor, head: Callable[[torch.Tensor], torch.Tensor]) -> None:
        cfg = draft.cfg
        if tuple(getattr(engine, "tap_layers", ())) != tuple(cfg.tap_layers):
            raise InferenceError(f"the engine taps layers {getattr(engine, 'tap_layers', ())}, the draft was trained on {tuple(cfg.tap_layers)}")
        self.engine, self.slot, self.draft, self.embed, self.head, self.cfg = engine, slot, draft.eval(), embed, head, cfg
        self.calls = 0

    def reset(self) -> None:
        self.calls = 0

    @torch.no_grad()
    def propose(self, history: Sequence[int], k: int) -> tuple[list[int], list[float] | None]:
        cfg, n = self.cfg, len(history) - 1                     # n tokens are cached; history[-1] is the pending anchor
        if k <= 0 or n <= 0 or n != self.engine.slot_length(self.slot):
            return [], None
        W = min(cfg.context_window, n)
        dev = self.embed.device
        taps = self.engine.read_taps(self.slot, n - W, W).to(self.embed.dtype)[None]                  # [1, W, taps * d]
        ids = torch.full((cfg.block_size,), cfg.mask_token_id, dtype=torch.long, device=dev)
        ids[0] = int(history[-1])
        mask = torch.ones(1, 1, cfg.block_size, W + cfg.block_size, dtype=torch.bool, device=dev)
        hidden = self.draft(self.embed[ids][None, None], taps, mask)[0, 0, 1:]                        # [S - 1, d]
        picks = self.head(hidden).float().argmax(-1)
        self.calls += 1
        return [int(t) for t in picks[:k].tolist()], None


def target_embed_and_head(config: EngineConfig, tensors: dict[str, torch.Tensor], device) -> tuple[torch.Tensor, Callable[[torch.Tensor], torch.Tensor]]:
    """(embedding table, final norm + LM head) of a Llama-family engine's weights, for ``DFlashProposer``. The head applies the
    plain RMS final norm, the (tied or separate) vocabulary projection, the output multiplier and the soft-cap."""
    if config.family != 1:
        raise InferenceError("target_embed_and_head covers the Llama-family tensor names")
    embed = tensors["tok_embeddings"].to(device, torch.bfloat16)
    norm = tensors["norm"].to(device, torch.float32)
    w = embed if config.tie_embeddings else tensors["lm_head"].to(device, torch.bfloat16)
    mult = config.output_multiplier if getattr(config, "output_multiplier", 0.0) > 0 else 1.0
    cap, eps, vocab = float(getattr(config, "logit_softcap", 0.0)), config.norm_eps, config.vocab

    def head(hidden: torch.Tensor) -> torch.Tensor:
        h = hidden.float()
        h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * norm
        logits = (h.to(w.dtype) @ w.T).float()[..., :vocab] * mult
        return cap * torch.tanh(logits / cap) if cap > 0 else logits

    return embed, head


def write_artifact(out_dir: str | Path, config: EngineConfig, tensors: dict[str, torch.Tensor], *, chat_template: str | None = None,
                   codec: str | None = None, stop_token_ids: Sequence[int] = (), extra: dict | None = None) -> Path:
    """Writes a loadable artifact directory: manifest + one named-tensor file."""
    from ..checkpoint.named import write_named_tensors
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    write_named_tensors(out / "weights.nfn", {k: v.detach().to(torch.bfloat16).cpu().contiguous() for k, v in tensors.items()})
    manifest = {"schema": MANIFEST_SCHEMA, "engine": asdict(config), "weights": "weights.nfn", "chat_template": chat_template,
                "text_codec": codec, "stop_token_ids": list(stop_token_ids), "resident_inference_abi": resident_inference_abi_version()}
    manifest.update(extra or {})
    (out / MANIFEST_NAME).write_text(json.dumps(manifest, indent=2, sort_keys=True), encoding="utf-8")
    return out


class NativeInferenceModel:
    """One resident engine plus its session table."""

    def __init__(self, engine: ResidentEngine, *, codec: TextCodec | None = None, manifest: dict | None = None, artifact_root: Path | None = None,
                 load_config: NativeModelLoadConfig | None = None, proposer_factory: Callable[[], Proposer] | None = None) -> None:
        self.engine = engine
        self.codec = codec or TokenIdTextCodec()
        self.manifest = manifest or {}
        self.artifact_root = artifact_root
        self.load_config = load_config or NativeModelLoadConfig(session_count=engine.config.max_batch)
        self.proposer_factory = proposer_factory
        self._free = list(range(engine.config.max_batch))[::-1]
        self._sessions: dict[int, "NativeInferenceSession"] = {}
        self._lazy: list["NativeInferenceSession"] = []       # forks that have not needed a slot of their own yet
        self._lock = threading.RLock()
        self._closed = False
        self._counters = {"prefill_tokens": 0, "decode_tokens": 0, "sessions_created": 0, "forks": 0}

    # -- loading ---------------------------------------------------------------------------
    @classmethod
    def load(cls, artifact_dir: str | Path, load_config: NativeModelLoadConfig | None = None, **kw) -> "NativeInferenceModel":
        root = Path(artifact_dir)
        path = root / MANIFEST_NAME
        if not path.is_file():
            raise InferenceError(f"{root} has no {MANIFEST_NAME}")
        manifest = json.loads(path.read_text(encoding="utf-8"))
        if manifest.get("schema") != MANIFEST_SCHEMA:
            raise InferenceError(f"unsupported manifest schema {manifest.get('schema')!r}")
        lc = load_config or NativeModelLoadConfig()
        fields = dict(manifest["engine"])
        fields["max_batch"] = max(int(fields.get("max_batch", 1)), lc.session_count)
        if lc.context_tokens:
            fields["max_seq"] = min(int(fields["max_seq"]), int(lc.context_tokens))
        cfg = EngineConfig(**fields)
        if torch.cuda.is_available():
            free, _total = torch.cuda.mem_get_info(lc.cuda_device)
            need = cls.estimate_device_bytes(cfg)
            if need + (lc.vram_reserve_bytes or 0) > free:
                raise InferenceError(f"artifact needs ~{need >> 20} MiB on the device, {free >> 20} MiB free (reserve {lc.vram_reserve_bytes or 0})")
        engine = ResidentEngine(cfg, device=lc.cuda_device)
        from ..checkpoint.named import read_named_tensors
        engine.load_named_tensors(read_named_tensors(root / manifest["weights"])[0])
        codec = load_text_codec(manifest.get("text_codec"), root)
        return cls(engine, codec=codec, manifest=manifest, artifact_root=root, load_config=lc, **kw)

    def attach_dflash(self, assistant, *, target_tensors: dict[str, torch.Tensor] | None = None) -> None:
        """Makes a DFlash (block-diffusion) draft the model's speculative proposer. ``assistant``: the file written by
        ``DFlashDistillationTrainer.export_native_assistant`` (or a ``DFlashDraftModel``). Must be called before the first
        decode step: the engine starts keeping the tapped hidden states from then on. ``target_tensors`` default to the
        artifact's own weights (embedding table, final norm, head)."""
        from ..tensor.dflash import DFlashConfig, DFlashDraftModel
        dev = torch.device("cuda", self.engine.device)
        if isinstance(assistant, (str, Path)):
            from ..checkpoint.named import read_named_tensors
            tensors, meta, _sha = read_named_tensors(assistant)
            if meta.get("kind") != "dflash_assistant":
                raise InferenceError(f"{assistant} is not a DFlash assistant file")
            raw = dict(meta["config"])
            raw["tap_layers"] = tuple(raw.get("tap_layers", ()))
            cfg = DFlashConfig(**{k: v for k, v in raw.items() if k in DFlashConfig.__dataclass_fields__})
            draft = DFlashDraftModel(cfg, self.engine.config.d_model)
            draft.load_state_dict({k: v.float() for k, v in tensors.items()})
        else:
            draft = assistant
        if target_tensors is None:
            if self.artifact_root is None or not self.manifest:
                raise InferenceError("attach_dflash needs target_tensors for a model that was not loaded from an artifact directory")
            from ..checkpoint.named import read_named_tensors
            target_tensors = read_named_tensors(self.artifact_root / self.manifest["weights"])[0]
        c = self.engine.config
        shaped = {k: (v.view(-1, c.d_model) if k in ("tok_embeddings", "lm_head") and v.dim() == 1 else v) for k, v in target_tensors.items()
                  if k in ("tok_embeddings", "lm_head", "norm")}
        embed, head = target_embed_and_head(c, shaped, dev)
        self.engine.enable_taps(draft.cfg.tap_layers)
        self._dflash = (draft.to(dev).to(torch.bfloat16), embed, head)

    def dflash_proposer(self, session: "NativeInferenceSession") -> "DFlashProposer":
        if getattr(self, "_dflash", None) is None:
            raise InferenceError("no DFlash assistant is attached (attach_dflash)")
        draft, embed, head = self._dflash
        return DFlashProposer(self.engine, session.slot, draft, embed, head)

    @staticmethod
    def estimate_device_bytes(cfg: EngineConfig) -> int:
        """Weights + KV caches + activations of an engine with this configuration."""
        hd, kvw = cfg.head_dim, cfg.n_kv_head * cfg.head_dim
        att = cfg.n_head * hd
        per_layer = (att + 2 * kvw) * cfg.d_model + att * cfg.d_model + (3 if cfg.family == 1 else 2) * cfg.d_model * cfg.d_ff
        weights = 2 * (cfg.n_layer * per_layer + cfg.padded_vocab * cfg.d_model * (1 if cfg.tie_embeddings or cfg.family == 0 else 2))
        caps = [min(cfg.window, cfg.max_seq) if (cfg.window > 0 and (cfg.global_every <= 0 or (l + 1) % cfg.global_every)) else cfg.max_seq
                for l in range(cfg.n_layer)]
        kv = sum(2 * 2 * cfg.max_batch * kvw * c for c in caps)
        rows = max(cfg.max_seq, cfg.max_batch)
        act = 2 * rows * (3 * cfg.d_model + att + 2 * kvw + att + 3 * cfg.d_ff) + 2 * cfg.max_batch * cfg.padded_vocab
        return int(weights + kv + act)

    # -- properties ------------------------------------------------------------------------
    @property
    def capabilities(self) -> NativeInferenceCapabilities:
        return NativeInferenceCapabilities(resident_inference_abi=resident_inference_abi_version(),
                                           speculative_decoding=self.load_config.speculative_decoding != "off")

    @property
    def closed(self) -> bool:
        return self._closed

    def _open(self) -> None:
        if self._closed:
            raise InferenceError("the model is closed")

    # -- sessions --------------------------------------------------------------------------
    def create_session(self, seed: int | None = None) -> "NativeInferenceSession":
        with self._lock:
            self._open()
            if not self._free:
                raise InferenceError("every session slot is in use")
            slot = self._free.pop()
            s = NativeInferenceSession(self, slot, seed)
            self._sessions[slot] = s
            self._counters["sessions_created"] += 1
            return s

    def fork_session(self, session: "NativeInferenceSession", prefix_tokens: int | None = None, seed: int | None = None, *,
                     lazy: bool = True) -> "NativeInferenceSession":
        """A new session that starts with the first ``prefix_tokens`` cached tokens of ``session``. The child caches all but
        the last prefix token and keeps that one pending: running it again is what gives the child valid logits for its own
        next token.

        Copy-on-write at whole-prefix granularity: the child is created WITHOUT a cache slot and reads the parent's rows; the
        device-to-device copy happens when the child first needs to write (any prefill / decode / logits call), or when the
        parent is about to invalidate the shared rows (truncate below them, reset, close, or any append while the engine has
        sliding-window caches that could wrap). A parent that closes hands its slot to its first unused child instead of copying.
        So a fork costs nothing until it is used, and more forks than cache slots may exist. ``lazy=False`` copies at once."""
        with self._lock:
            self._require_owned(session)
            n = session.cached_tokens if prefix_tokens is None else int(prefix_tokens)
            if n < 0 or n > session.cached_tokens:
                raise InferenceError("fork prefix longer than the cached tokens of the source session")
            self._open()
            child = NativeInferenceSession(self, None, seed)
            child._tokens = list(session._tokens[:max(n - 1, 0)])
            child._pending = session._tokens[n - 1] if n >= 1 else None
            self._counters["forks"] += 1
            self._counters["sessions_created"] += 1
            if len(child._tokens) > 0:
                root = session._origin[0] if session._slot is None else session      # an unused fork forwards to ITS source
                child._origin = (root, len(child._tokens))
                root._dependants.append(child)
            self._lazy.append(child)
            if not lazy:
                child.slot  # noqa: B018 - materialises
            return child

    def _materialise(self, child: "NativeInferenceSession") -> int:
        """Gives an unused fork its own slot and copies the shared rows into it."""
        with self._lock:
            if child._slot is not None:
                return child._slot
            if child.closed:
                raise InferenceError("the session is closed")
            if not self._free:
                raise InferenceError("every session slot is in use")
            slot = self._free.pop()
            origin = child._origin
            try:
                if origin is not None:
                    self.engine.fork(origin[0].slot, slot, origin[1])
                    self._counters["fork_copies"] = self._counters.get("fork_copies", 0) + 1
            except Exception:
                self._free.append(slot)
                raise
            if origin is not None and child in origin[0]._dependants:
                origin[0]._dependants.remove(child)
            child._origin, child._slot = None, slot
            if child in self._lazy:
                self._lazy.remove(child)
            self._sessions[slot] = child
            return slot

    def _detach_dependants(self, session: "NativeInferenceSession", keep_rows: int | None = None, *, closing: bool = False) -> None:
        """Before ``session`` invalidates cached rows: unused forks that read rows past ``keep_rows`` (all of them when None)
        get their own copy. When the session is closing, the fork that reads the most rows adopts its slot instead (the slot
        is shortened to that prefix, nothing is copied) and the other forks read from the adopter from then on."""
        with self._lock:
            if closing and session._dependants and session._slot is not None and self._sessions.get(session._slot) is session:
                heir = max(session._dependants, key=lambda c: c._origin[1])
                slot, rows = session._slot, heir._origin[1]
                if rows < self.engine.slot_length(slot):
                    self.engine.truncate(slot, rows)
                for other in session._dependants:
                    if other is not heir:
                        other._origin = (heir, other._origin[1])
                        heir._dependants.append(other)
                session._dependants = []
                heir._origin, heir._slot = None, slot
                self._lazy.remove(heir)
                self._sessions[slot] = heir
                session._slot_given_away = True
                self._counters["fork_adoptions"] = self._counters.get("fork_adoptions", 0) + 1
                return
            for child in list(session._dependants):
                if keep_rows is not None and child._origin[1] <= keep_rows:
                    continue
                self._materialise(child)

    def _require_owned(self, session: "NativeInferenceSession") -> None:
        if session.closed or session.model is not self or (session._slot is None and session not in self._lazy) or \
                (session._slot is not None and self._sessions.get(session._slot) is not session):
            raise InferenceError("the session does not belong to this model (or is closed)")

    def _discard(self, session: "NativeInferenceSession") -> None:
        with self._lock:
            self._detach_dependants(session, closing=True)
            if session._slot is None:
                if session._origin is not None and session in session._origin[0]._dependants:
                    session._origin[0]._dependants.remove(session)
                if session in self._lazy:
                    self._lazy.remove(session)
                return
            if getattr(session, "_slot_given_away", False):
                return
            if self._sessions.get(session._slot) is session:
                del self._sessions[session._slot]
                self.engine.release(session._slot)
                self._free.append(session._slot)

    # convenience forwards (the reference exposes both spellings)
    def prefill(self, session, token_ids):
        return session.prefill(token_ids)

    def decode(self, session, config=None, **kw):
        return session.decode(config, **kw)

    def current_logits(self, session):
        return session.current_logits()

    def truncate(self, session, token_count):
        return session.truncate(token_count)

    def reset(self, session):
        return session.reset()

    def cancel(self, session):
        return session.cancel()

    def stats(self) -> dict[str, Any]:
        with self._lock:
            return {**self._counters, "sessions_open": len(self._sessions) + len(self._lazy), "unused_forks": len(self._lazy),
                    "session_slots": self.engine.config.max_batch,
                    "device_bytes": self.engine.device_bytes, "kernel_launches": self.engine.launches,
                    "sessions": {slot: s.stats() for slot, s in self._sessions.items()}}

    def close(self) -> None:
        with self._lock:
            if self._closed:
                return
            for s in list(self._lazy) + list(self._sessions.values()):
                s.close()
            self.engine.close()
            self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class NativeInferenceSession:
    """One sequence. ``token_ids`` is everything the caller has seen (prompt + emitted tokens);
    the KV cache may lag it by the single pending token."""

    def __init__(self, model: NativeInferenceModel, slot: int | None, seed: int | None) -> None:
        self.model, self._slot, self.seed = model, slot, seed
        self._origin: tuple["NativeInferenceSession", int] | None = None   # an unused fork: (session whose rows it reads, how many)
        self._dependants: list["NativeInferenceSession"] = []              # unused forks that read this session's rows
        self._tokens: list[int] = []      # tokens in the KV cache
        self._pending: int | None = None  # seen by the caller but not cached
        self._cancel = threading.Event()
        self._closed = False
        self._stats = {"prefill_tokens": 0, "decode_tokens": 0, "speculative_proposed_tokens": 0, "speculative_accepted_tokens": 0,
                       "speculative_rejected_tokens": 0, "speculative_target_rows": 0, "speculative_assistant_blocks": 0,
                       "decode_seconds": 0.0, "prefill_seconds": 0.0}
        self._rng = torch.Generator().manual_seed(seed if seed is not None else 0x5EED)
        self._next_greedy: int | None = None  # the engine's own pick after the last cached token

    # -- state -----------------------------------------------------------------------------
    @property
    def slot(self) -> int:
        """The engine slot; an unused fork gets one (and its copy of the shared rows) on first access."""
        return self._slot if self._slot is not None else self.model._materialise(self)

    @property
    def shares_cache(self) -> bool:
        """True while this fork still reads its source's rows (nothing has been copied)."""
        return self._slot is None and self._origin is not None

    def _before_append(self) -> None:
        """Appends keep every earlier row, except where a sliding-window cache can wrap over them."""
        if self._dependants and self.model.engine.config.window > 0:
            self.model._detach_dependants(self)

    @property
    def token_ids(self) -> tuple[int, ...]:
        return tuple(self._tokens) + (() if self._pending is None else (self._pending,))

    @property
    def cached_tokens(self) -> int:
        return len(self._tokens)

    @property
    def cancelled(self) -> bool:
        return self._cancel.is_set()

    @property
    def closed(self) -> bool:
        return self._closed

    def _usable(self) -> None:
        if self._closed:
            raise InferenceError("the session is closed")
        self.model._open()

    def _advance(self, token: int, sampling: Sampling | None) -> int:
        """Runs one token through the engine (appending it to the cache); returns the engine's pick."""
        eng = self.model.engine
        self._before_append()
        if not self._tokens:
            return eng.prefill(self.slot, [token], sampling)
        return eng.decode({self.slot: token}, sampling)[self.slot]

    def _flush_pending(self) -> None:
        """Runs the pending token through the model so that cache and history agree."""
        if self._pending is None:
            return
        self._next_greedy = self._advance(self._pending, None)
        self._tokens.append(self._pending)
        self._pending = None

    # -- operations ------------------------------------------------------------------------
    def prefill(self, token_ids: Sequence[int]) -> dict[str, int]:
        """Appends prompt tokens at the current position. Returns token counts."""
        self._usable()
        ids = [int(t) for t in token_ids]
        eng = self.model.engine
        if not ids:
            return {"prompt_tokens": 0, "total_tokens": len(self.token_ids)}
        if any(t < 0 or t >= eng.config.vocab for t in ids):
            raise InferenceError("token id outside the vocabulary")
        if len(self.token_ids) + len(ids) >= eng.config.max_seq:
            raise InferenceError("the prompt does not fit the context window")
        t0 = time.perf_counter()
        with self.model._lock:
            self._flush_pending()
            self._before_append()
            if not self._tokens:
                self._next_greedy = eng.prefill(self.slot, ids)
            else:
                self._next_greedy = eng.append(self.slot, ids)
            self._tokens.extend(ids)
        self._stats["prefill_tokens"] += len(ids)
        self._stats["prefill_seconds"] += time.perf_counter() - t0
        self.model._counters["prefill_tokens"] += len(ids)
        return {"prompt_tokens": len(ids), "total_tokens": len(self._tokens)}

    def current_logits(self) -> torch.Tensor:
        """fp32 logits for the token that follows everything the caller has seen."""
        self._usable()
        with self.model._lock:
            if not self._tokens and self._pending is None:
                raise InferenceError("nothing has been prefilled")
            self._flush_pending()
            return self.model.engine.last_logits(self.slot)

    def truncate(self, token_count: int) -> None:
        self._usable()
        n = int(token_count)
        if n < 0 or n > len(self.token_ids):
            raise InferenceError("token_count outside [0, current length]")
        with self.model._lock:
            every = list(self.token_ids)
            if n == len(every):
                return
            self.model._detach_dependants(self, keep_rows=max(n - 1, 0))
            if n == 0:
                self.model.engine.release(self.slot)
                self._tokens, self._pending, self._next_greedy = [], None, None
                return
            # keep n - 1 tokens cached and make the n-th the pending one: running it again is what
            # yields the logits that follow the shortened history
            if n - 1 < len(self._tokens):
                self.model.engine.truncate(self.slot, n - 1)
            self._tokens, self._pending, self._next_greedy = every[:n - 1], every[n - 1], None

    def reset(self) -> None:
        self._usable()
        with self.model._lock:
            self.model._detach_dependants(self)
            self.model.engine.release(self.slot)
            self._tokens, self._pending, self._next_greedy = [], None, None
            self._cancel.clear()

    def cancel(self) -> None:
        """Asks a running ``decode`` to stop at the next token boundary."""
        self._cancel.set()

    def stats(self) -> dict[str, Any]:
        d = dict(self._stats)
        d.update(cached_tokens=len(self._tokens), total_tokens=len(self.token_ids))
        if d["decode_seconds"] > 0:
            d["decode_tokens_per_second"] = d["decode_tokens"] / d["decode_seconds"]
        return d

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            self.model._discard(self)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- decoding --------------------------------------------------------------------------
    def decode(self, config: GenerationConfig | None = None, *, on_event: Callable[[GenerationEvent], None] | None = None,
               proposer: Proposer | None = None, speculative_tokens: int = 15,
               allowed_tokens: Callable[[Sequence[int]], Sequence[int]] | None = None) -> GenerationResult:
        """Generates up to ``max_new_tokens`` tokens. With a proposer (or the model's proposer
        factory and speculative decoding not "off") blocks are verified speculatively.
        ``allowed_tokens(history)`` restricts every choice to a token subset (constrained
        decoding; implies greedy, non-speculative stepping)."""
        self._usable()
        cfg = config or GenerationConfig()
        if not self._tokens and self._pending is None:
            raise InferenceError("prefill the session before decoding")
        spec_mode = self.model.load_config.speculative_decoding
        if proposer is None and getattr(self.model, "_dflash", None) is not None and spec_mode != "off":
            proposer = self.model.dflash_proposer(self)
        if proposer is None and self.model.proposer_factory is not None and spec_mode != "off":
            proposer = self.model.proposer_factory()
        if spec_mode == "required" and proposer is None:
            raise InferenceError("speculative decoding is required but no proposer is available")
        if allowed_tokens is not None:
            proposer = None
        self._cancel.clear()
        prompt_tokens = len(self.token_ids)
        before = dict(self._stats)
        t0 = time.perf_counter()
        out: list[int] = []
        events: list[GenerationEvent] = []
        finish = "length"
        decoder = IncrementalTokenDecoder(self.model.codec)

        def emit(tok: int) -> bool:
            """Records one token; returns True when generation must stop."""
            nonlocal finish
            out.append(tok)
            stop = tok in cfg.stop_token_ids
            if stop:
                finish = "stop"
            ev = GenerationEvent(tok, len(out) - 1, prompt_tokens + len(out) - 1, decoder.push(tok), "stop" if stop else None)
            events.append(ev)
            if on_event:
                on_event(ev)
            return stop or len(out) >= cfg.max_new_tokens

        from ..inference_policy import compute_policy_payload, inference_execution
        with inference_execution(cfg.temperature, native_engine=True) as policy, self.model._lock:
            done = cfg.max_new_tokens == 0
            while not done:
                if self._cancel.is_set():
                    finish = "cancelled"
                    break
                if len(self.token_ids) + 1 >= self.model.engine.config.max_seq:
                    finish = "length"
                    break
                if proposer is not None:
                    done = self._speculative_step(cfg, proposer, speculative_tokens, emit, cfg.max_new_tokens - len(out))
                else:
                    done = self._plain_step(cfg, emit, allowed_tokens)
        dt = time.perf_counter() - t0
        self._stats["decode_tokens"] += len(out)
        self._stats["decode_seconds"] += dt
        self.model._counters["decode_tokens"] += len(out)
        if events and events[-1].finish_reason is None:
            last = events[-1]
            events[-1] = GenerationEvent(last.token_id, last.index, last.position, last.text, finish, last.committed, last.kind)
        d = {k: self._stats[k] - before[k] for k in before if k.startswith("speculative")}
        return GenerationResult(tuple(out), self.model.codec.decode(out), finish, prompt_tokens, len(out), tuple(events), finish == "cancelled", **d,
                                compute_policy=compute_policy_payload(policy, backend="resident-engine-sm100a"))

    def _plain_step(self, cfg: GenerationConfig, emit, allowed_tokens) -> bool:
        """One token without speculation."""
        eng = self.model.engine
        if allowed_tokens is not None:
            self._flush_pending()
            logits = eng.last_logits(self.slot)
            allowed = list(allowed_tokens(self.token_ids))
            if not allowed:
                raise InferenceError("the constraint allows no token here")
            idx = torch.tensor(allowed, dtype=torch.long)
            tok = int(idx[int(torch.argmax(logits[idx]))])
            self._next_greedy = None
        elif self._pending is None:
            # the token after the cached history: the greedy pick is known; sampling needs the logits
            if cfg.strict_model_compute and self._next_greedy is not None:
                tok = self._next_greedy
            else:
                tok = self._sample(eng.last_logits(self.slot), cfg)
            self._next_greedy = None
        else:
            s = cfg.sampling()
            if cfg.seed is None and not cfg.strict_model_compute:
                s = Sampling(temperature=s.temperature, top_k=s.top_k, top_p=s.top_p,
                             seed=int(torch.randint(0, 2 ** 31 - 1, (1,), generator=self._rng)))
            tok = self._advance(self._pending, s)
            self._tokens.append(self._pending)
            self._pending = None
        self._pending = tok
        return emit(tok)

    def _probs(self, logits: torch.Tensor, cfg: GenerationConfig) -> torch.Tensor:
        """The distribution sampling draws from: temperature, then top-k, then top-p."""
        z = logits.double() / max(cfg.temperature, 1e-6)
        if cfg.top_k:
            kth = torch.topk(z, min(cfg.top_k, z.numel())).values[-1]
            z = torch.where(z < kth, torch.full_like(z, -math.inf), z)
        p = torch.softmax(z, 0)
        if cfg.top_p < 1.0:
            sp, si = torch.sort(p, descending=True)
            keep = (torch.cumsum(sp, 0) - sp) < cfg.top_p
            mask = torch.zeros_like(p, dtype=torch.bool)
            mask[si[keep]] = True
            p = torch.where(mask, p, torch.zeros_like(p))
            p = p / p.sum()
        return p

    def _sample(self, logits: torch.Tensor, cfg: GenerationConfig) -> int:
        if cfg.strict_model_compute:
            return int(torch.argmax(logits))
        return int(torch.multinomial(self._probs(logits, cfg).float(), 1, generator=self._rng))

    def _speculative_step(self, cfg: GenerationConfig, proposer: Proposer, k: int, emit, room: int) -> bool:
        eng = self.model.engine
        if self._pending is None or not self._tokens:
            # right after a prefill (one target-only anchor token), or nothing cached to verify against
            return self._plain_step(cfg, emit, None)
        rows_cap = getattr(eng, "_verify_rows", 0) or 17
        budget = min(k, room - 1, eng.config.max_seq - 2 - len(self.token_ids), rows_cap - 1)
        props, q = proposer.propose(self.token_ids, budget) if budget > 0 else ([], None)
        props = [int(t) for t in props[:max(budget, 0)]]
        self._before_append()
        block = [self._pending] + props
        picks = eng.verify({self.slot: block})[self.slot]
        st = self._stats
        st["speculative_assistant_blocks"] += 1
        st["speculative_proposed_tokens"] += len(props)
        st["speculative_target_rows"] += len(block)
        accepted, final = 0, None
        if cfg.strict_model_compute:
            while accepted < len(props) and picks[accepted] == props[accepted]:
                accepted += 1
            final = picks[accepted]
        else:
            for i, x in enumerate(props):
                p = self._probs(eng.verify_logits(self.slot, i), cfg)
                qx = 1.0 if q is None else max(float(q[i]), 1e-12)
                if float(torch.rand((), generator=self._rng)) < min(1.0, float(p[x]) / qx):
                    accepted += 1
                    continue
                resid = p.clone()
                resid[x] = max(0.0, float(p[x]) - (1.0 if q is None else float(q[i])))
                total = float(resid.sum())
                final = int(torch.multinomial((resid / total).float(), 1, generator=self._rng)) if total > 0 else int(torch.argmax(p))
                break
            if final is None:
                final = self._sample(eng.verify_logits(self.slot, len(props)), cfg)
        st["speculative_accepted_tokens"] += accepted
        st["speculative_rejected_tokens"] += len(props) - accepted
        # report first, commit afterwards: when the request ends on an accepted proposal only the
        # rows the caller has seen are appended, so cache and history always agree
        stopped_at = None
        for j, t in enumerate(props[:accepted]):
            if emit(t):
                stopped_at = j
                break
        if stopped_at is not None:
            rows = 1 + stopped_at + 1
            eng.commit({self.slot: rows})
            self._tokens.extend(block[:rows])
            self._pending, self._next_greedy = None, None
            return True
        eng.commit({self.slot: accepted + 1})
        self._tokens.extend(block[:accepted + 1])
        self._pending, self._next_greedy = final, None
        return emit(final)
