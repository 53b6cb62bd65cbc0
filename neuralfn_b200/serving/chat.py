"""Text codecs and chat renderers of the serving stack.

Codecs turn text into token ids and back (``TokenIdTextCodec`` for raw ids, ``ByteTextCodec``
for byte-level vocabularies, ``TiktokenTextCodec`` and ``HuggingFaceTokenizerJSONCodec`` when
their libraries and vocabulary files are present). Renderers turn a list of chat messages
into the prompt string a model family expects: plain role headers, a placeholder form, and
the Muse-Glimmer ATEM envelope (``<|start|>role<|message|>...<|eot|>``, assistant messages
addressed ``to=user`` or ``to=self``; text addressed to ``self`` is private reasoning and is
never shown or fed back).

Behavioural counterpart: ``neuralfn/native_chat.py`` (codecs :125-396, renderers :397-577,
response parsing :1065-1131).
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from datetime import date
from pathlib import Path
from typing import Iterable, Sequence

__all__ = ["ChatConfigurationError", "ChatMessage", "AssistantResponse", "TextCodec", "TokenIdTextCodec", "ByteTextCodec",
           "TiktokenTextCodec", "HuggingFaceTokenizerJSONCodec", "IncrementalTokenDecoder", "ChatRenderer", "PlainRolesRenderer",
           "PlaceholderChatRenderer", "MuseGlimmerATEMRenderer", "ATEM_SPECIAL_TOKENS", "parse_assistant_response",
           "strip_text_delimiters", "load_text_codec", "resolve_chat_renderer"]

CHAT_ROLES = ("system", "developer", "user", "assistant", "tool")

ATEM_SPECIAL_TOKENS = {
    "bos": "<|begin_of_text|>", "eos": "<|end_of_text|>", "eom": "<|eom|>", "eot": "<|eot|>", "pad": "<|finetune_right_pad|>",
    "start": "<|start|>", "message": "<|message|>", "image_start": "<|image_start|>", "image_end": "<|image_end|>",
    "video_start": "<|vid_start|>", "video_end": "<|vid_end|>", "video_frame_separator": "<|vid_frame_separator|>",
    "image": "<|image|>", "video": "<|video|>", "patch": "<|patch|>", "dflash_mask": "<|reserved_special_token_1818|>",
}


class ChatConfigurationError(ValueError):
    pass


@dataclass(frozen=True)
class ChatMessage:
    role: str
    content: str
    name: str | None = None
    tool_call_id: str | None = None

    def __post_init__(self) -> None:
        if self.role not in CHAT_ROLES:
            raise ChatConfigurationError(f"unknown chat role {self.role!r}")
        if not isinstance(self.content, str):
            raise TypeError("message content must be a string")


@dataclass(frozen=True)
class AssistantResponse:
    visible_text: str
    raw_text: str
    reasoning_text: str = ""
    used_channel_protocol: bool = False
    final_channel_complete: bool = True


# ---------------------------------------------------------------------------------- codecs


class TextCodec:
    name = "abstract"
    vocab_size: int | None = None

    def encode(self, text: str) -> list[int]:
        raise NotImplementedError

    def decode(self, token_ids: Iterable[int]) -> str:
        raise NotImplementedError


class TokenIdTextCodec(TextCodec):
    """Whitespace- or comma-separated decimal ids; the fallback when no vocabulary is known."""
    name = "token-ids"

    def encode(self, text: str) -> list[int]:
        parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
        try:
            ids = [int(p) for p in parts]
        except ValueError as exc:
            raise ChatConfigurationError("token-id prompts hold decimal integers only") from exc
        if any(i < 0 for i in ids):
            raise ChatConfigurationError("token ids are non-negative")
        return ids

    def decode(self, token_ids: Iterable[int]) -> str:
        return " ".join(str(int(t)) for t in token_ids)


class ByteTextCodec(TextCodec):
    """UTF-8 bytes as tokens ``offset + byte`` (byte-level models, constrained decoding tests)."""
    name = "utf8-bytes"

    def __init__(self, offset: int = 0, vocab_size: int | None = None) -> None:
        self.offset = offset
        self.vocab_size = vocab_size or offset + 256

    def encode(self, text: str) -> list[int]:
        return [self.offset + b for b in text.encode("utf-8")]

    def decode(self, token_ids: Iterable[int]) -> str:
        data = bytes(t - self.offset for t in token_ids if 0 <= t - self.offset < 256)
        return data.decode("utf-8", errors="replace")


class TiktokenTextCodec(TextCodec):
    name = "tiktoken"

    def __init__(self, encoding: str = "gpt2") -> None:
        try:
            import tiktoken  # type: ignore
        except ImportError as exc:  # pragma: no cover - depends on the environment
            raise ChatConfigurationError("tiktoken is not installed") from exc
        self._enc = tiktoken.get_encoding(encoding)
        self.vocab_size = self._enc.n_vocab

    def encode(self, text: str) -> list[int]:
        return list(self._enc.encode(text, allowed_special="all"))

    def decode(self, token_ids: Iterable[int]) -> str:
        return self._enc.decode(list(token_ids))


class HuggingFaceTokenizerJSONCodec(TextCodec):
    """A ``tokenizer.json`` through the ``tokenizers`` library. Special tokens in the text are
    parsed as such; no BOS is added by the codec (renderers write it) so it is never doubled."""
    name = "hf-tokenizer-json"

    def __init__(self, path: str | Path) -> None:
        try:
            from tokenizers import Tokenizer  # type: ignore
        except ImportError as exc:  # pragma: no cover
            raise ChatConfigurationError("the tokenizers library is not installed") from exc
        self._tok = Tokenizer.from_file(str(path))
        self.vocab_size = self._tok.get_vocab_size(with_added_tokens=True)

    def encode(self, text: str) -> list[int]:
        return list(self._tok.encode(text, add_special_tokens=False).ids)

    def decode(self, token_ids: Iterable[int]) -> str:
        return self._tok.decode(list(token_ids), skip_special_tokens=False)

    def token_id(self, token: str) -> int | None:
        return self._tok.token_to_id(token)


class IncrementalTokenDecoder:
    """Streams text: returns only the characters that became stable after each new token
    (a multi-byte character split across tokens is held back until it is whole)."""

    def __init__(self, codec: TextCodec) -> None:
        self.codec = codec
        self.ids: list[int] = []
        self.emitted = ""

    def push(self, token_id: int) -> str:
        self.ids.append(int(token_id))
        text = self.codec.decode(self.ids)
        if text.endswith("�"):
            return ""
        if not text.startswith(self.emitted):  # a tokenizer that rewrites earlier text: resynchronise
            self.emitted = text
            return ""
        delta = text[len(self.emitted):]
        self.emitted = text
        return delta


def load_text_codec(spec: str | None, artifact_dir: str | Path | None = None) -> TextCodec:
    """``None``/"token-ids", "bytes[:offset]", "tiktoken[:encoding]", or a path to a
    ``tokenizer.json``; with an artifact directory a ``tokenizer.json`` inside it wins."""
    if artifact_dir is not None and (spec is None or spec == "auto"):
        cand = Path(artifact_dir) / "tokenizer.json"
        if cand.is_file():
            return HuggingFaceTokenizerJSONCodec(cand)
    if spec in (None, "auto", "token-ids"):
        return TokenIdTextCodec()
    if spec.startswith("bytes"):
        return ByteTextCodec(int(spec.split(":", 1)[1]) if ":" in spec else 0)
    if spec.startswith("tiktoken"):
        return TiktokenTextCodec(spec.split(":", 1)[1] if ":" in spec else "gpt2")
    if Path(spec).is_file():
        return HuggingFaceTokenizerJSONCodec(spec)
    raise ChatConfigurationError(f"unknown text codec {spec!r}")


# ------------------------------------------------------------------------------- renderers


class ChatRenderer:
    name = "role-headers"
    stop_delimiters: tuple[str, ...] = ("<|user|>", "<|system|>", "<|assistant|>", "<|tool|>", "<|developer|>")

    def render(self, messages: Sequence[ChatMessage], *, include_assistant_prompt: bool = True) -> str:
        out = [f"<|{m.role if m.name is None else m.role + ':' + m.name}|>\n{m.content}\n" for m in messages]
        if include_assistant_prompt:
            out.append("<|assistant|>\n")
        return "".join(out)


class PlainRolesRenderer(ChatRenderer):
    name = "plain-roles"
    stop_delimiters = ("\nUser:", "\nSystem:", "\nAssistant:", "\nTool:")

    def render(self, messages: Sequence[ChatMessage], *, include_assistant_prompt: bool = True) -> str:
        out = [f"{m.role.capitalize()}: {m.content}\n" for m in messages]
        if include_assistant_prompt:
            out.append("Assistant:")
        return "".join(out)


class PlaceholderChatRenderer(ChatRenderer):
    """For artifacts without a reviewed template: the last user message only."""
    name = "placeholder"

    def render(self, messages: Sequence[ChatMessage], *, include_assistant_prompt: bool = True) -> str:
        users = [m.content for m in messages if m.role == "user"]
        if not users:
            raise ChatConfigurationError("the placeholder renderer needs a user message")
        return users[-1] + ("\n<|assistant|>\n" if include_assistant_prompt else "")


class MuseGlimmerATEMRenderer(ChatRenderer):
    """Text-only ATEM envelope: system / user / assistant string messages. Tool roles, named
    messages and media parts are refused rather than guessed."""
    name = "muse-glimmer-atem-v1"
    stop_delimiters = ("<|eot|>", "<|end_of_text|>")

    def __init__(self, *, reasoning_strength: str = "high", knowledge_cutoff: str = "2026-01-04", current_date: str | None = None) -> None:
        strength = str(reasoning_strength).strip()
        if not strength or "<|" in strength or "\n" in strength or "\r" in strength:
            raise ChatConfigurationError("ATEM reasoning_strength is invalid")
        day = re.compile(r"\d{4}-\d{2}-\d{2}")
        if not day.fullmatch(str(knowledge_cutoff).strip()):
            raise ChatConfigurationError("ATEM knowledge_cutoff must be YYYY-MM-DD")
        today = date.today().isoformat() if current_date is None else str(current_date).strip()
        if today and not day.fullmatch(today):
            raise ChatConfigurationError("ATEM current_date must be YYYY-MM-DD")
        self.reasoning_strength, self.knowledge_cutoff, self.current_date = strength, str(knowledge_cutoff).strip(), today

    def _suffix(self, with_reasoning: bool) -> str:
        parts = [f"Reasoning strength: {self.reasoning_strength}."] if with_reasoning else []
        parts.append('# Valid recipients: "self", "user".')
        return "\n\n".join(parts)

    def render(self, messages: Sequence[ChatMessage], *, include_assistant_prompt: bool = True) -> str:
        for i, m in enumerate(messages):
            if m.role not in ("system", "user", "assistant"):
                raise ChatConfigurationError(f"ATEM text mode has system, user and assistant messages only; messages[{i}] is {m.role!r}")
            if m.name is not None or m.tool_call_id is not None:
                raise ChatConfigurationError("ATEM text mode has no named or tool messages")
        out = ["<|begin_of_text|>"]
        if not any(m.role == "system" for m in messages):
            head = f"<|start|>system<|message|>You are a helpful AI assistant.\nKnowledge cutoff: {self.knowledge_cutoff}."
            if self.current_date:
                head += f"\nCurrent date: {self.current_date}."
            out.append(head + "\n\n" + self._suffix(True) + "<|eot|>")
        for m in messages:
            if m.role == "system":
                text = m.content
                for a, b in (("Reasoning effort", "Reasoning strength"), ("Reasoning Effort", "Reasoning Strength"),
                             ("reasoning effort", "reasoning strength"), ("REASONING EFFORT", "REASONING STRENGTH")):
                    text = text.replace(a, b)
                out.append("<|start|>system<|message|>" + text + "\n\n" + self._suffix("reasoning strength" not in text.lower()) + "<|eot|>")
            elif m.role == "user":
                out.append("<|start|>user<|message|>" + m.content + "<|eot|>")
            else:
                out.append("<|start|>assistant to=user<|message|>" + m.content + "<|eot|>")
        if include_assistant_prompt:
            out.append("<|start|>assistant")
        return "".join(out)


def resolve_chat_renderer(profile: str | None) -> ChatRenderer:
    table = {None: ChatRenderer, "role-headers": ChatRenderer, "plain-roles": PlainRolesRenderer, "placeholder": PlaceholderChatRenderer,
             MuseGlimmerATEMRenderer.name: MuseGlimmerATEMRenderer, "atem": MuseGlimmerATEMRenderer}
    if profile not in table:
        raise ChatConfigurationError(f"unknown chat template profile {profile!r}")
    return table[profile]()


# ---------------------------------------------------------------------------- response parsing


def strip_text_delimiters(text: str, delimiters: Sequence[str]) -> str:
    """Cuts the text at the first stop delimiter (and drops a partial delimiter at the very end)."""
    cut = len(text)
    for d in delimiters:
        i = text.find(d)
        if i >= 0:
            cut = min(cut, i)
    text = text[:cut]
    for d in delimiters:  # "...<|eo" at the end of a length-limited generation
        for k in range(len(d) - 1, 0, -1):
            if text.endswith(d[:k]):
                return text[:-k]
    return text


_ATEM_CHANNEL = re.compile(r"(?:<\|start\|>assistant)?\s*to=(self|user)<\|message\|>")
_ATEM_END = re.compile(r"<\|(eom|eot|end_of_text)\|>")
_ATEM_CONTROL = re.compile(r"<\|(start|message|eom|eot)\|>|to=(self|user)")


def parse_assistant_response(text: str, renderer: ChatRenderer, *, delimiters: Sequence[str] = ()) -> AssistantResponse:
    """Splits one continuation into what the user may see and what is private. For ATEM the
    envelope is protocol: only ``to=user`` segments are visible; when control fragments appear
    but no well-formed channel does, nothing is shown (fail closed)."""
    raw = str(text)
    if renderer.name != MuseGlimmerATEMRenderer.name:
        return AssistantResponse(strip_text_delimiters(raw, delimiters or renderer.stop_delimiters), raw)
    found = list(_ATEM_CHANNEL.finditer(raw))
    if not found:
        if _ATEM_CONTROL.search(raw):
            return AssistantResponse("", raw, used_channel_protocol=True, final_channel_complete=False)
        return AssistantResponse(strip_text_delimiters(raw, delimiters or renderer.stop_delimiters), raw)
    shown, private, complete = [], [], False
    for i, m in enumerate(found):
        seg_end = found[i + 1].start() if i + 1 < len(found) else len(raw)
        end = _ATEM_END.search(raw, m.end(), seg_end)
        body = raw[m.end():(end.start() if end else seg_end)].strip()
        if m.group(1) == "self":
            if body:
                private.append(body)
            continue
        if body:
            shown.append(body)
        complete = bool(end and end.group(1) in ("eot", "end_of_text"))
    return AssistantResponse("\n\n".join(shown).rstrip(), raw, "\n\n".join(private).rstrip(), True, complete if shown else False)


def read_manifest(artifact_dir: str | Path) -> dict:
    path = Path(artifact_dir) / "native-execution-manifest.json"
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)
