"""Structured output: a JSON schema compiled into an ASCII byte grammar, and greedy
byte-exact generation over a model's single-byte tokens.

The grammar is a small pushdown machine over bytes. ``JsonSchemaByteGrammar(schema)`` accepts
a practical schema subset - ``object`` (properties emitted in declaration order; optional ones
may be skipped), ``array`` (``items``, ``minItems`` / ``maxItems``), ``string`` (printable
ASCII, ``\\"`` ``\\\\`` ``\\n`` ``\\t`` escapes, ``minLength`` / ``maxLength``, ``enum``),
``integer`` / ``number`` (optional sign, no leading zeros, ``maxDigits`` bound), ``boolean``,
``null``, ``enum`` / ``const`` of scalars - and emits compact JSON with no insignificant
whitespace, so every accepted byte string parses and validates. ``allowed_bytes()`` lists the
bytes that may come next; ``advance(byte)`` consumes one; ``complete`` tells when the document
is finished. ``ConstrainedDecoder`` maps bytes to the model's single-byte token ids and, at each
step, picks the highest-logit token among the allowed ones.

Behavioural counterpart: ``neuralfn/native_constrained.py`` (profile
``json-schema-ascii-byte-greedy-v1``).
"""
from __future__ import annotations

import json
from typing import Any, Callable, Sequence

__all__ = ["PROFILE", "SchemaError", "JsonSchemaByteGrammar", "ConstrainedDecoder", "single_byte_token_inventory"]

PROFILE = "json-schema-ascii-byte-greedy-v1"
_DIGITS = b"0123456789"
_STR_PLAIN = bytes(b for b in range(0x20, 0x7F) if b not in (0x22, 0x5C))  # printable ASCII except " and \
_ESCAPES = b'"\\nt'


class SchemaError(ValueError):
    pass


# Every node is a generator-like state object with: allowed() -> bytes, advance(b) -> None, done (may stop
# here), and dead-end freedom: allowed() is never empty unless done.


class _Literal:
    def __init__(self, text: bytes) -> None:
        self.text, self.i = text, 0

    @property
    def done(self) -> bool:
        return self.i == len(self.text)

    def allowed(self) -> bytes:
        return b"" if self.done else self.text[self.i:self.i + 1]

    def advance(self, b: int) -> None:
        self.i += 1


class _Choice:
    """One of several literals (enum / const / boolean / null), disambiguated byte by byte."""

    def __init__(self, options: Sequence[bytes]) -> None:
        if not options:
            raise SchemaError("an enum needs at least one value")
        self.options, self.i = list(dict.fromkeys(options)), 0

    @property
    def done(self) -> bool:
        return any(len(o) == self.i for o in self.options)

    def allowed(self) -> bytes:
        return bytes(sorted({o[self.i] for o in self.options if len(o) > self.i}))

    def advance(self, b: int) -> None:
        self.options = [o for o in self.options if len(o) > self.i and o[self.i] == b]
        self.i += 1


class _String:
    def __init__(self, min_len: int, max_len: int) -> None:
        self.min_len, self.max_len = min_len, max_len
        self.state, self.n = 0, 0  # 0: before opening quote, 1: inside, 2: after backslash, 3: closed

    @property
    def done(self) -> bool:
        return self.state == 3

    def allowed(self) -> bytes:
        if self.state == 0:
            return b'"'
        if self.state == 2:
            return _ESCAPES
        if self.state == 3:
            return b""
        out = b""
        if self.n < self.max_len:
            out += _STR_PLAIN + b"\\"
        if self.n >= self.min_len:
            out += b'"'
        return out

    def advance(self, b: int) -> None:
        if self.state == 0:
            self.state = 1
        elif self.state == 2:
            self.state, self.n = 1, self.n + 1
        elif b == 0x22:
            self.state = 3
        elif b == 0x5C:
            self.state = 2
        else:
            self.n += 1


class _Number:
    """-?(0|[1-9][0-9]*)(\\.[0-9]+)? ; the fraction only for ``number``. A number has no closing
    byte, so it reports ``done`` as soon as it is a valid number and the parent decides."""

    def __init__(self, integer: bool, max_digits: int, allow_negative: bool) -> None:
        self.integer, self.max_digits, self.neg_ok = integer, max_digits, allow_negative
        self.state, self.nd = 0, 0  # 0 start, 1 after '-', 2 after leading 0, 3 in int digits, 4 after '.', 5 in fraction

    @property
    def done(self) -> bool:
        return self.state in (2, 3, 5)

    def allowed(self) -> bytes:
        if self.state == 0:
            return (b"-" if self.neg_ok else b"") + _DIGITS
        if self.state == 1:
            return _DIGITS
        if self.state == 2:
            return b"" if self.integer else b"."
        if self.state == 3:
            return (_DIGITS if self.nd < self.max_digits else b"") + (b"" if self.integer else b".")
        if self.state == 4:
            return _DIGITS
        return _DIGITS if self.nd < self.max_digits else b""

    def advance(self, b: int) -> None:
        if b == 0x2D:
            self.state = 1
        elif b == 0x2E:
            self.state, self.nd = 4, 0
        elif self.state in (0, 1):
            self.state, self.nd = (2 if b == 0x30 else 3), 1
        elif self.state == 3:
            self.nd += 1
        else:
            self.state, self.nd = 5, self.nd + 1


class _Array:
    def __init__(self, make_item: Callable[[], Any], min_items: int, max_items: int) -> None:
        self.make_item, self.min_items, self.max_items = make_item, min_items, max_items
        self.state, self.n, self.item = 0, 0, None  # 0 before '[', 1 after '[' (empty so far), 2 in item, 3 closed

    @property
    def done(self) -> bool:
        return self.state == 3

    def _after_item(self) -> bytes:  # self.n counts the items BEFORE the current one
        return (b"," if self.n + 1 < self.max_items else b"") + (b"]" if self.n + 1 >= self.min_items else b"")

    def allowed(self) -> bytes:
        if self.state == 0:
            return b"["
        if self.state == 3:
            return b""
        if self.state == 1:
            first = self.make_item().allowed() if self.max_items > 0 else b""
            return first + (b"]" if self.min_items == 0 else b"")
        out = self.item.allowed()
        if self.item.done:
            out += self._after_item()
        return bytes(sorted(set(out)))

    def advance(self, b: int) -> None:
        if self.state == 0:
            self.state = 1
        elif self.state == 1:
            if b == 0x5D:
                self.state = 3
            else:
                self.item, self.state = self.make_item(), 2
                self.item.advance(b)
        else:
            if b in self.item.allowed():
                self.item.advance(b)
            elif b == 0x2C:
                self.n, self.item = self.n + 1, self.make_item()
            else:
                self.n, self.state = self.n + 1, 3


class _Object:
    """Properties in declaration order; an optional property may be skipped. After '{' or ',' the next
    byte is always '\"', so which property comes next is decided while its key is spelled out."""

    def __init__(self, props: list[tuple[str, Callable[[], Any], bool]]) -> None:
        self.props = props
        self.state = 0      # 0 before '{', 1 expecting key or '}', 2 spelling key, 3 in value, 4 closed
        self.next_prop = 0  # first property that may still appear
        self.emitted = 0
        self.cands: list[int] = []
        self.key_i = 0
        self.value = None

    def _key(self, idx: int) -> bytes:
        return json.dumps(self.props[idx][0]).encode("ascii") + b":"

    def _startable(self) -> list[int]:
        out = []
        for idx in range(self.next_prop, len(self.props)):
            out.append(idx)
            if self.props[idx][2]:  # required: nothing after it may come first
                break
        return out

    def _may_close(self) -> bool:
        return not any(self.props[idx][2] for idx in range(self.next_prop, len(self.props)))

    @property
    def done(self) -> bool:
        return self.state == 4

    def allowed(self) -> bytes:
        if self.state == 0:
            return b"{"
        if self.state == 4:
            return b""
        if self.state == 1:
            out = b'"' if self._startable() else b""
            if self.emitted == 0 and self._may_close():
                out += b"}"
            return out
        if self.state == 2:
            return bytes(sorted({self._key(i)[self.key_i] for i in self.cands}))
        out = self.value.allowed()
        if self.value.done:
            if self._startable():
                out += b","
            if self._may_close():
                out += b"}"
        return bytes(sorted(set(out)))

    def advance(self, b: int) -> None:
        if self.state == 0:
            self.state = 1
        elif self.state == 1:
            if b == 0x7D:
                self.state = 4
            else:
                self.cands, self.key_i, self.state = self._startable(), 1, 2
        elif self.state == 2:
            self.cands = [i for i in self.cands if self._key(i)[self.key_i] == b]
            self.key_i += 1
            if len(self.cands) == 1 and self.key_i == len(self._key(self.cands[0])):
                idx = self.cands[0]
                self.value, self.next_prop, self.state = self.props[idx][1](), idx + 1, 3
        else:
            if b in self.value.allowed():
                self.value.advance(b)
            elif b == 0x2C:
                self.emitted += 1
                self.state = 1
            else:
                self.state = 4


def _scalar_json(v: Any) -> bytes:
    if isinstance(v, (dict, list)):
        raise SchemaError("enum / const values must be scalars")
    text = json.dumps(v)
    if not text.isascii():
        raise SchemaError("enum values must be ASCII")
    return text.encode("ascii")


def _compile(schema: Any, depth: int = 0) -> Callable[[], Any]:
    if depth > 32:
        raise SchemaError("schema nests too deeply")
    if not isinstance(schema, dict):
        raise SchemaError("a schema node must be an object")
    if "const" in schema:
        lit = _scalar_json(schema["const"])
        return lambda: _Literal(lit)
    if "enum" in schema:
        opts = [_scalar_json(v) for v in schema["enum"]]
        return lambda: _Choice(opts)
    t = schema.get("type")
    if t == "boolean":
        return lambda: _Choice([b"true", b"false"])
    if t == "null":
        return lambda: _Literal(b"null")
    if t in ("integer", "number"):
        md = int(schema.get("maxDigits", 15))
        neg = not (schema.get("minimum", -1) >= 0)
        return lambda: _Number(t == "integer", md, neg)
    if t == "string":
        lo, hi = int(schema.get("minLength", 0)), int(schema.get("maxLength", 256))
        if lo > hi:
            raise SchemaError("minLength exceeds maxLength")
        return lambda: _String(lo, hi)
    if t == "array":
        item = _compile(schema.get("items", {"type": "string"}), depth + 1)
        lo, hi = int(schema.get("minItems", 0)), int(schema.get("maxItems", 64))
        if lo > hi:
            raise SchemaError("minItems exceeds maxItems")
        return lambda: _Array(item, lo, hi)
    if t == "object":
        props = schema.get("properties", {})
        if not isinstance(props, dict):
            raise SchemaError("properties must be an object")
        required = set(schema.get("required", []))
        unknown = required - set(props)
        if unknown:
            raise SchemaError(f"required names without a property schema: {sorted(unknown)}")
        for k in props:
            if not k.isascii():
                raise SchemaError("property names must be ASCII")
        keys = [json.dumps(k) for k in props]
        for a in keys:  # a key that is a strict prefix of another cannot be told apart before the ':'... json quotes end keys, so only duplicates clash
            if keys.count(a) > 1:
                raise SchemaError("duplicate property name")
        compiled = [(k, _compile(v, depth + 1), k in required) for k, v in props.items()]
        return lambda: _Object(compiled)
    raise SchemaError(f"unsupported schema node: {json.dumps(schema)[:80]}")


class JsonSchemaByteGrammar:
    def __init__(self, schema: dict) -> None:
        self._make = _compile(schema)
        self.reset()

    def reset(self) -> None:
        self.root = self._make()
        self.emitted = bytearray()

    @property
    def complete(self) -> bool:
        return self.root.done

    @property
    def must_stop(self) -> bool:
        return self.root.done and not self.root.allowed()

    def allowed_bytes(self) -> bytes:
        return self.root.allowed()

    def advance(self, byte: int) -> None:
        if byte not in self.root.allowed():
            raise SchemaError(f"byte {byte!r} is not allowed after {bytes(self.emitted)!r}")
        self.root.advance(byte)
        self.emitted.append(byte)

    def accepts(self, data: bytes) -> bool:
        g = JsonSchemaByteGrammar.__new__(JsonSchemaByteGrammar)
        g._make = self._make
        g.reset()
        try:
            for b in data:
                g.advance(b)
        except SchemaError:
            return False
        return g.complete


def single_byte_token_inventory(decode_token: Callable[[int], bytes | str], vocab_size: int) -> dict[int, int]:
    """byte -> token id for every token whose text is exactly one ASCII byte (the lowest id wins)."""
    inv: dict[int, int] = {}
    for tid in range(vocab_size):
        try:
            t = decode_token(tid)
        except Exception:
            continue
        raw = t.encode("utf-8", errors="ignore") if isinstance(t, str) else bytes(t)
        if len(raw) == 1 and raw[0] < 0x80 and raw[0] not in inv:
            inv[raw[0]] = tid
    return inv


class ConstrainedDecoder:
    """Drives a session: ``allowed_tokens(history)`` for ``NativeInferenceSession.decode`` plus the
    bookkeeping that feeds the chosen byte back into the grammar."""

    def __init__(self, schema: dict, byte_to_token: dict[int, int], stop_token: int | None = None) -> None:
        self.grammar = JsonSchemaByteGrammar(schema)
        self.byte_to_token = dict(byte_to_token)
        self.token_to_byte = {t: b for b, t in self.byte_to_token.items()}
        self.stop_token = stop_token
        self._seen = 0
        missing = [b for b in b'{}[]",:-.0123456789' if b not in self.byte_to_token]
        if missing:
            raise SchemaError(f"the model has no single-byte token for {bytes(missing)!r}")

    def start(self, history_len: int) -> None:
        self.grammar.reset()
        self._seen = history_len

    def _sync(self, history: Sequence[int]) -> None:
        """Feeds the grammar the bytes of the tokens generated since the last call."""
        for t in history[self._seen:]:
            if t in self.token_to_byte:
                self.grammar.advance(self.token_to_byte[t])
        self._seen = len(history)

    def allowed_tokens(self, history: Sequence[int]) -> list[int]:
        self._sync(history)
        out =[self.byte_to_token[b] for b in self.grammar.allowed_bytes() if b in self.byte_to_token]
        if self.grammar.complete and self.stop_token is not None:
            out.append(self.stop_token)
        return out

    def generate(self, session, max_new_tokens: int = 512):
        """Greedy byte-exact generation; returns (parsed JSON value, GenerationResult)."""
        from .inference import GenerationConfig
        self.start(len(session.token_ids))
        total = None
        for _ in range(max_new_tokens):
            self._sync(session.token_ids)
            if self.grammar.must_stop:
                break
            res = session.decode(GenerationConfig(max_new_tokens=1, temperature=0.0), allowed_tokens=self.allowed_tokens)
            total = res
            if res.token_ids[0] == self.stop_token:
                break
        self._sync(session.token_ids)
        if not self.grammar.complete:
            raise SchemaError("generation ended before the document was complete")
        return json.loads(bytes(self.grammar.emitted).decode("ascii")), total
