"""Chat codecs / renderers, structured-output grammar, generation config and proposers (CPU)."""
import json
import random

import pytest

from neuralfn_b200.serving.chat import (ByteTextCodec, ChatConfigurationError, ChatMessage, IncrementalTokenDecoder, MuseGlimmerATEMRenderer,
                                        PlainRolesRenderer, TokenIdTextCodec, parse_assistant_response, resolve_chat_renderer,
                                        strip_text_delimiters)
from neuralfn_b200.serving.constrained import ConstrainedDecoder, JsonSchemaByteGrammar, SchemaError
from neuralfn_b200.serving.inference import GenerationConfig, NGramProposer, NativeModelLoadConfig


def test_codecs_round_trip():
    c = ByteTextCodec(offset=3)
    ids = c.encode("héllo")
    assert c.decode(ids) == "héllo" and min(ids) >= 3
    assert TokenIdTextCodec().encode("1, 2  3") == [1, 2, 3]
    with pytest.raises(ChatConfigurationError):
        TokenIdTextCodec().encode("1 x")
    dec = IncrementalTokenDecoder(ByteTextCodec())
    pieces = [dec.push(t) for t in ByteTextCodec().encode("aé")]
    assert pieces == ["a", "", "é"]


def test_atem_render_and_parse():
    r = MuseGlimmerATEMRenderer(current_date="2026-02-03")
    text = r.render([ChatMessage("user", "hi")])
    assert text.startswith("<|begin_of_text|><|start|>system<|message|>You are a helpful AI assistant.\nKnowledge cutoff: 2026-01-04.\nCurrent date: 2026-02-03.")
    assert 'Reasoning strength: high.\n\n# Valid recipients: "self", "user".<|eot|>' in text
    assert text.endswith("<|start|>user<|message|>hi<|eot|><|start|>assistant")
    text = r.render([ChatMessage("system", "Be brief. Reasoning effort: low."), ChatMessage("user", "q"), ChatMessage("assistant", "a")],
                    include_assistant_prompt=False)
    assert "Reasoning strength: low." in text and text.count("Reasoning strength") == 1
    assert text.endswith("<|start|>assistant to=user<|message|>a<|eot|>")
    with pytest.raises(ChatConfigurationError):
        r.render([ChatMessage("tool", "x")])
    raw = " to=self<|message|>thinking...<|eom|><|start|>assistant to=user<|message|>The answer is 4.<|eot|>"
    resp = parse_assistant_response(raw, r)
    assert resp.visible_text == "The answer is 4." and resp.reasoning_text == "thinking..." and resp.final_channel_complete
    assert parse_assistant_response(" to=self<|message|>only private", r).visible_text == ""
    assert parse_assistant_response("<|message|>odd", r).visible_text == ""  # control fragments without a channel: fail closed
    assert parse_assistant_response("plain answer", r).visible_text == "plain answer"
    assert isinstance(resolve_chat_renderer("plain-roles"), PlainRolesRenderer)
    assert strip_text_delimiters("abc<|eot|>def", ["<|eot|>"]) == "abc" and strip_text_delimiters("abc<|eo", ["<|eot|>"]) == "abc"


def test_generation_and_load_config_validation():
    assert GenerationConfig(temperature=0).strict_model_compute and not GenerationConfig(temperature=1e-30).strict_model_compute
    for bad in (dict(temperature=-1), dict(top_p=0.0), dict(top_p=1.5), dict(max_new_tokens=-1), dict(top_k=-2), dict(temperature=float("nan"))):
        with pytest.raises((ValueError, TypeError)):
            GenerationConfig(**bad)
    with pytest.raises(ValueError):
        NativeModelLoadConfig(runtime="cpu")
    assert NGramProposer().propose([1, 2, 3, 4, 9, 1, 2, 3], 3)[0] == [4, 9, 1]
    assert NGramProposer().propose([1, 2, 3], 3)[0] == []


SCHEMA = {"type": "object", "required": ["name", "age", "tags"],
          "properties": {"name": {"type": "string", "minLength": 1, "maxLength": 8}, "nick": {"type": "string", "maxLength": 4},
                         "age": {"type": "integer", "minimum": 0, "maxDigits": 3}, "score": {"type": "number", "maxDigits": 4},
                         "ok": {"type": "boolean"}, "kind": {"enum": ["cat", "car", 7, None]},
                         "tags": {"type": "array", "items": {"type": "integer"}, "minItems": 1, "maxItems": 3},
                         "pos": {"type": "object", "properties": {"x": {"type": "number"}}, "required": ["x"]}}}


def _check(doc):
    assert set(doc) <= set(SCHEMA["properties"]) and {"name", "age", "tags"} <= set(doc)
    assert list(doc) == [k for k in SCHEMA["properties"] if k in doc]  # declaration order
    assert isinstance(doc["name"], str) and 1 <= len(doc["name"]) <= 8
    assert isinstance(doc["age"], int) and 0 <= doc["age"] <= 999
    assert 1 <= len(doc["tags"]) <= 3 and all(isinstance(t, int) for t in doc["tags"])
    if "kind" in doc:
        assert doc["kind"] in ("cat", "car", 7, None)
    if "pos" in doc:
        assert isinstance(doc["pos"]["x"], (int, float))


def test_grammar_random_walks_always_yield_valid_documents():
    rng = random.Random(0)
    g = JsonSchemaByteGrammar(SCHEMA)
    for _ in range(300):
        g.reset()
        for _step in range(400):
            allowed = g.allowed_bytes()
            if g.complete and (not allowed or rng.random() < 0.3):
                break
            assert allowed, bytes(g.emitted)
            # favour closers so walks end
            closers = [b for b in allowed if b in b'"}],']
            b = rng.choice(closers) if closers and rng.random() < 0.5 else rng.choice(list(allowed))
            g.advance(b)
        if g.complete:
            _check(json.loads(bytes(g.emitted).decode("ascii")))
    assert g.accepts(b'{"name":"bo","age":7,"tags":[1,2]}')
    assert g.accepts(b'{"name":"bo","nick":"","age":0,"score":-1.5,"ok":true,"kind":null,"tags":[3],"pos":{"x":2}}')
    for bad in (b'{"age":7,"name":"bo","tags":[1]}', b'{"name":"bo","age":07,"tags":[1]}', b'{"name":"","age":7,"tags":[1]}',
                b'{"name":"bo","age":7,"tags":[]}', b'{"name":"bo","age":7,"tags":[1,2,3,4]}', b'{"name":"bo","age":-1,"tags":[1]}',
                b'{"name":"bo","age":7,"tags":[1],}', b'{"name":"bo","age":7}'):
        assert not g.accepts(bad), bad
    with pytest.raises(SchemaError):
        JsonSchemaByteGrammar({"type": "object", "properties": {"a": {"type": "string"}}, "required": ["b"]})


class _FakeSession:
    """Prefers, at every step, the allowed token with the highest id."""

    def __init__(self):
        self.token_ids = (1, 2, 3)

    def decode(self, cfg, allowed_tokens=None):
        from neuralfn_b200.serving.inference import GenerationResult
        opts = allowed_tokens(self.token_ids)
        tok = max(opts)
        self.token_ids = self.token_ids + (tok,)
        return GenerationResult((tok,), "", "length", 0, 1)


def test_constrained_decoder_feeds_the_grammar():
    inv = {b: 1000 + b for b in range(0x20, 0x7F)}
    dec = ConstrainedDecoder({"type": "object", "required": ["n"], "properties": {"n": {"type": "integer", "maxDigits": 2}, "s": {"enum": ["a", "b"]}}},
                             inv, stop_token=5000)
    doc, _ = dec.generate(_FakeSession(), 64)
    assert isinstance(doc["n"], int)
    with pytest.raises(SchemaError):
        ConstrainedDecoder({"type": "null"}, {ord("n"): 1})
