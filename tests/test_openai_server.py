"""OpenAI-compatible server, state store, queue and prefix-cache logic against a fake model (CPU)."""
import json
import threading
import time

import pytest

from neuralfn_b200.serving.chat import ByteTextCodec, PlainRolesRenderer
from neuralfn_b200.serving.inference import GenerationEvent, GenerationResult
from neuralfn_b200.serving.openai_server import BoundedSingleWorkerQueue, QueueFull, ServingRuntime, create_openai_app
from neuralfn_b200.serving.state import SCHEMA_VERSION, StateStore

fastapi = pytest.importorskip("fastapi")
from fastapi.testclient import TestClient  # noqa: E402


class FakeSession:
    """Echoes 'ok:' + the last user line of the prompt, one byte per token."""

    def __init__(self, model):
        self.model, self.ids, self.closed = model, [], False

    def prefill(self, ids):
        self.ids += list(ids)
        self.model.prefilled.append(len(ids))

    def decode(self, cfg, on_event=None, proposer=None, allowed_tokens=None):
        text = bytes(self.ids).decode("utf-8", "replace")
        last = [ln for ln in text.split("\n") if ln.startswith("User: ")][-1][6:]
        reply = ("ok:" + last).encode()[:cfg.max_new_tokens]
        events = []
        for i, b in enumerate(reply):
            ev = GenerationEvent(b, i, len(self.ids) + i, chr(b))
            events.append(ev)
            if on_event:
                on_event(ev)
        return GenerationResult(tuple(reply), reply.decode(), "stop" if len(reply) < cfg.max_new_tokens else "length", len(self.ids), len(reply), tuple(events))

    def close(self):
        self.closed = True


class FakeModel:
    codec = ByteTextCodec()

    def __init__(self):
        self.prefilled, self.sessions = [], []

    def create_session(self, seed=None):
        s = FakeSession(self)
        self.sessions.append(s)
        return s


@pytest.fixture()
def client():
    rt = ServingRuntime(model=FakeModel(), model_id="fake", renderer=PlainRolesRenderer(), state=StateStore(), max_output_tokens=64)
    return TestClient(create_openai_app(rt)), rt


def test_models_chat_and_streaming(client):
    c, rt = client
    assert c.get("/health").json()["status"] == "ok"
    assert c.get("/v1/models").json()["data"][0]["id"] == "fake"
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hello"}], "temperature": 0}).json()
    assert r["choices"][0]["message"]["content"] == "ok:hello" and r["usage"]["completion_tokens"] == 8
    assert all(s.closed for s in rt.model.sessions)
    with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "stream me please, slowly"}], "stream": True}) as resp:
        lines = [ln[6:] for ln in resp.iter_lines() if ln.startswith("data: ")]
    assert lines[-1] == "[DONE]"
    chunks = [json.loads(ln) for ln in lines[:-1]]
    text = "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks)
    assert text == "ok:stream me please, slowly" and chunks[-1]["choices"][0]["finish_reason"] == "stop"
    assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 400
    assert c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "temperature": -1}).status_code == 400
    r = c.post("/v1/completions", json={"prompt": "User: raw\n", "max_tokens": 4}).json()
    assert r["choices"][0]["text"] == "ok:r" and r["choices"][0]["finish_reason"] == "length"


def test_responses_and_conversations(client):
    c, _rt = client
    r1 = c.post("/v1/responses", json={"input": "first"}).json()
    assert r1["output_text"] == "ok:first" and r1["status"] == "completed"
    r2 = c.post("/v1/responses", json={"input": "second", "previous_response_id": r1["id"]}).json()
    assert r2["output_text"] == "ok:second" and r2["usage"]["input_tokens"] > r1["usage"]["input_tokens"]
    assert c.get(f"/v1/responses/{r2['id']}").json()["previous_response_id"] == r1["id"]
    assert c.delete(f"/v1/responses/{r1['id']}").json()["deleted"] and c.get(f"/v1/responses/{r1['id']}").status_code == 404
    conv = c.post("/v1/conversations", json={"metadata": {"k": "v"}, "items": [{"role": "user", "content": "earlier"}]}).json()
    r3 = c.post("/v1/responses", json={"input": "now", "conversation": conv["id"]}).json()
    assert r3["conversation"]["id"] == conv["id"]
    items = c.get(f"/v1/conversations/{conv['id']}/items").json()["data"]
    assert [it["content"] for it in items] == ["earlier", "now", "ok:now"]
    assert c.post("/v1/responses", json={"input": "x", "conversation": "conv_missing"}).status_code == 404
    assert c.delete(f"/v1/conversations/{conv['id']}").json()["deleted"]


def test_bearer_auth_and_loopback_rule(tmp_path):
    key = tmp_path / "key"
    key.write_text("s3cret\n")
    rt = ServingRuntime(model=FakeModel(), renderer=PlainRolesRenderer(), state=None)
    c = TestClient(create_openai_app(rt, api_key_file=key))
    assert c.get("/v1/models").status_code == 401
    assert c.get("/v1/models", headers={"Authorization": "Bearer nope"}).status_code == 401
    assert c.get("/v1/models", headers={"Authorization": "Bearer s3cret"}).status_code == 200
    assert c.get("/health").status_code == 200
    remote = TestClient(create_openai_app(ServingRuntime(model=FakeModel(), state=None)), client=("10.1.2.3", 5000))
    assert remote.get("/v1/models").status_code == 403
    remote_ok = TestClient(create_openai_app(ServingRuntime(model=FakeModel(), state=None), allow_unauthenticated_remote=True), client=("10.1.2.3", 5000))
    assert remote_ok.get("/v1/models").status_code == 200


def test_bounded_queue_rejects_when_full():
    q = BoundedSingleWorkerQueue(capacity=2)
    gate = threading.Event()
    order = []
    b1 = q.admit(lambda: (gate.wait(5), order.append(1)))
    b2 = q.admit(lambda: order.append(2))
    with pytest.raises(QueueFull):
        q.admit(lambda: None)
    gate.set()
    assert b1["done"].wait(5) and b2["done"].wait(5) and order == [1, 2]
    assert q.run(lambda: 7) == 7 and q.rejected == 1
    with pytest.raises(ZeroDivisionError):
        q.run(lambda: 1 / 0)
    q.close()


def test_state_store_persists(tmp_path):
    path = tmp_path / "state" / "db.sqlite"
    s = StateStore(path)
    conv = s.create_conversation({"a": 1}, [{"type": "message", "role": "user", "content": "hi"}])
    r = s.put_response({"output_text": "x"}, conversation_id=conv["id"])
    s.close()
    s2 = StateStore(path)
    assert s2.schema_version() == SCHEMA_VERSION and s2.get_response(r["id"])["output_text"] == "x"
    assert s2.list_items(conv["id"])[0]["content"] == "hi"
    assert s2.delete_conversation(conv["id"]) and s2.list_items(conv["id"]) == []


def test_train_dashboard_and_infer_tui(tmp_path):
    import io
    import json as _json

    from neuralfn_b200.cli.tui import InferTUI, TrainDashboard, sparkline
    assert sparkline([1, 2, 3, 4]) == "▁▃▆█" and sparkline([]) == ""
    log = io.StringIO()
    d = TrainDashboard(total_steps=10, tee=log)
    for i in range(1, 6):
        d.feed(_json.dumps({"event": "train_step", "step": i, "loss": 5.0 - 0.5 * i, "tokens_per_second": 1000.0 * i}))
    d.feed("plain text line")
    d.feed(_json.dumps({"event": "validation", "loss": 3.3}))
    d.feed(_json.dumps({"event": "checkpoint", "path": "/tmp/x/model_00000005.bin"}))
    d.feed(_json.dumps({"status": "ok", "steps": 10, "train_compute_tokens_per_second": 1234.0}))
    assert d.step == 5 and d.status == "complete" and d.val_losses == [3.3] and d.tokens_per_second == 1234.0
    assert log.getvalue().count("\n") == 9
    from rich.console import Console
    buf = io.StringIO()
    Console(file=buf, width=100).print(d.render())
    assert "model_00000005.bin" in buf.getvalue() and "complete" in buf.getvalue()

    class Sess(FakeSession):
        cached_tokens = 0
        token_ids = ()

        def prefill(self, ids):
            super().prefill(ids)
            self.token_ids = tuple(self.ids)

        def truncate(self, n):
            self.ids = self.ids[:n]
            self.token_ids = tuple(self.ids)

        def reset(self):
            self.ids, self.token_ids = [], ()

    class Model(FakeModel):
        manifest = {}

        def create_session(self, seed=None):
            return Sess(self)

    out = io.StringIO()
    tui = InferTUI(Model(), PlainRolesRenderer(), stdin=["hello there\n", "/mode sample\n", "/tokens 5\n", "again\n", "/show\n", "/reset\n", "/bogus\n", "/quit\n", "never\n"],
                   stdout=out, max_new_tokens=32)
    assert tui.run() == 0
    text = out.getvalue()
    assert "ok:hello there" in text and "(mode: sample)" in text and "ok:ag" in text and "turns 2" in text and "(conversation cleared)" in text
    assert "never" not in text and "commands:" in text
