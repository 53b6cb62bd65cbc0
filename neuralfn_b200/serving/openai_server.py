"""OpenAI-compatible HTTP front end of the resident engine.

Routes: ``/health``, ``/v1/models``, ``/v1/chat/completions`` (JSON or server-sent-event
streaming), ``/v1/completions``, and the stateful ``/v1/responses`` and ``/v1/conversations``
families backed by ``StateStore``. One worker thread owns the model: requests are admitted
into a bounded queue (HTTP 429 when it is full) and run one at a time, with the finished
session parked in the prefix cache so that the next turn of the same conversation only
prefills its new tokens. Bearer authentication reads the key from a file; without a key the
server only answers loopback clients unless ``allow_unauthenticated_remote`` is set.

Behavioural counterpart: ``neuralfn/native_serve.py`` (runtime :646, queue :1123-1290,
routes :1880-2546) and ``neuralfn/native_responses.py``.
"""
import json
import queue
import secrets
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterator

from .chat import ChatConfigurationError, ChatMessage, ChatRenderer, parse_assistant_response, resolve_chat_renderer
from .constrained import ConstrainedDecoder, SchemaError, single_byte_token_inventory
from .inference import GenerationConfig, InferenceError
from .state import StateStore

__all__ = ["QueueFull", "BoundedSingleWorkerQueue", "ServingRuntime", "create_openai_app", "run_server"]


class QueueFull(RuntimeError):
    pass


class BoundedSingleWorkerQueue:
    """At most ``capacity`` requests waiting or running; one worker thread runs them in order."""

    def __init__(self, capacity: int = 8) -> None:
        if capacity < 1:
            raise ValueError("capacity must be >= 1")
        self.capacity = capacity
        self._q: "queue.Queue[tuple[Callable[[], Any], dict] | None]" = queue.Queue()
        self._inflight = 0
        self._lock = threading.Lock()
        self._thread = threading.Thread(target=self._run, name="nfn-serve-worker", daemon=True)
        self._thread.start()
        self.completed = 0
        self.rejected = 0

    def _run(self) -> None:
        while True:
            job = self._q.get()
            if job is None:
                return
            fn, box = job
            try:
                box["result"] = fn()
            except BaseException as exc:  # delivered to the waiting request
                box["error"] = exc
            finally:
                with self._lock:
                    self._inflight -= 1
                    self.completed += 1
                box["done"].set()

    def admit(self, fn: Callable[[], Any]) -> dict:
        with self._lock:
            if self._inflight >= self.capacity:
                self.rejected += 1
                raise QueueFull(f"{self._inflight} requests already admitted (capacity {self.capacity})")
            self._inflight += 1
        box: dict = {"done": threading.Event()}
        self._q.put((fn, box))
        return box

    def run(self, fn: Callable[[], Any], timeout: float | None = None) -> Any:
        box = self.admit(fn)
        if not box["done"].wait(timeout):
            raise TimeoutError("request timed out in the serving queue")
        if "error" in box:
            raise box["error"]
        return box["result"]

    @property
    def depth(self) -> int:
        return self._inflight

    def close(self) -> None:
        self._q.put(None)
        self._thread.join(timeout=5)


@dataclass
class ServingRuntime:
    """Everything a request needs: the model, how to turn chat into tokens, limits, state."""
    model: Any
    model_id: str = "neuralfn-b200"
    renderer: ChatRenderer = field(default_factory=ChatRenderer)
    stop_token_ids: tuple[int, ...] = ()
    prefix_cache: Any = None
    state: StateStore | None = None
    max_output_tokens: int = 512
    queue: BoundedSingleWorkerQueue = field(default_factory=BoundedSingleWorkerQueue)
    proposer_factory: Callable[[], Any] | None = None
    created: int = field(default_factory=lambda: int(time.time()))

    @classmethod
    def load(cls, artifact_dir: str | Path, *, sessions: int = 4, state_db: str | Path | None = None, queue_capacity: int = 8,
             prefix_cache_entries: int = 2, **kw) -> "ServingRuntime":
        from .inference import NativeInferenceModel, NativeModelLoadConfig
        from .prefix_cache import PrefixCache
        model = NativeInferenceModel.load(artifact_dir, NativeModelLoadConfig(session_count=sessions))
        man = model.manifest
        return cls(model=model, model_id=man.get("model_id", Path(artifact_dir).name), renderer=resolve_chat_renderer(man.get("chat_template")),
                   stop_token_ids=tuple(man.get("stop_token_ids", ())), prefix_cache=PrefixCache(model, prefix_cache_entries) if prefix_cache_entries else None,
                   state=StateStore(state_db) if state_db else StateStore(), queue=BoundedSingleWorkerQueue(queue_capacity), **kw)

    # -- request preparation ---------------------------------------------------------------
    def context_limit(self) -> int:
        eng = getattr(self.model, "engine", None)
        return int(getattr(getattr(eng, "config", None), "max_seq", 1 << 30))

    def prepare_chat(self, messages: list[dict], max_tokens: int | None) -> tuple[list[int], int]:
        if not isinstance(messages, list) or not messages:
            raise ValueError("messages must be a non-empty list")
        msgs = []
        for m in messages:
            content = m.get("content")
            if isinstance(content, list):  # content parts: text only
                if any(p.get("type") not in ("text", "input_text", "output_text") for p in content):
                    raise ValueError("only text content parts are supported")
                content = "".join(p.get("text", "") for p in content)
            msgs.append(ChatMessage(m.get("role", "user"), content if isinstance(content, str) else "", m.get("name"), m.get("tool_call_id")))
        prompt = self.renderer.render(msgs, include_assistant_prompt=True)
        ids = self.model.codec.encode(prompt)
        budget = min(self.max_output_tokens, max_tokens if max_tokens is not None else self.max_output_tokens)
        room = self.context_limit() - 1 - len(ids)
        if room < 1:
            raise ValueError(f"the prompt holds {len(ids)} tokens; the context window is {self.context_limit()}")
        return ids, max(0, min(budget, room))

    # -- generation (runs on the worker thread) -------------------------------------------
    def generate(self, prompt_ids: list[int], cfg: GenerationConfig, on_event=None, schema: dict | None = None):
        lease = self.prefix_cache.acquire(prompt_ids, cfg.seed) if self.prefix_cache is not None else None
        session = lease.session if lease else self.model.create_session(cfg.seed)
        reused = lease.reused_tokens if lease else 0
        keep = False
        try:
            session.prefill(prompt_ids[reused:])
            if schema is not None:
                codec = self.model.codec
                inv = single_byte_token_inventory(lambda t: codec.decode([t]), int(codec.vocab_size or 0))
                doc, res = ConstrainedDecoder(schema, inv).generate(session, cfg.max_new_tokens)
                text = json.dumps(doc, separators=(",", ":"))
                out = {"text": text, "token_ids": codec.encode(text), "finish_reason": "stop", "prompt_tokens": len(prompt_ids), "reused_tokens": reused}
            else:
                proposer = self.proposer_factory() if self.proposer_factory else None
                res = session.decode(cfg, on_event=on_event, proposer=proposer)
                out = {"text": res.text, "token_ids": list(res.token_ids), "finish_reason": res.finish_reason, "prompt_tokens": len(prompt_ids),
                       "reused_tokens": reused, "speculative": {"proposed": res.speculative_proposed_tokens, "accepted": res.speculative_accepted_tokens}}
            keep = True
            return out
        finally:
            if self.prefix_cache is not None:
                self.prefix_cache.release(session, keep=keep)
            else:
                session.close()


def _sse(payload: dict | str) -> bytes:
    return ("data: " + (payload if isinstance(payload, str) else json.dumps(payload, separators=(",", ":"))) + "\n\n").encode("utf-8")


def create_openai_app(runtime: ServingRuntime, *, api_key_file: str | Path | None = None, allow_unauthenticated_remote: bool = False,
                      enable_stateful: bool = True, request_timeout: float = 600.0):
    from fastapi import Body, Depends, FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse, StreamingResponse

    api_key = None
    if api_key_file is not None:
        api_key = Path(api_key_file).read_text(encoding="utf-8").strip()
        if not api_key:
            raise ValueError("the API key file is empty")
    app = FastAPI(title="neuralfn_b200 inference")

    def auth(request: Request) -> None:
        if api_key is not None:
            got = request.headers.get("authorization", "")
            if not (got.startswith("Bearer ") and secrets.compare_digest(got[7:].strip(), api_key)):
                raise HTTPException(401, detail={"error": {"message": "invalid API key", "type": "invalid_request_error"}})
            return
        host = request.client.host if request.client else ""
        if not allow_unauthenticated_remote and host not in ("127.0.0.1", "::1", "localhost", "testclient"):
            raise HTTPException(403, detail={"error": {"message": "unauthenticated access is limited to loopback clients", "type": "forbidden"}})

    def gen_config(body: dict, max_new: int) -> GenerationConfig:
        stop = tuple(runtime.stop_token_ids) + tuple(int(t) for t in body.get("stop_token_ids", ()))
        try:
            return GenerationConfig(max_new_tokens=max_new, temperature=float(body.get("temperature", 0.8)), top_k=body.get("top_k"),
                                    top_p=float(body.get("top_p", 1.0)), seed=body.get("seed"), stop_token_ids=stop)
        except (TypeError, ValueError) as exc:
            raise HTTPException(400, detail={"error": {"message": str(exc), "type": "invalid_request_error"}})

    def schema_of(body: dict) -> dict | None:
        rf = body.get("response_format") or (body.get("text") or {}).get("format")
        if not rf or rf.get("type") in (None, "text"):
            return None
        if rf.get("type") == "json_schema":
            js = rf.get("json_schema", rf)
            return js.get("schema", js)
        raise HTTPException(400, detail={"error": {"message": "response_format must be text or json_schema", "type": "invalid_request_error"}})

    def run_job(fn):
        try:
            return runtime.queue.run(fn, request_timeout)
        except QueueFull as exc:
            raise HTTPException(429, detail={"error": {"message": str(exc), "type": "rate_limit_error"}})
        except (InferenceError, ChatConfigurationError, SchemaError, ValueError) as exc:
            raise HTTPException(400, detail={"error": {"message": str(exc), "type": "invalid_request_error"}})

    def usage(out: dict) -> dict:
        n = len(out["token_ids"])
        return {"prompt_tokens": out["prompt_tokens"], "completion_tokens": n, "total_tokens": out["prompt_tokens"] + n,
                "prompt_tokens_details": {"cached_tokens": out.get("reused_tokens", 0)}}

    @app.get("/health")
    def health() -> dict:
        return {"status": "ok", "model": runtime.model_id, "queue_depth": runtime.queue.depth, "queue_capacity": runtime.queue.capacity}

    @app.get("/v1/models", dependencies=[Depends(auth)])
    def models() -> dict:
        return {"object": "list", "data": [{"id": runtime.model_id, "object": "model", "created": runtime.created, "owned_by": "neuralfn_b200"}]}

    @app.post("/v1/chat/completions", dependencies=[Depends(auth)])
    def chat_completions(body: dict = Body(...)):
        try:
            ids, max_new = runtime.prepare_chat(body.get("messages"), body.get("max_completion_tokens", body.get("max_tokens")))
        except (ValueError, ChatConfigurationError) as exc:
            raise HTTPException(400, detail={"error": {"message": str(exc), "type": "invalid_request_error"}})
        cfg, schema = gen_config(body, max_new), schema_of(body)
        cid, created = "chatcmpl-" + secrets.token_hex(12), int(time.time())

        def finish(out: dict) -> dict:
            shown = parse_assistant_response(out["text"], runtime.renderer)
            return {"id": cid, "object": "chat.completion", "created": created, "model": runtime.model_id,
                    "choices": [{"index": 0, "message": {"role": "assistant", "content": shown.visible_text}, "finish_reason": out["finish_reason"]}],
                    "usage": usage(out)}

        if not body.get("stream"):
            return finish(run_job(lambda: runtime.generate(ids, cfg, schema=schema)))

        events: "queue.Queue[Any]" = queue.Queue()

        def job():
            try:
                out = runtime.generate(ids, cfg, on_event=lambda ev: events.put(ev), schema=schema)
                events.put(("done", out))
            except BaseException as exc:
                events.put(("error", exc))
                raise

        try:
            runtime.queue.admit(job)
        except QueueFull as exc:
            raise HTTPException(429, detail={"error": {"message": str(exc), "type": "rate_limit_error"}})

        def stream() -> Iterator[bytes]:
            chunk = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": runtime.model_id}
            yield _sse(dict(chunk, choices=[{"index": 0, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]))
            raw, sent = "", 0
            while True:
                ev = events.get()
                if isinstance(ev, tuple):
                    kind, val = ev
                    if kind == "error":
                        yield _sse({"error": {"message": str(val), "type": "server_error"}})
                    else:
                        shown = parse_assistant_response(val["text"], runtime.renderer).visible_text
                        if len(shown) > sent:
                            yield _sse(dict(chunk, choices=[{"index": 0, "delta": {"content": shown[sent:]}, "finish_reason": None}]))
                        yield _sse(dict(chunk, choices=[{"index": 0, "delta": {}, "finish_reason": val["finish_reason"]}], usage=usage(val)))
                    break
                raw += ev.text
                # stream only text that can no longer turn out to be private or a stop delimiter
                shown = parse_assistant_response(raw, runtime.renderer).visible_text
                safe = max(sent, len(shown) - 16)
                if safe > sent:
                    yield _sse(dict(chunk, choices=[{"index": 0, "delta": {"content": shown[sent:safe]}, "finish_reason": None}]))
                    sent = safe
            yield _sse("[DONE]")

        return StreamingResponse(stream(), media_type="text/event-stream")

    @app.post("/v1/completions", dependencies=[Depends(auth)])
    def completions(body: dict = Body(...)):
        prompt = body.get("prompt")
        ids = [int(t) for t in prompt] if isinstance(prompt, list) else runtime.model.codec.encode(str(prompt or ""))
        if not ids:
            raise HTTPException(400, detail={"error": {"message": "empty prompt", "type": "invalid_request_error"}})
        max_new = max(0, min(int(body.get("max_tokens", 16)), runtime.max_output_tokens, runtime.context_limit() - 1 - len(ids)))
        out = run_job(lambda: runtime.generate(ids, gen_config(body, max_new)))
        return {"id": "cmpl-" + secrets.token_hex(12), "object": "text_completion", "created": int(time.time()), "model": runtime.model_id,
                "choices": [{"index": 0, "text": out["text"], "token_ids": out["token_ids"], "finish_reason": out["finish_reason"]}], "usage": usage(out)}

    if enable_stateful and runtime.state is not None:
        store = runtime.state

        def input_messages(inp) -> list[dict]:
            if isinstance(inp, str):
                return [{"role": "user", "content": inp}]
            if isinstance(inp, list):
                return [{"role": it.get("role", "user"), "content": it.get("content", "")} for it in inp if it.get("type", "message") == "message"]
            raise HTTPException(400, detail={"error": {"message": "input must be a string or a list of messages", "type": "invalid_request_error"}})

        @app.post("/v1/responses", dependencies=[Depends(auth)])
        def create_response(body: dict = Body(...)):
            history: list[dict] = []
            prev, conv = body.get("previous_response_id"), body.get("conversation")
            conv_id = conv.get("id") if isinstance(conv, dict) else conv
            if prev and conv_id:
                raise HTTPException(400, detail={"error": {"message": "give previous_response_id or conversation, not both", "type": "invalid_request_error"}})
            if prev:
                chain = store.response_chain(prev)
                if not chain:
                    raise HTTPException(404, detail={"error": {"message": f"no response {prev}", "type": "not_found"}})
                for r in chain:
                    history += r.get("_input_messages", []) + [{"role": "assistant", "content": r.get("output_text", "")}]
            if conv_id:
                if store.get_conversation(conv_id) is None:
                    raise HTTPException(404, detail={"error": {"message": f"no conversation {conv_id}", "type": "not_found"}})
                history += [{"role": it["role"], "content": it["content"]} for it in store.list_items(conv_id) if it.get("type") == "message"]
            new_msgs = input_messages(body.get("input", ""))
            if body.get("instructions"):
                history = [{"role": "system", "content": str(body["instructions"])}] + history
            try:
                ids, max_new = runtime.prepare_chat(history + new_msgs, body.get("max_output_tokens"))
            except (ValueError, ChatConfigurationError) as exc:
                raise HTTPException(400, detail={"error": {"message": str(exc), "type": "invalid_request_error"}})
            out = run_job(lambda: runtime.generate(ids, gen_config(body, max_new), schema=schema_of(body)))
            text = parse_assistant_response(out["text"], runtime.renderer).visible_text
            u = usage(out)
            payload = {"object": "response", "created_at": int(time.time()), "status": "completed" if out["finish_reason"] != "length" else "incomplete",
                       "model": runtime.model_id, "output_text": text, "previous_response_id": prev, "conversation": {"id": conv_id} if conv_id else None,
                       "output": [{"type": "message", "role": "assistant", "status": "completed", "content": [{"type": "output_text", "text": text}]}],
                       "usage": {"input_tokens": u["prompt_tokens"], "output_tokens": u["completion_tokens"], "total_tokens": u["total_tokens"]},
                       "_input_messages": new_msgs}
            if body.get("store", True):
                payload = store.put_response(payload, conversation_id=conv_id, previous_response_id=prev)
            else:
                payload["id"] = "resp_" + secrets.token_hex(12)
            if conv_id:
                store.add_items(conv_id, [dict(m, type="message") for m in new_msgs] + [{"type": "message", "role": "assistant", "content": text}])
            return {k: v for k, v in payload.items() if not k.startswith("_")}

        @app.get("/v1/responses/{rid}", dependencies=[Depends(auth)])
        def get_response(rid: str):
            r = store.get_response(rid)
            if r is None:
                raise HTTPException(404, detail={"error": {"message": f"no response {rid}", "type": "not_found"}})
            return {k: v for k, v in r.items() if not k.startswith("_")}

        @app.delete("/v1/responses/{rid}", dependencies=[Depends(auth)])
        def delete_response(rid: str):
            if not store.delete_response(rid):
                raise HTTPException(404, detail={"error": {"message": f"no response {rid}", "type": "not_found"}})
            return {"id": rid, "object": "response.deleted", "deleted": True}

        @app.post("/v1/conversations", dependencies=[Depends(auth)])
        def create_conversation(body: dict = Body(default={})):
            items = [dict(it, type=it.get("type", "message")) for it in body.get("items", [])]
            return store.create_conversation(body.get("metadata"), items)

        @app.get("/v1/conversations/{cid}", dependencies=[Depends(auth)])
        def get_conversation(cid: str):
            c = store.get_conversation(cid)
            if c is None:
                raise HTTPException(404, detail={"error": {"message": f"no conversation {cid}", "type": "not_found"}})
            return c

        @app.delete("/v1/conversations/{cid}", dependencies=[Depends(auth)])
        def delete_conversation(cid: str):
            if not store.delete_conversation(cid):
                raise HTTPException(404, detail={"error": {"message": f"no conversation {cid}", "type": "not_found"}})
            return {"id": cid, "object": "conversation.deleted", "deleted": True}

        @app.get("/v1/conversations/{cid}/items", dependencies=[Depends(auth)])
        def list_items(cid: str):
            if store.get_conversation(cid) is None:
                raise HTTPException(404, detail={"error": {"message": f"no conversation {cid}", "type": "not_found"}})
            return {"object": "list", "data": store.list_items(cid)}

        @app.post("/v1/conversations/{cid}/items", dependencies=[Depends(auth)])
        def add_items(cid: str, body: dict = Body(...)):
            try:
                return {"object": "list", "data": store.add_items(cid, [dict(it, type=it.get("type", "message")) for it in body.get("items", [])])}
            except KeyError:
                raise HTTPException(404, detail={"error": {"message": f"no conversation {cid}", "type": "not_found"}})

    @app.exception_handler(HTTPException)
    async def http_error(_request, exc: HTTPException):
        detail = exc.detail if isinstance(exc.detail, dict) else {"error": {"message": str(exc.detail), "type": "error"}}
        return JSONResponse(detail, status_code=exc.status_code)

    return app


def run_server(artifact_dir: str | Path, *, host: str = "127.0.0.1", port: int = 8000, api_key_file: str | None = None,
               allow_unauthenticated_remote: bool = False, **runtime_kw) -> None:  # pragma: no cover - needs a GPU and a socket
    import uvicorn
    if host not in ("127.0.0.1", "::1", "localhost") and api_key_file is None and not allow_unauthenticated_remote:
        raise SystemExit("refusing to listen on a non-loopback address without --api-key-file (or --allow-unauthenticated-remote)")
    runtime = ServingRuntime.load(artifact_dir, **runtime_kw)
    uvicorn.run(create_openai_app(runtime, api_key_file=api_key_file, allow_unauthenticated_remote=allow_unauthenticated_remote), host=host, port=port)
