"""REST platform (FastAPI): sessions (graph CRUD, execute, trace), training runs, presets,
datasets, semantic helpers, and token-level generation through the resident engine.

    uvicorn neuralfn_b200.server.app:create_app --factory --host 127.0.0.1 --port 8000

Authentication: a bearer token from ``NEURALFN_API_TOKEN`` (unset = open, for local use), and,
when ``NEURALFN_DATABASE_PATH`` names a SQLite file, accounts with cookie sessions, projects,
revisioned graph snapshots and run records (``accounts.py`` / ``platform_db.py``;
``NEURALFN_BOOTSTRAP_ADMIN_EMAIL`` / ``_PASSWORD`` create the first administrator). Live state is a
``LiveStateStore`` (``NEURALFN_SNAPSHOT_DIR`` enables JSON snapshots). Reference counterpart:
``server/app.py``, ``server/routers``, ``server/settings.py:38-63``.
"""
from __future__ import annotations

import os
import threading
from typing import Any

from .store import LiveStateStore

__all__ = ["create_app", "InferenceConcurrencyGate"]


class InferenceConcurrencyGate:
    """Serialises access to one resident engine: the engine owns one stream and one set of
    activation buffers, so requests queue here instead of interleaving inside it."""

    def __init__(self, max_waiting: int = 64) -> None:
        self._lock = threading.Lock()
        self._waiting = 0
        self._max = max_waiting
        self._count = threading.Lock()

    def __enter__(self):
        with self._count:
            if self._waiting >= self._max:
                raise RuntimeError("inference queue is full")
            self._waiting += 1
        self._lock.acquire()
        return self

    def __exit__(self, *exc):
        self._lock.release()
        with self._count:
            self._waiting -= 1


def create_app(store: LiveStateStore | None = None, engine=None, db=None):
    from fastapi import Body, Cookie, Depends, FastAPI, Header, HTTPException

    store = store or LiveStateStore(os.environ.get("NEURALFN_SNAPSHOT_DIR") or None)
    token = os.environ.get("NEURALFN_API_TOKEN", "")
    if db is None and os.environ.get("NEURALFN_DATABASE_PATH"):
        from .platform_db import PlatformDB
        db = PlatformDB(os.environ["NEURALFN_DATABASE_PATH"])
    gate = InferenceConcurrencyGate()
    app = FastAPI(title="neuralfn_b200", version="0.1")
    app.state.store, app.state.engine, app.state.db = store, engine, db
    if db is not None:
        from .accounts import mount_account_routes
        db.ensure_bootstrap_admin()
        mount_account_routes(app, db, store, secure_cookies=os.environ.get("NEURALFN_SECURE_COOKIES", "") == "1")

    def auth(authorization: str | None = Header(default=None), nfn_session: str | None = Cookie(default=None)) -> None:
        """With accounts configured a signed-in cookie is required (or the bearer token, for
        automation); without them the bearer token alone guards the routes."""
        if token and authorization == f"Bearer {token}":
            return
        if db is not None:
            from .platform_db import AuthError
            try:
                db.authenticate(nfn_session)
                return
            except AuthError as exc:
                raise HTTPException(status_code=401, detail=str(exc)) from None
        if token:
            raise HTTPException(status_code=401, detail="missing or wrong bearer token")

    def guard(fn, *a, **k):
        try:
            return fn(*a, **k)
        except KeyError as exc:
            raise HTTPException(status_code=404, detail=str(exc)) from None
        except (ValueError, TypeError) as exc:
            raise HTTPException(status_code=422, detail=str(exc)) from None

    @app.get("/api/bootstrap")
    def bootstrap() -> dict:
        from ..ops import _lib
        return {"status": "ok", "auth_required": bool(token) or db is not None, "accounts": db is not None, "kernel_library": _lib.available(), "sessions": len(store.sessions)}

    @app.get("/", include_in_schema=False)
    @app.get("/editor", include_in_schema=False)
    def editor():
        """The single-page graph editor (vanilla JS over this API; the reference ships a React editor)."""
        from pathlib import Path

        from fastapi.responses import HTMLResponse
        return HTMLResponse((Path(__file__).with_name("editor.html")).read_text(encoding="utf-8"))

    @app.get("/api/builtins", dependencies=[Depends(auth)])
    def builtins() -> list[str]:
        from ..builtins import BUILTIN_MAP
        from ..scalar_builtins import SPEC_BY_NAME
        return sorted(set(BUILTIN_MAP) | set(SPEC_BY_NAME))

    @app.delete("/api/sessions/{sid}/nodes/{node_id}", dependencies=[Depends(auth)])
    def remove_node(sid: str, node_id: str) -> dict:
        guard(store.remove_node, sid, node_id)
        return {"deleted": node_id}

    @app.get("/api/sessions", dependencies=[Depends(auth)])
    def sessions() -> list[dict]:
        return store.list_sessions()

    @app.post("/api/sessions", dependencies=[Depends(auth)])
    def create(body: dict = Body(default={})) -> dict:
        return {"session_id": guard(store.create_session, body.get("name", "untitled"), body.get("graph"))}

    @app.get("/api/sessions/{sid}/graph", dependencies=[Depends(auth)])
    def get_graph(sid: str) -> dict:
        return guard(store.get_graph, sid)

    @app.put("/api/sessions/{sid}/graph", dependencies=[Depends(auth)])
    def put_graph(sid: str, body: dict = Body(...)) -> dict:
        return guard(store.replace_graph, sid, body)

    @app.delete("/api/sessions/{sid}", dependencies=[Depends(auth)])
    def delete(sid: str) -> dict:
        guard(store.delete_session, sid)
        return {"deleted": sid}

    @app.post("/api/sessions/{sid}/nodes", dependencies=[Depends(auth)])
    def add_node(sid: str, body: dict = Body(...)) -> dict:
        return {"node_id": guard(store.add_builtin_node, sid, body["builtin"], role=body.get("role"))}

    @app.post("/api/sessions/{sid}/edges", dependencies=[Depends(auth)])
    def add_edge(sid: str, body: dict = Body(...)) -> dict:
        return {"edge_id": guard(store.add_edge, sid, body["src_node"], body["dst_node"], body.get("src_port", 0), body.get("dst_port", 0),
                                 body.get("weight", 1.0), body.get("bias", 0.0))}

    @app.post("/api/sessions/{sid}/execute", dependencies=[Depends(auth)])
    def execute(sid: str, body: dict = Body(...)) -> dict:
        return {"outputs": guard(store.execute, sid, body["inputs"])}

    @app.post("/api/sessions/{sid}/trace", dependencies=[Depends(auth)])
    def trace(sid: str, body: dict = Body(...)) -> Any:
        return guard(store.trace, sid, body["inputs"])

    @app.post("/api/sessions/{sid}/runs", dependencies=[Depends(auth)])
    def train(sid: str, body: dict = Body(...)) -> dict:
        return {"run_id": guard(store.train_start, sid, body["inputs"], body["targets"], method=body.get("method", "sgd"),
                                steps=int(body.get("steps", 500)), learning_rate=float(body.get("learning_rate", 0.5)))}

    @app.get("/api/runs/{rid}", dependencies=[Depends(auth)])
    def run_status(rid: str) -> dict:
        return guard(store.train_status, rid)

    @app.post("/api/runs/{rid}/stop", dependencies=[Depends(auth)])
    def run_stop(rid: str) -> dict:
        return guard(store.train_stop, rid)

    @app.get("/api/presets", dependencies=[Depends(auth)])
    def presets() -> list[str]:
        from ..presets import PRESET_BUILDERS
        return sorted(PRESET_BUILDERS)

    @app.get("/api/presets/{name}", dependencies=[Depends(auth)])
    def preset(name: str) -> dict:
        from ..presets import build_preset
        return guard(lambda: build_preset(name).to_dict())

    @app.post("/api/semantic/match", dependencies=[Depends(auth)])
    def semantic_match(body: dict = Body(...)) -> dict:
        from ..semantic import ConversationalVocabulary
        return ConversationalVocabulary().match_topics_in_text(body["text"])

    @app.post("/api/datasets/info", dependencies=[Depends(auth)])
    def dataset_info(body: dict = Body(...)) -> dict:
        from ..data import TokenDataset
        return guard(lambda: TokenDataset(body["path"], allow_train_as_val=True).describe(int(body.get("seq_len", 1024)),
                                                                                         int(body.get("batch_size", 64))))

    @app.post("/v1/generate", dependencies=[Depends(auth)])
    def generate(body: dict = Body(...)) -> dict:
        if app.state.engine is None:
            raise HTTPException(status_code=503, detail="no resident engine is loaded")
        from ..serving import Sampling
        samp = Sampling(temperature=float(body.get("temperature", 0.0)), top_k=int(body.get("top_k", 0)), top_p=float(body.get("top_p", 1.0)),
                        seed=int(body.get("seed", 0)))
        with gate:
            out = app.state.engine.generate(body["prompts"], max_new_tokens=int(body.get("max_new_tokens", 32)), sampling=samp,
                                            eos_token=body.get("eos_token"))
        return {"generated": out}

    return app
