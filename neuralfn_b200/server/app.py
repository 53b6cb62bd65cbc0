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

    import hmac

    flat_owner: dict[str, str] = {}  # sessions created through the flat routes by a signed-in user -> user id
    run_session: dict[str, str] = {}  # run id -> session id, for the flat run routes

    def auth(authorization: str | None = Header(default=None), nfn_session: str | None = Cookie(default=None)):
        """Returns the signed-in user, or None for the bearer token / an open server (automation has
        full access). With accounts configured a signed-in cookie is required unless the bearer
        token is presented; without them the bearer token alone guards the routes."""
        if token and authorization is not None and hmac.compare_digest(authorization.encode(), f"Bearer {token}".encode()):
            return None
        if db is not None:
            from .platform_db import AuthError
            try:
                return db.authenticate(nfn_session)
            except AuthError as exc:
                raise HTTPException(status_code=401, detail=str(exc)) from None
        if token:
            raise HTTPException(status_code=401, detail="missing or wrong bearer token")
        return None

    def session_access(sid: str, user, *roles: str) -> None:
        """The flat /api/sessions routes address the same live store as the project-bound editor
        sessions. A signed-in user may touch a session only through a membership of its project
        (with one of ``roles`` when given) or, for sessions made through the flat routes, as their
        creator; everybody else gets 404 so that session ids do not leak."""
        if db is None or user is None or user.get("is_admin"):
            return
        from .platform_db import AuthError
        try:
            row = db.editor_session(sid)
        except KeyError:
            row = None
        if row is not None:
            try:
                db.require_role(row["project_id"], user, *roles)
                return
            except (AuthError, KeyError):
                raise HTTPException(status_code=404, detail=f"unknown session {sid!r}") from None
        if flat_owner.get(sid) != user["id"]:
            raise HTTPException(status_code=404, detail=f"unknown session {sid!r}")

    def visible_sessions(user) -> list[dict]:
        rows = store.list_sessions()
        if db is None or user is None or user.get("is_admin"):
            return rows
        out = []
        for r in rows:
            sid = r.get("session_id") or r.get("id")
            try:
                session_access(sid, user)
                out.append(r)
            except HTTPException:
                pass
        return out

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

    @app.delete("/api/sessions/{sid}/nodes/{node_id}")
    def remove_node(sid: str, node_id: str, user=Depends(auth)) -> dict:
        session_access(sid, user, "owner", "editor")
        guard(store.remove_node, sid, node_id)
        return {"deleted": node_id}

    @app.get("/api/sessions")
    def sessions(user=Depends(auth)) -> list[dict]:
        return visible_sessions(user)

    @app.post("/api/sessions")
    def create(body: dict = Body(default={}), user=Depends(auth)) -> dict:
        sid = guard(store.create_session, body.get("name", "untitled"), body.get("graph"))
        if user is not None:
            flat_owner[sid] = user["id"]
        return {"session_id": sid}

    @app.get("/api/sessions/{sid}/graph")
    def get_graph(sid: str, user=Depends(auth)) -> dict:
        session_access(sid, user)
        return guard(store.get_graph, sid)

    @app.put("/api/sessions/{sid}/graph")
    def put_graph(sid: str, body: dict = Body(...), user=Depends(auth)) -> dict:
        session_access(sid, user, "owner", "editor")
        if db is not None and user is not None:
            # a project-bound session keeps revisions: writes go through the project route (409 on a stale base)
            try:
                db.editor_session(sid)
                raise HTTPException(status_code=409, detail="this session belongs to a project: use PUT /api/projects/{pid}/sessions/{sid}/graph")
            except KeyError:
                pass
        return guard(store.replace_graph, sid, body)

    @app.delete("/api/sessions/{sid}")
    def delete(sid: str, user=Depends(auth)) -> dict:
        session_access(sid, user, "owner", "editor")
        guard(store.delete_session, sid)
        flat_owner.pop(sid, None)
        return {"deleted": sid}

    @app.post("/api/sessions/{sid}/nodes")
    def add_node(sid: str, body: dict = Body(...), user=Depends(auth)) -> dict:
        session_access(sid, user, "owner", "editor")
        return {"node_id": guard(store.add_builtin_node, sid, body["builtin"], role=body.get("role"))}

    @app.post("/api/sessions/{sid}/edges")
    def add_edge(sid: str, body: dict = Body(...), user=Depends(auth)) -> dict:
        session_access(sid, user, "owner", "editor")
        return {"edge_id": guard(store.add_edge, sid, body["src_node"], body["dst_node"], body.get("src_port", 0), body.get("dst_port", 0),
                                 body.get("weight", 1.0), body.get("bias", 0.0))}

    @app.post("/api/sessions/{sid}/execute")
    def execute(sid: str, body: dict = Body(...), user=Depends(auth)) -> dict:
        session_access(sid, user)
        return {"outputs": guard(store.execute, sid, body["inputs"])}

    @app.post("/api/sessions/{sid}/trace")
    def trace(sid: str, body: dict = Body(...), user=Depends(auth)) -> Any:
        session_access(sid, user)
        return guard(store.trace, sid, body["inputs"])

    @app.post("/api/sessions/{sid}/runs")
    def train(sid: str, body: dict = Body(...), user=Depends(auth)) -> dict:
        session_access(sid, user, "owner", "editor")
        rid = guard(store.train_start, sid, body["inputs"], body["targets"], method=body.get("method", "sgd"),
                    steps=int(body.get("steps", 500)), learning_rate=float(body.get("learning_rate", 0.5)))
        run_session[rid] = sid
        return {"run_id": rid}

    def run_access(rid: str, user, *roles: str) -> None:
        sid = run_session.get(rid)
        if sid is None and db is not None:
            rows = [r for r in db.runs() if r["id"] == rid]
            sid = rows[0]["session_id"] if rows else None
        if sid is not None:
            session_access(sid, user, *roles)
        elif db is not None and user is not None and not user.get("is_admin"):
            raise HTTPException(status_code=404, detail=f"unknown run {rid!r}")

    @app.get("/api/runs/{rid}")
    def run_status(rid: str, user=Depends(auth)) -> dict:
        run_access(rid, user)
        return guard(store.train_status, rid)

    @app.post("/api/runs/{rid}/stop")
    def run_stop(rid: str, user=Depends(auth)) -> dict:
        run_access(rid, user, "owner", "editor")
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

    @app.post("/api/datasets/info")
    def dataset_info(body: dict = Body(...), user=Depends(auth)) -> dict:
        from ..data import TokenDataset
        if db is not None and user is not None and not user.get("is_admin"):
            # a signed-in user may only look at dataset assets granted to one of their projects
            allowed = {os.path.realpath(d["path"]) for p_ in db.projects_for(user) for d in db.datasets_for_project(p_["id"])}
            if os.path.realpath(str(body.get("path", ""))) not in allowed:
                raise HTTPException(status_code=403, detail="this dataset is not granted to any of your projects")
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
