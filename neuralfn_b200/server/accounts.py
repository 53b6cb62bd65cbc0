"""Account, project and persistence routes of the platform, mounted on the REST app when a
``PlatformDB`` is configured.

    POST /api/auth/login {email, password}     sets the ``nfn_session`` cookie (HttpOnly, SameSite=Lax)
    POST /api/auth/logout                      GET /api/auth/me
    GET/POST /api/admin/users                  POST /api/admin/users/{id}/active      (administrators)
    GET/POST /api/projects                     GET/DELETE /api/projects/{pid}
    PUT  /api/projects/{pid}/members/{uid} {role | null}
    GET/POST /api/projects/{pid}/sessions      editor sessions bound to a project
    PUT  /api/projects/{pid}/sessions/{sid}/graph {graph, base_revision}   409 on a stale revision
    GET  /api/projects/{pid}/sessions/{sid}/revisions/{n}
    GET  /api/projects/{pid}/runs              GET /api/runs/{rid}/events   (server-sent events)

Behavioural counterparts: ``server/routers/{auth,admin,projects,sessions,runs}.py`` and
``server/services/{auth_service,session_service,run_service}.py``.
"""
import json
import time

from ..serialization import graph_from_json, graph_to_json
from .platform_db import AuthError, PlatformDB, RevisionConflict

__all__ = ["mount_account_routes", "COOKIE_NAME"]

COOKIE_NAME = "nfn_session"


def mount_account_routes(app, db: PlatformDB, store, *, secure_cookies: bool = False):
    from fastapi import Body, Cookie, Depends, HTTPException, Response
    from fastapi.responses import StreamingResponse

    def current_user(nfn_session: str | None = Cookie(default=None)) -> dict:
        try:
            return db.authenticate(nfn_session)
        except AuthError as exc:
            raise HTTPException(status_code=401, detail=str(exc)) from None

    def admin(user: dict = Depends(current_user)) -> dict:
        if not user["is_admin"]:
            raise HTTPException(status_code=403, detail="administrators only")
        return user

    def guard(fn, *a, **k):
        try:
            return fn(*a, **k)
        except KeyError as exc:
            raise HTTPException(status_code=404, detail=str(exc)) from None
        except AuthError as exc:
            raise HTTPException(status_code=403, detail=str(exc)) from None
        except RevisionConflict as exc:
            raise HTTPException(status_code=409, detail={"message": str(exc), "current_revision": exc.current}) from None
        except (ValueError, TypeError) as exc:
            raise HTTPException(status_code=422, detail=str(exc)) from None

    # -- authentication ---------------------------------------------------------------------------
    @app.post("/api/auth/login")
    def login(response: Response, body: dict = Body(...)) -> dict:
        try:
            token, user = db.login(str(body.get("email", "")), str(body.get("password", "")))
        except AuthError as exc:
            raise HTTPException(status_code=401, detail=str(exc)) from None
        response.set_cookie(COOKIE_NAME, token, max_age=int(db.session_ttl), httponly=True, samesite="lax", secure=secure_cookies, path="/")
        return {"user": user}

    @app.post("/api/auth/logout")
    def logout(response: Response, nfn_session: str | None = Cookie(default=None)) -> dict:
        if nfn_session:
            db.logout(nfn_session)
        response.delete_cookie(COOKIE_NAME, path="/")
        return {"status": "signed out"}

    @app.get("/api/auth/me")
    def me(user: dict = Depends(current_user)) -> dict:
        return {"user": user, "projects": db.projects_for(user)}

    # -- administration ---------------------------------------------------------------------------
    @app.get("/api/admin/users")
    def users(_: dict = Depends(admin)) -> list[dict]:
        return db.list_users()

    @app.post("/api/admin/users")
    def add_user(body: dict = Body(...), _: dict = Depends(admin)) -> dict:
        return guard(db.create_user, str(body.get("email", "")), str(body.get("password", "")), display_name=str(body.get("display_name", "")),
                     is_admin=bool(body.get("is_admin", False)))

    @app.post("/api/admin/users/{uid}/active")
    def set_active(uid: str, body: dict = Body(...), me_: dict = Depends(admin)) -> dict:
        if uid == me_["id"] and not body.get("active", True):
            raise HTTPException(status_code=422, detail="an administrator cannot deactivate their own account")
        return guard(db.set_user_active, uid, bool(body.get("active", True)))

    # -- projects ---------------------------------------------------------------------------------
    @app.get("/api/projects")
    def projects(user: dict = Depends(current_user)) -> list[dict]:
        return db.projects_for(user)

    @app.post("/api/projects")
    def add_project(body: dict = Body(...), user: dict = Depends(current_user)) -> dict:
        return guard(db.create_project, user["id"], str(body.get("name", "")), str(body.get("description", "")))

    @app.get("/api/projects/{pid}")
    def project(pid: str, user: dict = Depends(current_user)) -> dict:
        guard(db.require_role, pid, user)
        return db.project(pid) | {"datasets": db.datasets_for_project(pid)}

    @app.delete("/api/projects/{pid}")
    def drop_project(pid: str, user: dict = Depends(current_user)) -> dict:
        guard(db.require_role, pid, user, "owner")
        for s in db.editor_sessions(pid):
            if s["id"] in store.sessions:
                store.delete_session(s["id"])
        db.delete_project(pid)
        return {"deleted": pid}

    @app.put("/api/projects/{pid}/members/{uid}")
    def member(pid: str, uid: str, body: dict = Body(...), user: dict = Depends(current_user)) -> dict:
        guard(db.require_role, pid, user, "owner")
        return guard(db.set_member, pid, uid, body.get("role"))

    # -- editor sessions --------------------------------------------------------------------------
    def live(sid: str):
        """The live graph of a stored session, loading its latest snapshot on first use."""
        if sid not in store.sessions:
            _, text = db.load_snapshot(sid)
            store.sessions[sid] = graph_from_json(text)
        return store.sessions[sid]

    @app.get("/api/projects/{pid}/sessions")
    def sessions(pid: str, user: dict = Depends(current_user)) -> list[dict]:
        guard(db.require_role, pid, user)
        return db.editor_sessions(pid)

    @app.post("/api/projects/{pid}/sessions")
    def add_session(pid: str, body: dict = Body(default={}), user: dict = Depends(current_user)) -> dict:
        guard(db.require_role, pid, user, "owner", "editor")
        sid = guard(store.create_session, str(body.get("name", "untitled")), body.get("graph"))
        return guard(db.create_editor_session, pid, str(body.get("name", "untitled")), graph_to_json(store.sessions[sid]), session_id=sid)

    def session_of(pid: str, sid: str, user: dict, *roles: str) -> dict:
        guard(db.require_role, pid, user, *roles)
        s = guard(db.editor_session, sid)
        if s["project_id"] != pid:
            raise HTTPException(status_code=404, detail=f"session {sid} is not part of project {pid}")
        return s

    @app.get("/api/projects/{pid}/sessions/{sid}/graph")
    def graph(pid: str, sid: str, user: dict = Depends(current_user)) -> dict:
        s = session_of(pid, sid, user)
        return {"revision": s["revision"], "graph": guard(live, sid).to_dict()}

    @app.put("/api/projects/{pid}/sessions/{sid}/graph")
    def put_graph(pid: str, sid: str, body: dict = Body(...), user: dict = Depends(current_user)) -> dict:
        session_of(pid, sid, user, "owner", "editor")
        guard(live, sid)
        base = body.get("base_revision")
        from ..graph import NeuronGraph
        new = guard(NeuronGraph.from_dict, body["graph"])
        rev = guard(db.save_snapshot, sid, graph_to_json(new), base_revision=None if base is None else int(base))
        store.sessions[sid] = new
        return {"revision": rev, "nodes": len(new.nodes), "edges": len(new.edges)}

    @app.get("/api/projects/{pid}/sessions/{sid}/revisions/{revision}")
    def revision(pid: str, sid: str, revision: int, user: dict = Depends(current_user)) -> dict:
        session_of(pid, sid, user)
        rev, text = guard(db.load_snapshot, sid, revision)
        return {"revision": rev, "graph": json.loads(text)}

    @app.delete("/api/projects/{pid}/sessions/{sid}")
    def drop_session(pid: str, sid: str, user: dict = Depends(current_user)) -> dict:
        session_of(pid, sid, user, "owner", "editor")
        if sid in store.sessions:
            store.delete_session(sid)
        db.delete_editor_session(sid)
        return {"deleted": sid}

    # -- runs -------------------------------------------------------------------------------------
    @app.post("/api/projects/{pid}/sessions/{sid}/runs")
    def start_run(pid: str, sid: str, body: dict = Body(...), user: dict = Depends(current_user)) -> dict:
        session_of(pid, sid, user, "owner", "editor")
        guard(live, sid)
        cfg = {"method": body.get("method", "sgd"), "steps": int(body.get("steps", 500)), "learning_rate": float(body.get("learning_rate", 0.5))}
        rid = guard(store.train_start, sid, body["inputs"], body["targets"], **cfg)
        db.record_run(rid, kind=cfg["method"], status="running", session_id=sid, project_id=pid, user_id=user["id"], config=cfg)
        return {"run_id": rid}

    @app.get("/api/projects/{pid}/runs")
    def runs(pid: str, user: dict = Depends(current_user)) -> list[dict]:
        guard(db.require_role, pid, user)
        out = db.runs(project_id=pid)
        for r in out:  # fold finished live runs into the table on the way
            lr = store.runs.get(r["id"])
            if lr is not None and r["status"] == "running" and lr.status not in ("queued", "running"):
                db.finish_run(r["id"], lr.status, lr.result, lr.error)
                if lr.status in ("finished", "stopped"):
                    db.save_snapshot(r["session_id"], graph_to_json(store.sessions[r["session_id"]]))
                r.update(status=lr.status, error=lr.error, result_json=json.dumps(lr.result) if lr.result is not None else None)
        return out

    @app.get("/api/runs/{rid}/events")
    def run_events(rid: str, user: dict = Depends(current_user)):
        if rid not in store.runs:
            raise HTTPException(status_code=404, detail=f"unknown run {rid!r}")
        rows = db.runs()
        row = next((r for r in rows if r["id"] == rid), None)
        if row is not None and row["project_id"]:
            guard(db.require_role, row["project_id"], user)
        run = store.runs[rid]

        def stream():
            sent = 0
            while True:
                hist = run.progress
                while sent < len(hist):
                    yield f"event: step\ndata: {json.dumps({'step': sent, 'loss': hist[sent]})}\n\n"
                    sent += 1
                if run.status not in ("queued", "running"):
                    yield f"event: done\ndata: {json.dumps(run.public())}\n\n"
                    return
                time.sleep(0.05)

        return StreamingResponse(stream(), media_type="text/event-stream", headers={"Cache-Control": "no-cache"})

    return current_user
