"""Accounts, projects, revisioned snapshots and run events of the REST platform (CPU only)."""
import json

import pytest

from neuralfn_b200.server.platform_db import AuthError, PersistenceWorker, PlatformDB, RevisionConflict, hash_password, verify_password


def test_password_hashing_and_login_tokens():
    h = hash_password("correct horse")
    assert verify_password("correct horse", h) and not verify_password("wrong horse", h) and not verify_password("x", "garbage")
    with pytest.raises(ValueError):
        hash_password("short")
    db = PlatformDB()
    assert db.ensure_bootstrap_admin("Root@Example.org", "admin-password")["is_admin"]
    assert db.ensure_bootstrap_admin("other@example.org", "admin-password") is None  # only when empty
    with pytest.raises(AuthError):
        db.login("root@example.org", "nope-nope")
    with pytest.raises(AuthError):
        db.login("nobody@example.org", "admin-password")
    tok, user = db.login("root@example.org", "admin-password")
    assert db.authenticate(tok)["email"] == "root@example.org"
    db.logout(tok)
    with pytest.raises(AuthError):
        db.authenticate(tok)
    short = PlatformDB(session_ttl_seconds=-1.0)
    short.create_user("a@b.c", "password1")
    with pytest.raises(AuthError):
        short.authenticate(short.login("a@b.c", "password1")[0])
    with pytest.raises(ValueError):
        db.create_user("root@example.org", "another-password")


def test_projects_roles_snapshots_and_grants():
    db = PlatformDB()
    owner = db.create_user("o@x.io", "password1")
    guest = db.create_user("g@x.io", "password2")
    p = db.create_project(owner["id"], "demo")
    assert db.role(p["id"], owner) == "owner" and db.role(p["id"], guest) is None
    with pytest.raises(AuthError):
        db.require_role(p["id"], guest)
    db.set_member(p["id"], guest["id"], "viewer")
    with pytest.raises(AuthError):
        db.require_role(p["id"], guest, "owner", "editor")
    assert [x["id"] for x in db.projects_for(guest)] == [p["id"]]
    with pytest.raises(ValueError):
        db.set_member(p["id"], owner["id"], "viewer")
    s = db.create_editor_session(p["id"], "g", '{"v": 1}')
    assert db.save_snapshot(s["id"], '{"v": 2}', base_revision=1) == 2
    with pytest.raises(RevisionConflict) as e:
        db.save_snapshot(s["id"], '{"v": 3}', base_revision=1)
    assert e.value.current == 2
    assert db.load_snapshot(s["id"]) == (2, '{"v": 2}') and db.load_snapshot(s["id"], 1)[1] == '{"v": 1}'
    for i in range(30):
        db.save_snapshot(s["id"], json.dumps({"v": 3 + i}), keep=5)
    with pytest.raises(KeyError):
        db.load_snapshot(s["id"], 2)
    d = db.register_dataset("tiny", "bytes", "/data/tiny", {"train_tokens": 10})
    db.grant_dataset(p["id"], d["id"])
    assert [x["name"] for x in db.datasets_for_project(p["id"])] == ["tiny"]
    db.grant_dataset(p["id"], d["id"], granted=False)
    assert db.datasets_for_project(p["id"]) == []
    db.record_run("r1", kind="sgd", status="running", session_id=s["id"], project_id=p["id"])
    db.finish_run("r1", "finished", {"final_loss": 0.1})
    assert db.runs(project_id=p["id"])[0]["status"] == "finished"
    db.delete_project(p["id"])  # cascades
    with pytest.raises(KeyError):
        db.editor_session(s["id"])


def test_persistence_worker_flushes_dirty_sessions():
    db = PlatformDB()
    u = db.create_user("o@x.io", "password1")
    s = db.create_editor_session(db.create_project(u["id"], "p")["id"], "g", "{}")
    pending = [[(s["id"], '{"a": 1}'), ("unknown", "{}")]]
    w = PersistenceWorker(db, lambda: pending.pop() if pending else [], interval=0.01).start()
    w.stop()
    assert w.saved == 1 and db.load_snapshot(s["id"]) == (2, '{"a": 1}')


def test_rest_accounts_flow(tmp_path):
    pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient

    import importlib.util
    from pathlib import Path

    from neuralfn_b200.server.app import create_app
    spec = importlib.util.spec_from_file_location("xor_graph_example", Path(__file__).resolve().parents[1] / "examples" / "xor_graph.py")
    xor = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(xor)
    db = PlatformDB(str(tmp_path / "platform.sqlite"))
    db.ensure_bootstrap_admin("admin@x.io", "admin-password")
    app = create_app(db=db)
    c = TestClient(app)
    assert c.get("/api/bootstrap").json()["accounts"] is True
    assert c.get("/api/sessions").status_code == 401 and c.get("/api/projects").status_code == 401
    assert c.post("/api/auth/login", json={"email": "admin@x.io", "password": "wrong-password"}).status_code == 401
    assert c.post("/api/auth/login", json={"email": "admin@x.io", "password": "admin-password"}).status_code == 200
    assert c.get("/api/auth/me").json()["user"]["is_admin"] and c.get("/api/sessions").status_code == 200
    uid = c.post("/api/admin/users", json={"email": "eve@x.io", "password": "eve-password"}).json()["id"]
    pid = c.post("/api/projects", json={"name": "xor"}).json()["id"]
    g = xor.build_xor_graph().to_dict()
    sid = c.post(f"/api/projects/{pid}/sessions", json={"name": "xor", "graph": g}).json()["id"]
    got = c.get(f"/api/projects/{pid}/sessions/{sid}/graph").json()
    assert got["revision"] == 1 and len(got["graph"]["nodes"]) == len(g["nodes"])
    assert c.put(f"/api/projects/{pid}/sessions/{sid}/graph", json={"graph": g, "base_revision": 1}).json()["revision"] == 2
    r = c.put(f"/api/projects/{pid}/sessions/{sid}/graph", json={"graph": g, "base_revision": 1})
    assert r.status_code == 409 and r.json()["detail"]["current_revision"] == 2
    assert c.get(f"/api/projects/{pid}/sessions/{sid}/revisions/1").json()["revision"] == 1

    rid = c.post(f"/api/projects/{pid}/sessions/{sid}/runs", json={"inputs": [[0, 0], [0, 1], [1, 0], [1, 1]], "targets": [[0], [1], [1], [0]],
                                                                    "steps": 20}).json()["run_id"]
    with c.stream("GET", f"/api/runs/{rid}/events") as resp:
        text = "".join(resp.iter_text())
    assert text.count("event: step") == 20 and "event: done" in text
    runs = c.get(f"/api/projects/{pid}/runs").json()
    assert runs[0]["id"] == rid and runs[0]["status"] == "finished"
    assert db.editor_session(sid)["revision"] == 3  # the trained graph was snapshotted

    # a second user sees nothing until invited, and a viewer cannot write
    e = TestClient(app)
    e.post("/api/auth/login", json={"email": "eve@x.io", "password": "eve-password"})
    assert e.get("/api/projects").json() == [] and e.get(f"/api/projects/{pid}").status_code == 403 and e.get("/api/admin/users").status_code == 403
    assert c.put(f"/api/projects/{pid}/members/{uid}", json={"role": "viewer"}).status_code == 200
    assert e.get(f"/api/projects/{pid}").status_code == 200
    assert e.put(f"/api/projects/{pid}/sessions/{sid}/graph", json={"graph": g}).status_code == 403
    c.post(f"/api/admin/users/{uid}/active", json={"active": False})
    assert e.get("/api/projects").status_code == 401
    assert c.post("/api/auth/logout").status_code == 200 and c.get("/api/auth/me").status_code == 401

    # a new process finds the sessions again
    app2 = create_app(db=PlatformDB(str(tmp_path / "platform.sqlite")))
    c2 = TestClient(app2)
    c2.post("/api/auth/login", json={"email": "admin@x.io", "password": "admin-password"})
    assert c2.get(f"/api/projects/{pid}/sessions/{sid}/graph").json()["revision"] == 3


def test_flat_session_routes_respect_project_membership(tmp_path):
    """The flat /api/sessions routes address the same live store as project-bound sessions: a signed-in
    user without a membership must not list, read, overwrite, run or delete another project's session."""
    from fastapi.testclient import TestClient

    from neuralfn_b200.server.app import create_app
    from neuralfn_b200.server.platform_db import PlatformDB
    db = PlatformDB(str(tmp_path / "p.db"))
    db.create_user("admin@example.org", "root-pass-1", is_admin=True)
    db.create_user("a@example.org", "alice-pass-1")
    db.create_user("b@example.org", "bobby-pass-1")
    app = create_app(db=db)
    alice, bob = TestClient(app), TestClient(app)
    assert alice.post("/api/auth/login", json={"email": "a@example.org", "password": "alice-pass-1"}).status_code == 200
    assert bob.post("/api/auth/login", json={"email": "b@example.org", "password": "bobby-pass-1"}).status_code == 200
    pid = alice.post("/api/projects", json={"name": "secret"}).json()["id"]
    sid = alice.post(f"/api/projects/{pid}/sessions", json={"name": "g"}).json()["id"]
    # the owner sees it through both route families
    assert alice.get(f"/api/sessions/{sid}/graph").status_code == 200
    assert any((r.get("id") or r.get("session_id")) == sid for r in alice.get("/api/sessions").json())
    # a stranger does not
    assert all((r.get("id") or r.get("session_id")) != sid for r in bob.get("/api/sessions").json())
    assert bob.get(f"/api/sessions/{sid}/graph").status_code == 404
    assert bob.put(f"/api/sessions/{sid}/graph", json={"name": "x", "nodes": {}, "edges": {}}).status_code == 404
    assert bob.post(f"/api/sessions/{sid}/runs", json={"inputs": [[0.0]], "targets": [[0.0]]}).status_code == 404
    assert bob.delete(f"/api/sessions/{sid}").status_code == 404
    assert alice.get(f"/api/sessions/{sid}/graph").status_code == 200      # still there
    # writes to a project-bound session must keep the revision check: the flat PUT refuses
    assert alice.put(f"/api/sessions/{sid}/graph", json={"name": "x", "nodes": {}, "edges": {}}).status_code == 409
    # flat sessions belong to their creator
    own = bob.post("/api/sessions", json={"name": "mine"}).json()["session_id"]
    assert bob.get(f"/api/sessions/{own}/graph").status_code == 200
    assert alice.get(f"/api/sessions/{own}/graph").status_code == 404
    # dataset paths: only granted assets
    assert bob.post("/api/datasets/info", json={"path": str(tmp_path)}).status_code == 403
