"""Relational side of the platform: accounts, cookie sessions, projects and memberships, editor
sessions with revisioned graph snapshots, dataset assets with per-project grants, and the
record of training runs - on SQLite through the standard library.

Passwords are stored as PBKDF2-HMAC-SHA256 (salted, 200k iterations); a login hands out a random
token of which only the SHA-256 is stored, with an expiry. The first account can be created from
``NEURALFN_BOOTSTRAP_ADMIN_EMAIL`` / ``NEURALFN_BOOTSTRAP_ADMIN_PASSWORD`` (``ensure_bootstrap_admin``).
Graph snapshots carry a revision number per editor session; ``save_snapshot`` with a stale
``base_revision`` raises ``RevisionConflict`` (the REST layer answers 409).

``PersistenceWorker`` is the background thread that copies dirty live sessions into snapshots.

Behavioural counterparts: ``server/db_models.py`` (User, AuthSession, Project,
ProjectMembership, DatasetAsset, ProjectDatasetGrant, EditorSession, SessionSnapshot,
TrainingRun), ``server/security.py``, ``server/services/auth_service.py``,
``server/services/persistence_worker.py``.
"""
from __future__ import annotations

import hashlib
import hmac
import json
import os
import secrets
import sqlite3
import threading
import time
import uuid
from typing import Any, Callable

__all__ = ["PlatformDB", "RevisionConflict", "AuthError", "PersistenceWorker", "hash_password", "verify_password"]

_SCHEMA = """
CREATE TABLE IF NOT EXISTS schema_version (version INTEGER NOT NULL);
CREATE TABLE IF NOT EXISTS users (id TEXT PRIMARY KEY, email TEXT UNIQUE NOT NULL, password_hash TEXT NOT NULL, display_name TEXT NOT NULL DEFAULT '',
    is_admin INTEGER NOT NULL DEFAULT 0, is_active INTEGER NOT NULL DEFAULT 1, created REAL NOT NULL);
CREATE TABLE IF NOT EXISTS auth_sessions (token_sha256 TEXT PRIMARY KEY, user_id TEXT NOT NULL REFERENCES users(id) ON DELETE CASCADE,
    created REAL NOT NULL, expires REAL NOT NULL);
CREATE TABLE IF NOT EXISTS projects (id TEXT PRIMARY KEY, name TEXT NOT NULL, description TEXT NOT NULL DEFAULT '', owner_id TEXT NOT NULL REFERENCES users(id),
    created REAL NOT NULL);
CREATE TABLE IF NOT EXISTS project_memberships (project_id TEXT NOT NULL REFERENCES projects(id) ON DELETE CASCADE,
    user_id TEXT NOT NULL REFERENCES users(id) ON DELETE CASCADE, role TEXT NOT NULL, PRIMARY KEY (project_id, user_id));
CREATE TABLE IF NOT EXISTS dataset_assets (id TEXT PRIMARY KEY, name TEXT NOT NULL, variant TEXT NOT NULL, path TEXT NOT NULL, manifest_json TEXT NOT NULL,
    owner_id TEXT REFERENCES users(id), created REAL NOT NULL, UNIQUE (name, variant));
CREATE TABLE IF NOT EXISTS project_dataset_grants (project_id TEXT NOT NULL REFERENCES projects(id) ON DELETE CASCADE,
    dataset_id TEXT NOT NULL REFERENCES dataset_assets(id) ON DELETE CASCADE, PRIMARY KEY (project_id, dataset_id));
CREATE TABLE IF NOT EXISTS editor_sessions (id TEXT PRIMARY KEY, project_id TEXT NOT NULL REFERENCES projects(id) ON DELETE CASCADE, name TEXT NOT NULL,
    revision INTEGER NOT NULL DEFAULT 0, created REAL NOT NULL, updated REAL NOT NULL);
CREATE TABLE IF NOT EXISTS session_snapshots (session_id TEXT NOT NULL REFERENCES editor_sessions(id) ON DELETE CASCADE, revision INTEGER NOT NULL,
    graph_json TEXT NOT NULL, created REAL NOT NULL, PRIMARY KEY (session_id, revision));
CREATE TABLE IF NOT EXISTS training_runs (id TEXT PRIMARY KEY, session_id TEXT, project_id TEXT, user_id TEXT, kind TEXT NOT NULL, status TEXT NOT NULL,
    config_json TEXT NOT NULL DEFAULT '{}', result_json TEXT, error TEXT, created REAL NOT NULL, finished REAL);
"""
SCHEMA_VERSION = 1
ROLES = ("owner", "editor", "viewer")
_PBKDF2_ROUNDS = 200_000
_DUMMY_HASH: str | None = None


class RevisionConflict(RuntimeError):
    def __init__(self, current: int) -> None:
        super().__init__(f"the session is at revision {current}")
        self.current = current


class AuthError(PermissionError):
    pass


def hash_password(password: str, *, salt: bytes | None = None, rounds: int = _PBKDF2_ROUNDS) -> str:
    if len(password) < 8:
        raise ValueError("passwords need at least 8 characters")
    salt = salt or secrets.token_bytes(16)
    dk = hashlib.pbkdf2_hmac("sha256", password.encode("utf-8"), salt, rounds)
    return f"pbkdf2_sha256${rounds}${salt.hex()}${dk.hex()}"


def verify_password(password: str, stored: str) -> bool:
    try:
        scheme, rounds, salt, digest = stored.split("$")
        if scheme != "pbkdf2_sha256":
            return False
        dk = hashlib.pbkdf2_hmac("sha256", password.encode("utf-8"), bytes.fromhex(salt), int(rounds))
        return hmac.compare_digest(dk.hex(), digest)
    except (ValueError, TypeError):
        return False


def _token_digest(token: str) -> str:
    return hashlib.sha256(token.encode("utf-8")).hexdigest()


class PlatformDB:
    """One SQLite file (``":memory:"`` for tests). All methods are safe to call from several
    threads: one connection guarded by a lock, foreign keys on, every mutation in a transaction."""

    def __init__(self, path: str = ":memory:", *, session_ttl_seconds: float = 14 * 24 * 3600.0) -> None:
        self._db = sqlite3.connect(path, check_same_thread=False, isolation_level=None)
        self._db.row_factory = sqlite3.Row
        self._lock = threading.RLock()
        self.session_ttl = float(session_ttl_seconds)
        with self._lock:
            self._db.execute("PRAGMA foreign_keys = ON")
            self._db.executescript(_SCHEMA)
            row = self._db.execute("SELECT version FROM schema_version").fetchone()
            if row is None:
                self._db.execute("INSERT INTO schema_version VALUES (?)", (SCHEMA_VERSION,))
            elif row["version"] > SCHEMA_VERSION:
                raise RuntimeError(f"database schema {row['version']} is newer than this build ({SCHEMA_VERSION})")

    def close(self) -> None:
        with self._lock:
            self._db.close()

    # -- helpers ------------------------------------------------------------------------------------
    def _tx(self, fn: Callable[[sqlite3.Connection], Any]) -> Any:
        with self._lock:
            self._db.execute("BEGIN IMMEDIATE")
            try:
                out = fn(self._db)
                self._db.execute("COMMIT")
                return out
            except BaseException:
                self._db.execute("ROLLBACK")
                raise

    def _one(self, sql: str, args: tuple = ()) -> dict | None:
        with self._lock:
            r = self._db.execute(sql, args).fetchone()
        return dict(r) if r is not None else None

    def _all(self, sql: str, args: tuple = ()) -> list[dict]:
        with self._lock:
            return [dict(r) for r in self._db.execute(sql, args).fetchall()]

    @staticmethod
    def _public_user(u: dict) -> dict:
        return {k: u[k] for k in ("id", "email", "display_name", "created")} | {"is_admin": bool(u["is_admin"]), "is_active": bool(u["is_active"])}

    # -- accounts -----------------------------------------------------------------------------------
    def create_user(self, email: str, password: str, *, display_name: str = "", is_admin: bool = False) -> dict:
        email = email.strip().lower()
        if "@" not in email or len(email) > 254:
            raise ValueError("not an e-mail address")
        uid = uuid.uuid4().hex
        try:
            self._tx(lambda db: db.execute("INSERT INTO users (id, email, password_hash, display_name, is_admin, created) VALUES (?,?,?,?,?,?)",
                                           (uid, email, hash_password(password), display_name, int(is_admin), time.time())))
        except sqlite3.IntegrityError:
            raise ValueError(f"an account for {email} exists") from None
        return self.user(uid)

    def user(self, uid: str) -> dict:
        u = self._one("SELECT * FROM users WHERE id = ?", (uid,))
        if u is None:
            raise KeyError(f"unknown user {uid!r}")
        return self._public_user(u)

    def list_users(self) -> list[dict]:
        return [self._public_user(u) for u in self._all("SELECT * FROM users ORDER BY created")]

    def set_user_active(self, uid: str, active: bool) -> dict:
        self.user(uid)

        def work(db):
            db.execute("UPDATE users SET is_active = ? WHERE id = ?", (int(active), uid))
            if not active:
                db.execute("DELETE FROM auth_sessions WHERE user_id = ?", (uid,))
        self._tx(work)
        return self.user(uid)

    def ensure_bootstrap_admin(self, email: str | None = None, password: str | None = None) -> dict | None:
        """Creates the first administrator when the table is empty; the values default to the
        ``NEURALFN_BOOTSTRAP_ADMIN_*`` environment variables. Returns the account or ``None``."""
        email = email or os.environ.get("NEURALFN_BOOTSTRAP_ADMIN_EMAIL")
        password = password or os.environ.get("NEURALFN_BOOTSTRAP_ADMIN_PASSWORD")
        if not email or not password or self._one("SELECT id FROM users LIMIT 1") is not None:
            return None
        return self.create_user(email, password, display_name="admin", is_admin=True)

    def login(self, email: str, password: str) -> tuple[str, dict]:
        """(session token, user). The same error for an unknown account and a wrong password."""
        u = self._one("SELECT * FROM users WHERE email = ?", (email.strip().lower(),))
        global _DUMMY_HASH
        if _DUMMY_HASH is None:
            _DUMMY_HASH = hash_password("not a password", salt=b"\0" * 16)
        ok = verify_password(password, u["password_hash"] if u else _DUMMY_HASH) and u is not None  # same work either way
        if not u or not ok or not u["is_active"]:
            raise AuthError("wrong e-mail or password")
        token = secrets.token_urlsafe(32)
        now = time.time()
        self._tx(lambda db: (db.execute("DELETE FROM auth_sessions WHERE expires < ?", (now,)),
                             db.execute("INSERT INTO auth_sessions VALUES (?,?,?,?)", (_token_digest(token), u["id"], now, now + self.session_ttl))))
        return token, self._public_user(u)

    def authenticate(self, token: str | None) -> dict:
        if not token:
            raise AuthError("not signed in")
        row = self._one("SELECT u.* , s.expires AS expires FROM auth_sessions s JOIN users u ON u.id = s.user_id WHERE s.token_sha256 = ?",
                        (_token_digest(token),))
        if row is None or row["expires"] < time.time() or not row["is_active"]:
            raise AuthError("the session has expired")
        return self._public_user(row)

    def logout(self, token: str) -> None:
        self._tx(lambda db: db.execute("DELETE FROM auth_sessions WHERE token_sha256 = ?", (_token_digest(token),)))

    # -- projects -----------------------------------------------------------------------------------
    def create_project(self, owner_id: str, name: str, description: str = "") -> dict:
        if not name.strip():
            raise ValueError("a project needs a name")
        pid = uuid.uuid4().hex[:16]

        def work(db):
            db.execute("INSERT INTO projects VALUES (?,?,?,?,?)", (pid, name.strip(), description, owner_id, time.time()))
            db.execute("INSERT INTO project_memberships VALUES (?,?,?)", (pid, owner_id, "owner"))
        self._tx(work)
        return self.project(pid)

    def project(self, pid: str) -> dict:
        p = self._one("SELECT * FROM projects WHERE id = ?", (pid,))
        if p is None:
            raise KeyError(f"unknown project {pid!r}")
        p["members"] = self._all("SELECT m.user_id, u.email, m.role FROM project_memberships m JOIN users u ON u.id = m.user_id WHERE m.project_id = ? ORDER BY u.email",
                                 (pid,))
        return p

    def projects_for(self, user: dict) -> list[dict]:
        if user["is_admin"]:
            return self._all("SELECT * FROM projects ORDER BY created")
        return self._all("SELECT p.* FROM projects p JOIN project_memberships m ON m.project_id = p.id WHERE m.user_id = ? ORDER BY p.created", (user["id"],))

    def role(self, pid: str, user: dict) -> str | None:
        if user["is_admin"]:
            return "owner"
        r = self._one("SELECT role FROM project_memberships WHERE project_id = ? AND user_id = ?", (pid, user["id"]))
        return r["role"] if r else None

    def require_role(self, pid: str, user: dict, *allowed: str) -> str:
        self.project(pid)
        r = self.role(pid, user)
        if r is None or (allowed and r not in allowed):
            raise AuthError(f"needs one of {allowed or ROLES} on project {pid}")
        return r

    def set_member(self, pid: str, user_id: str, role: str | None) -> dict:
        """``role=None`` removes the member. The owner's own membership cannot be changed."""
        p = self.project(pid)
        self.user(user_id)
        if user_id == p["owner_id"]:
            raise ValueError("the owner's membership is fixed")
        if role is None:
            self._tx(lambda db: db.execute("DELETE FROM project_memberships WHERE project_id = ? AND user_id = ?", (pid, user_id)))
        else:
            if role not in ROLES[1:]:
                raise ValueError(f"role must be one of {ROLES[1:]}")
            self._tx(lambda db: db.execute("INSERT INTO project_memberships VALUES (?,?,?) ON CONFLICT (project_id, user_id) DO UPDATE SET role = excluded.role",
                                           (pid, user_id, role)))
        return self.project(pid)

    def delete_project(self, pid: str) -> None:
        self.project(pid)
        self._tx(lambda db: db.execute("DELETE FROM projects WHERE id = ?", (pid,)))

    # -- editor sessions and snapshots --------------------------------------------------------------
    def create_editor_session(self, pid: str, name: str, graph_json: str, *, session_id: str | None = None) -> dict:
        self.project(pid)
        sid = session_id or uuid.uuid4().hex[:12]
        now = time.time()

        def work(db):
            db.execute("INSERT INTO editor_sessions VALUES (?,?,?,?,?,?)", (sid, pid, name, 1, now, now))
            db.execute("INSERT INTO session_snapshots VALUES (?,?,?,?)", (sid, 1, graph_json, now))
        self._tx(work)
        return self.editor_session(sid)

    def editor_session(self, sid: str) -> dict:
        s = self._one("SELECT * FROM editor_sessions WHERE id = ?", (sid,))
        if s is None:
            raise KeyError(f"unknown session {sid!r}")
        return s

    def editor_sessions(self, pid: str) -> list[dict]:
        return self._all("SELECT * FROM editor_sessions WHERE project_id = ? ORDER BY created", (pid,))

    def save_snapshot(self, sid: str, graph_json: str, *, base_revision: int | None = None, keep: int = 20) -> int:
        """Stores a new revision and returns its number. With ``base_revision`` the write only
        succeeds when that is still the latest revision. Only the newest ``keep`` are retained."""
        def work(db):
            row = db.execute("SELECT revision FROM editor_sessions WHERE id = ?", (sid,)).fetchone()
            if row is None:
                raise KeyError(f"unknown session {sid!r}")
            cur = row["revision"]
            if base_revision is not None and base_revision != cur:
                raise RevisionConflict(cur)
            now = time.time()
            db.execute("INSERT INTO session_snapshots VALUES (?,?,?,?)", (sid, cur + 1, graph_json, now))
            db.execute("UPDATE editor_sessions SET revision = ?, updated = ? WHERE id = ?", (cur + 1, now, sid))
            db.execute("DELETE FROM session_snapshots WHERE session_id = ? AND revision <= ?", (sid, cur + 1 - keep))
            return cur + 1
        return self._tx(work)

    def load_snapshot(self, sid: str, revision: int | None = None) -> tuple[int, str]:
        if revision is None:
            revision = self.editor_session(sid)["revision"]
        r = self._one("SELECT graph_json FROM session_snapshots WHERE session_id = ? AND revision = ?", (sid, revision))
        if r is None:
            raise KeyError(f"session {sid!r} has no revision {revision}")
        return revision, r["graph_json"]

    def delete_editor_session(self, sid: str) -> None:
        self.editor_session(sid)
        self._tx(lambda db: db.execute("DELETE FROM editor_sessions WHERE id = ?", (sid,)))

    # -- datasets -----------------------------------------------------------------------------------
    def register_dataset(self, name: str, variant: str, path: str, manifest: dict, owner_id: str | None = None) -> dict:
        did = uuid.uuid4().hex[:16]
        try:
            self._tx(lambda db: db.execute("INSERT INTO dataset_assets VALUES (?,?,?,?,?,?,?)",
                                           (did, name, variant, path, json.dumps(manifest), owner_id, time.time())))
        except sqlite3.IntegrityError:
            raise ValueError(f"dataset {name}/{variant} is already registered") from None
        return self._one("SELECT * FROM dataset_assets WHERE id = ?", (did,))

    def grant_dataset(self, pid: str, dataset_id: str, granted: bool = True) -> None:
        self.project(pid)
        if self._one("SELECT id FROM dataset_assets WHERE id = ?", (dataset_id,)) is None:
            raise KeyError(f"unknown dataset {dataset_id!r}")
        if granted:
            self._tx(lambda db: db.execute("INSERT OR IGNORE INTO project_dataset_grants VALUES (?,?)", (pid, dataset_id)))
        else:
            self._tx(lambda db: db.execute("DELETE FROM project_dataset_grants WHERE project_id = ? AND dataset_id = ?", (pid, dataset_id)))

    def datasets_for_project(self, pid: str) -> list[dict]:
        return self._all("SELECT d.id, d.name, d.variant, d.path FROM dataset_assets d JOIN project_dataset_grants g ON g.dataset_id = d.id "
                         "WHERE g.project_id = ? ORDER BY d.name, d.variant", (pid,))

    # -- training runs ------------------------------------------------------------------------------
    def record_run(self, run_id: str, *, kind: str, status: str, session_id: str | None = None, project_id: str | None = None, user_id: str | None = None,
                   config: dict | None = None) -> None:
        self._tx(lambda db: db.execute("INSERT INTO training_runs (id, session_id, project_id, user_id, kind, status, config_json, created) VALUES (?,?,?,?,?,?,?,?)",
                                       (run_id, session_id, project_id, user_id, kind, status, json.dumps(config or {}), time.time())))

    def finish_run(self, run_id: str, status: str, result: dict | None = None, error: str | None = None) -> None:
        self._tx(lambda db: db.execute("UPDATE training_runs SET status = ?, result_json = ?, error = ?, finished = ? WHERE id = ?",
                                       (status, json.dumps(result) if result is not None else None, error, time.time(), run_id)))

    def runs(self, *, project_id: str | None = None, session_id: str | None = None) -> list[dict]:
        sql, args = "SELECT * FROM training_runs", []
        conds = [(c, v) for c, v in (("project_id", project_id), ("session_id", session_id)) if v is not None]
        if conds:
            sql += " WHERE " + " AND ".join(f"{c} = ?" for c, _ in conds)
            args = [v for _, v in conds]
        return self._all(sql + " ORDER BY created", tuple(args))


class PersistenceWorker:
    """Copies live sessions that changed since their last snapshot into the database, every
    ``interval`` seconds and once more on ``stop``. ``dirty()`` yields (session id, graph JSON)
    pairs and is expected to clear its own marks; sessions unknown to the database are skipped."""

    def __init__(self, db: PlatformDB, dirty: Callable[[], list[tuple[str, str]]], interval: float = 2.0) -> None:
        self.db, self.dirty, self.interval = db, dirty, interval
        self.saved = 0
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def flush(self) -> int:
        n = 0
        for sid, text in self.dirty():
            try:
                self.db.save_snapshot(sid, text)
                n += 1
            except KeyError:
                continue
        self.saved += n
        return n

    def start(self) -> "PersistenceWorker":
        def loop() -> None:
            while not self._stop.wait(self.interval):
                self.flush()
        self._thread = threading.Thread(target=loop, daemon=True, name="persistence-worker")
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5.0)
        self.flush()
