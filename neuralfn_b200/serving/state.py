"""SQLite store behind the stateful endpoints (``/v1/responses``, ``/v1/conversations``).

One file, WAL mode, a ``meta`` table carrying the schema version; every public method opens a
short transaction on a connection guarded by a lock (the server runs one worker thread plus
the event loop). Stored payloads are JSON text; ids are opaque strings generated here.

Behavioural counterpart: ``neuralfn/native_state.py`` (schema v4).
"""
from __future__ import annotations

import json
import secrets
import sqlite3
import threading
import time
from pathlib import Path
from typing import Any

__all__ = ["StateStore", "SCHEMA_VERSION"]

SCHEMA_VERSION = 4

_DDL = """
CREATE TABLE IF NOT EXISTS meta (key TEXT PRIMARY KEY, value TEXT NOT NULL);
CREATE TABLE IF NOT EXISTS conversations (id TEXT PRIMARY KEY, created_at REAL NOT NULL, metadata TEXT NOT NULL);
CREATE TABLE IF NOT EXISTS items (id TEXT PRIMARY KEY, conversation_id TEXT NOT NULL REFERENCES conversations(id) ON DELETE CASCADE,
                                  seq INTEGER NOT NULL, created_at REAL NOT NULL, payload TEXT NOT NULL);
CREATE INDEX IF NOT EXISTS items_by_conversation ON items(conversation_id, seq);
CREATE TABLE IF NOT EXISTS responses (id TEXT PRIMARY KEY, created_at REAL NOT NULL, conversation_id TEXT, previous_response_id TEXT,
                                      status TEXT NOT NULL, payload TEXT NOT NULL);
"""


def _new_id(prefix: str) -> str:
    return f"{prefix}_{secrets.token_hex(12)}"


class StateStore:
    def __init__(self, path: str | Path = ":memory:") -> None:
        self.path = str(path)
        if self.path != ":memory:":
            Path(self.path).parent.mkdir(parents=True, exist_ok=True)
        self._db = sqlite3.connect(self.path, check_same_thread=False, isolation_level=None)
        self._lock = threading.RLock()
        with self._lock:
            self._db.execute("PRAGMA foreign_keys = ON")
            if self.path != ":memory:":
                self._db.execute("PRAGMA journal_mode = WAL")
            self._db.executescript(_DDL)
            row = self._db.execute("SELECT value FROM meta WHERE key = 'schema_version'").fetchone()
            if row is None:
                self._db.execute("INSERT INTO meta(key, value) VALUES ('schema_version', ?)", (str(SCHEMA_VERSION),))
            elif int(row[0]) > SCHEMA_VERSION:
                raise RuntimeError(f"state database has schema {row[0]}, this build understands up to {SCHEMA_VERSION}")
            elif int(row[0]) < SCHEMA_VERSION:
                self._db.execute("UPDATE meta SET value = ? WHERE key = 'schema_version'", (str(SCHEMA_VERSION),))

    def close(self) -> None:
        with self._lock:
            self._db.close()

    def schema_version(self) -> int:
        with self._lock:
            return int(self._db.execute("SELECT value FROM meta WHERE key = 'schema_version'").fetchone()[0])

    # -- conversations ---------------------------------------------------------------------
    def create_conversation(self, metadata: dict | None = None, items: list[dict] | None = None) -> dict:
        cid, now = _new_id("conv"), time.time()
        with self._lock:
            self._db.execute("BEGIN")
            self._db.execute("INSERT INTO conversations(id, created_at, metadata) VALUES (?, ?, ?)", (cid, now, json.dumps(metadata or {})))
            self._db.execute("COMMIT")
        if items:
            self.add_items(cid, items)
        return self.get_conversation(cid)

    def get_conversation(self, cid: str) -> dict | None:
        with self._lock:
            row = self._db.execute("SELECT id, created_at, metadata FROM conversations WHERE id = ?", (cid,)).fetchone()
        if row is None:
            return None
        return {"id": row[0], "object": "conversation", "created_at": int(row[1]), "metadata": json.loads(row[2])}

    def delete_conversation(self, cid: str) -> bool:
        with self._lock:
            cur = self._db.execute("DELETE FROM conversations WHERE id = ?", (cid,))
            return cur.rowcount > 0

    def add_items(self, cid: str, items: list[dict]) -> list[dict]:
        out = []
        with self._lock:
            if self._db.execute("SELECT 1 FROM conversations WHERE id = ?", (cid,)).fetchone() is None:
                raise KeyError(cid)
            self._db.execute("BEGIN")
            seq = self._db.execute("SELECT COALESCE(MAX(seq), -1) FROM items WHERE conversation_id = ?", (cid,)).fetchone()[0]
            for it in items:
                seq += 1
                iid = it.get("id") or _new_id("item")
                payload = dict(it, id=iid)
                self._db.execute("INSERT INTO items(id, conversation_id, seq, created_at, payload) VALUES (?, ?, ?, ?, ?)",
                                 (iid, cid, seq, time.time(), json.dumps(payload)))
                out.append(payload)
            self._db.execute("COMMIT")
        return out

    def list_items(self, cid: str, limit: int = 1000) -> list[dict]:
        with self._lock:
            rows = self._db.execute("SELECT payload FROM items WHERE conversation_id = ? ORDER BY seq LIMIT ?", (cid, limit)).fetchall()
        return [json.loads(r[0]) for r in rows]

    # -- responses -------------------------------------------------------------------------
    def put_response(self, payload: dict[str, Any], *, conversation_id: str | None = None, previous_response_id: str | None = None) -> dict:
        rid = payload.get("id") or _new_id("resp")
        payload = dict(payload, id=rid)
        with self._lock:
            self._db.execute("INSERT OR REPLACE INTO responses(id, created_at, conversation_id, previous_response_id, status, payload) "
                             "VALUES (?, ?, ?, ?, ?, ?)",
                             (rid, time.time(), conversation_id, previous_response_id, payload.get("status", "completed"), json.dumps(payload)))
        return payload

    def get_response(self, rid: str) -> dict | None:
        with self._lock:
            row = self._db.execute("SELECT payload FROM responses WHERE id = ?", (rid,)).fetchone()
        return None if row is None else json.loads(row[0])

    def delete_response(self, rid: str) -> bool:
        with self._lock:
            return self._db.execute("DELETE FROM responses WHERE id = ?", (rid,)).rowcount > 0

    def response_chain(self, rid: str, limit: int = 64) -> list[dict]:
        """The response and its ancestors through ``previous_response_id``, oldest first."""
        chain: list[dict] = []
        with self._lock:
            cur: str | None = rid
            while cur and len(chain) < limit:
                row = self._db.execute("SELECT payload, previous_response_id FROM responses WHERE id = ?", (cur,)).fetchone()
                if row is None:
                    break
                chain.append(json.loads(row[0]))
                cur = row[1]
        return chain[::-1]
