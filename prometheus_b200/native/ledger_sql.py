"""The experiment ledger in the reference's SQLite layout.

The C++ ledger (``native.ledger.Ledger``) keeps its rows in an append-only JSONL file. The
reference keeps them in one SQLite table (harness/ledger/src/lib.rs:94-104):

    records(experiment_id TEXT PRIMARY KEY NOT NULL, author_role TEXT NOT NULL,
            rung INTEGER, record_json TEXT NOT NULL)   + indexes on author_role and rung

``export_sqlite`` writes a ledger into a database file of exactly that layout (a file the
reference's ``Ledger::open`` reads as its own), ``import_sqlite`` appends the rows of such a
file, in insertion order, to a C++ ledger. Both go through the standard-library ``sqlite3``.
"""
from __future__ import annotations

import json
import sqlite3

SCHEMA = """
CREATE TABLE IF NOT EXISTS records (
    experiment_id TEXT PRIMARY KEY NOT NULL,
    author_role TEXT NOT NULL,
    rung INTEGER,
    record_json TEXT NOT NULL
);
CREATE INDEX IF NOT EXISTS idx_records_author_role ON records(author_role);
CREATE INDEX IF NOT EXISTS idx_records_rung ON records(rung);
"""

# field order of the reference's Record struct: serde writes record_json in this order
_FIELDS = ("experiment_id", "hypothesis", "prediction", "config_hash", "results", "delta_rci",
           "replication", "gpu_hours", "author_role", "rung", "created_at", "closed_at", "supersedes")


def _record_json(rec: dict) -> str:
    ordered = {k: rec.get(k) for k in _FIELDS}
    ordered.update({k: v for k, v in rec.items() if k not in ordered})
    return json.dumps(ordered, separators=(",", ":"), ensure_ascii=False)


def export_sqlite(ledger, path: str) -> int:
    """Write every row of ``ledger`` to the SQLite file ``path`` (created if missing; rows already
    there are kept, a duplicate ``experiment_id`` raises ``sqlite3.IntegrityError`` and nothing is
    written). Returns the number of rows written."""
    rows = [json.loads(r) for r in ledger.query("all")]
    con = sqlite3.connect(path)
    try:
        con.executescript(SCHEMA)
        with con:        # one transaction: all rows or none
            con.executemany(
                "INSERT INTO records (experiment_id, author_role, rung, record_json) VALUES (?, ?, ?, ?)",
                [(r["experiment_id"], r["author_role"], r.get("rung"), _record_json(r)) for r in rows])
    finally:
        con.close()
    return len(rows)


def import_sqlite(path: str, ledger) -> int:
    """Append the rows of the SQLite ledger ``path`` to ``ledger`` in insertion order (so a
    ``supersedes`` target precedes the row that names it). The ledger's own rules apply: a
    duplicate id or a missing ``supersedes`` target raises. Returns the number of rows appended."""
    con = sqlite3.connect(f"file:{path}?mode=ro", uri=True)
    try:
        rows = con.execute("SELECT experiment_id, author_role, rung, record_json FROM records ORDER BY rowid").fetchall()
    finally:
        con.close()
    for eid, role, rung, text in rows:
        rec = json.loads(text)
        if rec.get("experiment_id") != eid or rec.get("author_role") != role or rec.get("rung") != rung:
            raise ValueError(f"row {eid!r}: indexed columns disagree with record_json")
        ledger.append(json.dumps(rec))
    return len(rows)
