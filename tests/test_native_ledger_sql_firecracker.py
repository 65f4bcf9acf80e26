"""The ledger in the reference's SQLite layout (harness/ledger/src/lib.rs:94-104) and the
Firecracker backend gate of the sandbox pool (rl/envs/src/lib.rs:327-378)."""
import json
import sqlite3

import pytest

from prometheus_b200 import native
from prometheus_b200.native import ledger_sql


def _rec(eid, hyp, role="researcher", rung=None, **kw):
    r = {"experiment_id": eid, "hypothesis": hyp, "prediction": "p", "config_hash": "c" * 8, "results": None,
         "delta_rci": None, "replication": None, "gpu_hours": None, "author_role": role, "rung": rung,
         "created_at": "2026-01-01T00:00:00Z", "closed_at": None, "supersedes": None}
    r.update(kw)
    return json.dumps(r)


def test_ledger_round_trips_through_the_sqlite_layout(tmp_path):
    src = native.ledger.Ledger(str(tmp_path / "a.jsonl"))
    src.append(_rec("e1", "CHECK:muon lr transfer", rung=1))
    src.append(_rec("e2", "fp8 matches bf16", role="engineer", results={"passed": False}))
    src.append(_rec("e3", "fp8 matches bf16 after fix", supersedes="e2", rung=2))
    db = str(tmp_path / "ledger.sqlite")
    assert ledger_sql.export_sqlite(src, db) == 3
    con = sqlite3.connect(db)
    cols = [(c[1], c[2], c[3], c[5]) for c in con.execute("PRAGMA table_info(records)")]
    assert cols == [("experiment_id", "TEXT", 1, 1), ("author_role", "TEXT", 1, 0), ("rung", "INTEGER", 0, 0),
                    ("record_json", "TEXT", 1, 0)]
    idx = {r[1] for r in con.execute("PRAGMA index_list(records)")}
    assert {"idx_records_author_role", "idx_records_rung"} <= idx
    rows = con.execute("SELECT experiment_id, author_role, rung, record_json FROM records ORDER BY rowid").fetchall()
    assert [(r[0], r[1], r[2]) for r in rows] == [("e1", "researcher", 1), ("e2", "engineer", None), ("e3", "researcher", 2)]
    first = json.loads(rows[0][3])
    assert list(first)[:4] == ["experiment_id", "hypothesis", "prediction", "config_hash"]     # struct order
    assert con.execute("SELECT experiment_id FROM records WHERE rung = 2").fetchall() == [("e3",)]
    con.close()
    with pytest.raises(sqlite3.IntegrityError):
        ledger_sql.export_sqlite(src, db)                     # same ids again: nothing is written
    assert sqlite3.connect(db).execute("SELECT COUNT(*) FROM records").fetchone() == (3,)
    dst = native.ledger.Ledger(str(tmp_path / "b.jsonl"))
    assert ledger_sql.import_sqlite(db, dst) == 3
    assert [json.loads(r) for r in dst.query("all")] == [json.loads(r) for r in src.query("all")]
    with pytest.raises(native.NativeError):
        ledger_sql.import_sqlite(db, dst)                     # the ledger's duplicate rule still holds


def test_firecracker_backend_needs_kvm_and_boot_images(tmp_path):
    E = native.envs
    with pytest.raises(native.NativeError) as e:
        E.Pool.firecracker("sock", "vmlinux", "rootfs.ext4", kvm_device=str(tmp_path / "no-kvm"))
    assert e.value.kind == "Backend" and "kvm device missing" in str(e.value)
    kvm = tmp_path / "kvm"
    kvm.write_bytes(b"")
    kernel, rootfs = tmp_path / "vmlinux", tmp_path / "rootfs.ext4"
    pool = E.Pool.firecracker(str(tmp_path / "fc.sock"), str(kernel), str(rootfs), kvm_device=str(kvm))
    assert pool.backend == "firecracker" and pool.firecracker_paths[1] == str(kernel)
    assert E.Pool().backend == "in_process" and E.Pool().firecracker_paths is None
    img = E.Image("img", {"/work/a.txt": b"x"}, {}, {})
    pool.register_image(img)
    with pytest.raises(native.NativeError) as e:
        pool.snapshot_from_image("img")
    assert e.value.kind == "Backend" and "kernel image missing" in str(e.value)
    kernel.write_bytes(b"k")
    with pytest.raises(native.NativeError) as e:
        pool.snapshot_from_image("img")
    assert "rootfs image missing" in str(e.value)
    rootfs.write_bytes(b"r")
    snap = pool.snapshot_from_image("img")                    # same isolation as the in-process engine
    a, b = pool.fork_pair(snap)
    assert pool.live_count() == 2 and pool.agent_view(a) == pool.agent_view(b)
