"""Supervisor (restart-on-spare) with CPU ranks: failures are made on the host (a rank that exits non-zero, a rank
whose heartbeat stops); no GPU is involved."""
import os
import sys
import textwrap

from ml_b200.parallel.launch import Supervisor


def _script(tmp_path, body):
    p = tmp_path / "child.py"
    p.write_text(textwrap.dedent(body))
    return str(p)


def test_failed_rank_is_restarted_on_spare(tmp_path):
    marker = tmp_path / "log.txt"
    child = _script(tmp_path, f"""
        import os, sys
        r, att, dev = os.environ["RANK"], int(os.environ["ENTROPY_ATTEMPT"]), os.environ["LOCAL_RANK"]
        open({str(marker)!r}, "a").write(f"{{att}} {{r}} {{dev}}\\n")
        if att == 0 and r == "1":
            sys.exit(17)          # first attempt: rank 1 dies
    """)
    logs = []
    sup = Supervisor(2, [child], spare=1, max_restarts=2, log=logs.append, poll_s=0.05)
    assert sup.run() == 0
    assert sup.attempts == 1 and sup.retired == [1] and sup.devices == [0, 2]
    lines = marker.read_text().split("\n")
    assert "1 1 2" in lines          # second attempt: rank 1 runs on the spare device 2
    assert any("exited with code 17" in l for l in logs)


def test_restart_budget_and_no_spare(tmp_path):
    child = _script(tmp_path, "import sys; sys.exit(3)")
    sup = Supervisor(1, [child], spare=0, max_restarts=1, log=lambda *_: None, poll_s=0.05)
    assert sup.run() == 1 and sup.attempts == 2


def test_stale_heartbeat_counts_as_failure(tmp_path):
    hb = tmp_path / "hb"
    hb.mkdir()
    child = _script(tmp_path, """
        import os, time
        att = int(os.environ["ENTROPY_ATTEMPT"])
        p = os.path.join(os.environ["ENTROPY_HEARTBEAT_DIR"], "rank_" + os.environ["RANK"])
        if att == 0:
            open(p, "w").close()
            time.sleep(30)            # hangs without touching its heartbeat again
        else:
            open(p, "w").close()
    """)
    logs = []
    sup = Supervisor(1, [child], spare=1, max_restarts=1, heartbeat_dir=str(hb), heartbeat_timeout=1.0, log=logs.append, poll_s=0.1)
    assert sup.run() == 0
    assert any("heartbeat is stale" in l for l in logs) and sup.devices == [1]
