"""The multi-replica bookkeeping (brasa_b200/replicas.py) on CPU: two gloo ranks as child processes."""
import os
import socket
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

CHILD = r"""
import json, sys
sys.path.insert(0, {root!r})
from brasa_b200.replicas import Replicas, whole_job_rate
r = Replicas("gloo")
r.barrier()
mine = r.sessions_of_rank(7)
out = {{"rank": r.rank, "world": r.world, "max": r.max(1.5 + r.rank), "sum": r.sum(10 * (r.rank + 1)), "sessions": mine,
       "rate": whole_job_rate(100.0 * (r.rank + 1), 2.0 + r.rank, r)}}
r.barrier()
r.close()
print(json.dumps(out))
"""


def test_two_gloo_ranks_reduce_and_share_sessions(tmp_path):
    import json
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=str(ROOT)))
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        o, e = p.communicate(timeout=120)
        assert p.returncode == 0, e
        outs.append(json.loads(o.strip().splitlines()[-1]))
    outs.sort(key=lambda d: d["rank"])
    assert [d["world"] for d in outs] == [2, 2]
    assert all(d["max"] == 2.5 and d["sum"] == 30.0 for d in outs)
    assert outs[0]["sessions"] == [0, 2, 4, 6] and outs[1]["sessions"] == [1, 3, 5]
    # 100 + 200 units over the slower replica's 3 seconds
    assert all(abs(d["rate"] - 100.0) < 1e-9 for d in outs)


def test_single_process_is_its_own_world(monkeypatch):
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    sys.path.insert(0, str(ROOT))
    from brasa_b200.replicas import Replicas, whole_job_rate
    r = Replicas()
    assert (r.rank, r.world) == (0, 1) and r.max(3.0) == 3.0 and r.sum(4.0) == 4.0
    assert r.sessions_of_rank(3) == [0, 1, 2] and whole_job_rate(10.0, 2.0, r) == 5.0
