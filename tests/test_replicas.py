"""The N > 1 bookkeeping of the benchmark (barrier, max of times, sum of work) with two gloo ranks on the CPU."""
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import json, os, sys
sys.path.insert(0, {root!r})
from tacker_b200.replicas import Replicas
r = Replicas(backend="gloo")
r.barrier()
t = [2.0, 5.0][r.rank]                      # rank 1 is the slow one
out = dict(rank=r.rank, world=r.world, tmax=r.max(t), total=r.sum(10.0 * (r.rank + 1)),
           tput=r.throughput(100.0, t), names=r.gather("gpu%d" % r.rank))
r.barrier()
r.close()
print("RESULT " + json.dumps(out))
"""


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_ranks_agree_on_max_time_and_total_work(tmp_path):
    import json

    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    results = []
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0, err[-2000:]
        results.append(json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:]))
    for r in results:
        assert r["world"] == 2 and r["tmax"] == 5.0 and r["total"] == 30.0
        assert r["tput"] == 200.0 / 5.0                 # all ranks' work over the slowest rank's time
        assert r["names"] == ["gpu0", "gpu1"]


def test_single_process_is_the_identity():
    from tacker_b200.replicas import Replicas

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    r = Replicas()
    assert (r.rank, r.world) == (0, 1)
    assert r.max(3.5) == 3.5 and r.sum(2.0) == 2.0 and r.gather("x") == ["x"] and r.throughput(10.0, 2.0) == 5.0
    r.barrier()
    r.close()
