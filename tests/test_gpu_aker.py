"""The `aker` binary on a GPU: the reference's experiment and the request-driven co-location (B200 only)."""
import json
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "tacker_b200", "host")


def _aker():
    from tacker_b200 import _build

    exe = os.path.join(_build.LIB_DIR, "aker")
    assert os.path.exists(exe), "aker was not built (python -m tacker_b200._build)"
    return exe


@pytest.mark.parametrize("model", ["vgg16", "resnet50"])
def test_reference_experiment_runs_both_modes(cuda, model, tmp_path):
    out = subprocess.run([_aker(), "-s", "both", "-m", model, "-c", os.path.join(HOST, "config")], capture_output=True,
                         text=True, timeout=600, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    results = re.findall(r"\[Result\] (Aker|Tacker) BE task took ([\d.]+) \+ ([\d.eE+-]+)", out.stdout)
    assert [r[0] for r in results] == ["Aker", "Tacker"]
    assert all(float(r[1]) >= 0 for r in results)
    assert "mix times:" in out.stdout and os.path.exists(tmp_path / "recorder_output.txt")


def test_colocation_meets_qos(cuda, tmp_path):
    out = subprocess.run([_aker(), "-s", "aker", "-m", "vgg16", "-c", os.path.join(HOST, "config"), "--colocate", "3",
                          "--qps", "200", "--qos", "1.5", "--be", "bert"], capture_output=True, text=True, timeout=600,
                         cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    r = json.loads(line)
    assert r["lc_served"] > 400 and r["be_queries"] > 0 and r["be_qps"] > 0
    assert r["lc_p99_ms"] >= r["lc_p50_ms"] > 0


def test_bert_as_the_lc_task(cuda, tmp_path):
    """The reference also schedules its BERT graph as the latency-critical task (src/main.cu:227-244)."""
    out = subprocess.run([_aker(), "-s", "tacker", "-m", "bert", "-c", os.path.join(HOST, "config")], capture_output=True,
                         text=True, timeout=600, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert re.search(r"\[Result\] Tacker BE task took", out.stdout)
    m = re.search(r"mix times: (\d+)/(\d+)", out.stdout)
    assert m and int(m.group(2)) == 72          # 12 layers x 6 tzgemm-backed dense layers


def test_resource_query_for_every_key(cuda):
    import tacker_b200
    from tacker_b200 import ops

    for key in tacker_b200.KEYS:
        info = ops.query(key)
        assert info.regs_per_thread > 0 and info.max_ctas_per_sm >= 1 and info.nparams > 0, key
        if key.startswith("tzgemm_") or key.startswith("gptb_tzgemm"):
            assert info.threads_tensor == 192 and info.tmem_columns == 512 and info.dynamic_smem > 100000
        else:
            assert info.threads_tensor == 0 and info.threads_cd_min == 32
    with pytest.raises(tacker_b200.TackerError):
        ops.query("gptb_fft")
