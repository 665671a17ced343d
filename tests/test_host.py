"""The C++ host runtime without a GPU: builds, and its self-test (recording double of the device library) passes."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "tacker_b200", "host")


def test_host_selftest_passes():
    from tacker_b200 import _build

    exe = _build.build_host_selftest()
    out = subprocess.run([exe, os.path.join(HOST, "tests", "config")], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "0 failed" in out.stdout


def test_aker_builds_and_reports_missing_gpu_loudly():
    import torch

    from tacker_b200 import _build

    _build.build_library()
    exe = _build.build_host()
    assert exe and os.path.exists(exe)
    usage = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert usage.returncode == 0 and "-s <system_name> -m <model_name>" in usage.stdout
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the loud-failure path needs a machine without one")
    run = subprocess.run([exe, "-s", "aker", "-m", "vgg16", "-c", os.path.join(HOST, "config")], capture_output=True,
                         text=True, timeout=120)
    assert run.returncode == 1 and "[ERROR]" in run.stderr     # no device: an error, never a CPU path


def test_config_files_keep_the_reference_keys():
    import json

    for model in ("vgg16", "resnet50", "bert"):
        d = json.load(open(os.path.join(HOST, "config", f"kinfo-{model}.json")))
        for pair in ("tzgemm_cp", "tzgemm_stencil", "tzgemm_mriq"):
            assert {"gridsize", "blocksize", "block_ratio", "4096"} <= set(d[pair])
        assert set(d["throughput_test"]) == {"a", "b"}
        for k in ("cp", "stencil", "mriq"):
            assert {"register", "shared_memory", "blocksize", "ori_blks"} <= set(d[k])
