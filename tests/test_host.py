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


def test_profile_ratios_writes_the_reference_schema(tmp_path):
    """profile_ratios.write_configs: the measured tables land in every model file under the reference's keys
    ("<K>": ratio, block_ratio = the K = 4096 entry, best_block_ratio, launch shapes), without touching the source files."""
    import json

    from tacker_b200 import profile_ratios

    table = {str(k): {"ratio": 0.001 * (i + 1), "blocks": 8, "gemm_us": 1.0, "cd_us": 1.0, "fused_us": 1.5,
                      "fused_vs_sequential": 0.75} for i, k in enumerate(profile_ratios.KS)}
    table["2304"]["ratio"] = 0.0                                # a pair / K where fusing did not pay: never fused
    result = {"tzgemm_mrif": {"cd_us_per_block": 0.25, "cd_threads": 704, "solo_shape": (2, 512), "blocks": 1024,
                              "fused_us_by_cd_threads": {"704": 10.0}, "table": table}}
    before = {p: open(os.path.join(HOST, "config", p)).read() for p in os.listdir(os.path.join(HOST, "config"))}
    touched = profile_ratios.write_configs(result, out_dir=str(tmp_path))
    assert sorted(os.path.basename(p) for p in touched) == ["kinfo-bert.json", "kinfo-resnet50.json", "kinfo-vgg16.json"]
    for p in touched:
        cfg = json.load(open(p))
        e = cfg["tzgemm_mrif"]
        assert e["gridsize"] == 1 and e["blocksize"] == 192 + 704
        assert [e[str(k)] for k in profile_ratios.KS] == [0.001, 0.002, 0.003, 0.0, 0.005, 0.006]
        assert e["block_ratio"] == e["4096"] == 0.005 and e["best_block_ratio"] == 0.006
        assert cfg["mrif"]["gridsize"] == 2 and cfg["mrif"]["blocksize"] == 512 and cfg["mrif"]["ori_blks"] == 1024
        assert "throughput_test" in cfg and "tzgemm_stencil" in cfg          # everything else is carried over
    after = {p: open(os.path.join(HOST, "config", p)).read() for p in os.listdir(os.path.join(HOST, "config"))}
    assert before == after
