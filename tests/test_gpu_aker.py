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
    # the scheduler fuses: in both modes some layers carried best-effort blocks and that saved time
    mixes = re.findall(r"execed be blks: (\d+), mix times: (\d+)/(\d+), time earned: ([\d.]+)", out.stdout)
    assert len(mixes) == 2
    for blks, fused, mixable, earned in mixes:
        assert 0 <= int(fused) <= int(mixable)
        if model == "vgg16":
            assert int(blks) > 0 and int(fused) > 0 and float(earned) > 0.0
    # stage 2 ran best-effort kernels in the leftover budget and reports what ran
    stage2 = re.findall(r"\[Stage2\] (\d+) solo launches in the ([\d.]+) ms left: (\d+) blocks of \w+, (\d+) blocks of \w+, "
                        r"([\d.]+) ms of device time", out.stdout)
    assert len(stage2) == 2
    for launches, window, b1, b2, ms in stage2:
        assert int(launches) > 0 and int(b1) > 0 and int(b2) > 0 and 0 < float(ms) <= float(window) * 1.05


def test_one_best_effort_kernel_variant(cuda, tmp_path):
    """execute_with_one_cd_kernel (src/TaskManager.cu:717-1005): whole rounds of blocks from block 0, no stage 2."""
    out = subprocess.run([_aker(), "-s", "aker", "-m", "vgg16", "-c", os.path.join(HOST, "config"), "--one-cd"],
                         capture_output=True, text=True, timeout=600, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    m = re.search(r"execed be blks: (\d+), mix times: (\d+)/16, time earned: ([\d.]+)", out.stdout)
    assert m and int(m.group(1)) > 0 and int(m.group(2)) > 0
    assert re.search(r"\[Result\] Aker throughput [\d.]+ \+ [\d.]+ = [\d.]+ ms", out.stdout) and "[Stage2]" not in out.stdout


def test_fused_colocation_beats_time_slicing_within_qos(cuda, tmp_path):
    """Request-driven co-location with the benchmark kernel as the best-effort job: layers of the LC pass carry
    best-effort blocks, the latency bound holds in both phases, and riding does not cost throughput."""
    out = subprocess.run([_aker(), "-s", "aker", "-m", "vgg16", "-c", os.path.join(HOST, "config"), "--colocate-fused", "4",
                          "--qps", "200", "--qos", "1.5"], capture_output=True, text=True, timeout=600, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    r = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert r["mixable_layers"] == 16 and r["fused_layers"] > 0 and r["blocks_per_fused_query"] > 0
    assert r["timesliced"]["qos_met"] and r["fused"]["qos_met"]
    assert r["fused"]["fused_queries"] > 0 and r["fused"]["be_blocks_in_lc"] > 0
    assert r["fused"]["be_blocks_per_s"] >= 0.98 * r["timesliced"]["be_blocks_per_s"]


def test_colocation_meets_qos(cuda, tmp_path):
    # 10 s per phase: the bound is 1.5 x the p99 of the solo phase, and a p99 over a few hundred queries is too noisy
    out = subprocess.run([_aker(), "-s", "aker", "-m", "vgg16", "-c", os.path.join(HOST, "config"), "--colocate", "10",
                          "--qps", "200", "--qos", "1.5", "--be", "bert"], capture_output=True, text=True, timeout=600,
                         cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    r = json.loads(line)
    assert r["lc_served"] > 1500 and r["be_queries"] > 0 and r["be_qps"] > 0
    assert r["lc_p99_ms"] >= r["lc_p50_ms"] > 0
    assert r["qos_met"] is True and r["lc_p99_ms"] <= r["qos_bound_ms"], r


def test_vgg16_scores_match_the_cpu_forward(cuda, oracle, tmp_path):
    """The whole LC model, end to end: the class scores `aker` computes on its seeded input and weights against
    a numpy forward of the same network (fp16 operands, fp32 accumulation), within 1e-2 of the largest score."""
    import numpy as np

    import vgg16_numpy

    dump = tmp_path / "vgg16_result.bin"
    out = subprocess.run([_aker(), "-s", "aker", "-m", "vgg16", "-c", os.path.join(HOST, "config"), "--dump-output",
                          str(dump), "--colocate", "0.2"], capture_output=True, text=True, timeout=600, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    got = np.fromfile(dump, dtype=np.float32)
    assert got.size == 2000
    scores, probs = vgg16_numpy.forward(oracle)
    scale = float(np.abs(scores).max())
    assert scale > 0 and np.isfinite(got).all()
    assert np.abs(got[:1000] - scores).max() <= 1e-2 * scale
    assert int(np.argmax(got[:1000])) == int(np.argmax(scores))
    assert np.abs(got[1000:] - probs).max() <= 1e-2 * float(probs.max())
    assert abs(float(got[1000:].sum()) - 1.0) <= 1e-4


def _dump_of(model, tmp_path):
    import numpy as np

    dump = tmp_path / (model + "_result.bin")
    out = subprocess.run([_aker(), "-s", "aker", "-m", model, "-c", os.path.join(HOST, "config"), "--dump-output",
                          str(dump), "--colocate", "0.2"], capture_output=True, text=True, timeout=900, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    return np.fromfile(dump, dtype=np.float32)


def test_resnet50_scores_match_the_cpu_forward(cuda, oracle, tmp_path):
    """ResNet-50 end to end (53 convolutions of four shapes, 16 residual additions, one dense layer): the class scores
    of `aker` against a numpy forward of the same seeded network, within 1e-2 of the largest score."""
    import numpy as np

    import resnet50_numpy

    got = _dump_of("resnet50", tmp_path)
    want = resnet50_numpy.forward(oracle)
    assert got.size == want.size == 1000 and np.isfinite(got).all()
    scale = float(np.abs(want).max())
    assert scale > 0 and np.abs(got - want).max() <= 1e-2 * scale
    assert int(np.argmax(got)) == int(np.argmax(want))


def test_bert_hidden_states_match_the_cpu_forward(cuda, oracle, tmp_path):
    """BERT-base end to end (12 layers, batch 8, 128 tokens: dense layers, batched attention products, softmax, GELU,
    layer normalisation): the last hidden states of `aker` against a numpy forward of the same seeded encoder."""
    import numpy as np

    import bert_numpy

    got = _dump_of("bert", tmp_path)
    want = bert_numpy.forward(oracle)
    assert got.size == want.size == 8 * 128 * 768 and np.isfinite(got).all()
    scale = float(np.abs(want).max())
    err = np.abs(got.reshape(want.shape) - want)
    assert err.max() <= 2e-2 * scale and float(np.sqrt((err ** 2).mean())) <= 2e-3 * scale


def test_model_from_description_and_constant_files(cuda, tmp_path):
    """A model read from a description with NNFusion-style constant files (raw fp32: filters [3][3][Cin][Cout], dense
    weights [in][out]) -- what the reference's generated classes do with Constant_<n>_0.bin
    (src/dnn/vgg16/vgg16_kernel_class.h:378-391): the scores `aker` computes against a numpy forward of the same files."""
    import numpy as np

    import graph_numpy
    from tacker_b200 import nnf

    layers = [{"op": "conv3x3", "out": 64, "act": "relu"}, {"op": "conv3x3", "out": 64, "act": "relu"}, {"op": "maxpool"},
              {"op": "conv3x3", "out": 128, "act": "relu"}, {"op": "maxpool"}, {"op": "dense", "out": 256, "act": "relu"},
              {"op": "dense", "out": 10, "act": "none"}, {"op": "softmax"}]
    x = np.random.default_rng(3).standard_normal((32, 32, 3)).astype(np.float32)
    model = nnf.write_model(str(tmp_path / "m"), "tiny", 32, 32, 3, layers, nnf.random_constants(layers, 32, 32, 3, seed=5),
                            input_array=x)
    dump = tmp_path / "result.bin"
    out = subprocess.run([_aker(), "-s", "aker", "-m", model, "-c", os.path.join(HOST, "config"), "--dump-output", str(dump),
                          "--colocate", "0.2"], capture_output=True, text=True, timeout=600, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    got = np.fromfile(dump, dtype=np.float32)
    assert got.size == 20
    scores, probs = graph_numpy.forward(model, x)
    scale = float(np.abs(scores).max())
    assert scale > 0 and np.abs(got[:10] - scores).max() <= 1e-2 * scale
    assert int(np.argmax(got[:10])) == int(np.argmax(scores)) and np.abs(got[10:] - probs).max() <= 1e-2
    # a constant of the wrong size is refused with the file's name, as the reference's loader refuses a missing file
    with open(tmp_path / "m" / "Constant" / "Constant_1_0.bin", "ab") as f:
        f.write(b"\0\0\0\0")
    bad = subprocess.run([_aker(), "-s", "aker", "-m", model, "-c", os.path.join(HOST, "config")], capture_output=True,
                         text=True, timeout=600, cwd=tmp_path)
    assert bad.returncode != 0 and "Constant_1_0.bin" in bad.stdout + bad.stderr


def test_scheduler_launches_a_generated_module(cuda, tmp_path):
    """Generator -> runtime: a fused kernel emitted for one thread ratio, compiled into a module and registered
    under the pair's key replaces the library's kernel in the scheduler's fused launches
    (reference: generated kernels become src/mix_kernel/*.cu and are picked via the model file, src/TaskManager.cu:253-264)."""
    from tacker_b200.fusion import data, gen_run

    c = [x for x in data.fuse_kernel_info("mriq") if x.r2 == 16][0]
    so = gen_run.compile_module(gen_run.emit(c, str(tmp_path)))
    out = subprocess.run([_aker(), "-s", "aker", "-m", "bert", "-c", os.path.join(HOST, "config"), "--be-kernel", "mriq",
                          "--mix-module", f"tzgemm_mriq={so}"], capture_output=True, text=True, timeout=600, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    m = re.search(r"fused kernels launched through generated modules: (\d+)", out.stdout)
    assert m and int(m.group(1)) > 0
    m = re.search(r"execed be blks: (\d+), mix times: (\d+)/48", out.stdout)    # 4 products per layer
    assert m and int(m.group(1)) > 0 and int(m.group(2)) > 0
    assert "device status word" not in out.stdout + out.stderr


@pytest.mark.parametrize("a,b", [("cutcp", "fft"), ("lbm", "sgemm")])
def test_scheduler_with_the_other_parboil_kernels(cuda, tmp_path, a, b):
    """sgemm, lbm, fft and cutcp as the best-effort pair (src/Creator.cu:53-178): the experiment runs in both modes,
    stage 2 launches the solo kernels, and the pairs whose measured ratios are not zero ride along LC layers."""
    out = subprocess.run([_aker(), "-s", "both", "-m", "vgg16", "-c", os.path.join(HOST, "config"), "--be-kernel", a,
                          "--be-kernel2", b], capture_output=True, text=True, timeout=600, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    results = re.findall(r"\[Result\] (Aker|Tacker) BE task took ([\d.]+) \+ ([\d.eE+-]+)", out.stdout)
    assert [r[0] for r in results] == ["Aker", "Tacker"]
    mixes = re.findall(r"execed be blks: (\d+), mix times: (\d+)/(\d+), time earned: ([\d.]+)", out.stdout)
    assert len(mixes) == 2 and all(0 <= int(f) <= int(m) for _, f, m, _ in mixes)
    # whether a layer carries blocks is the scheduler's call (a quarter region of cutcp or half a block of sgemm outlasts
    # most VGG16 layers, so it mostly declines); what ran must be accounted for
    stage2 = re.findall(r"\[Stage2\] (\d+) solo launches in the ([\d.]+) ms left: (\d+) blocks of (\w+), (\d+) blocks of (\w+)",
                        out.stdout)
    assert len(stage2) == 2 and all(s[3] == a and s[5] == b for s in stage2)
    assert "device status word" not in out.stdout + out.stderr


def test_bert_as_the_lc_task(cuda, tmp_path):
    """The reference also schedules its BERT graph as the latency-critical task (src/main.cu:227-244)."""
    out = subprocess.run([_aker(), "-s", "tacker", "-m", "bert", "-c", os.path.join(HOST, "config")], capture_output=True,
                         text=True, timeout=600, cwd=tmp_path)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert re.search(r"\[Result\] Tacker BE task took", out.stdout)
    m = re.search(r"mix times: (\d+)/(\d+)", out.stdout)
    assert m and int(m.group(2)) == 48          # 12 layers x 4 tzgemm-backed products (fused q-k-v, projection, two feed-forward)


def test_resource_query_for_every_key(cuda):
    import tacker_b200
    from tacker_b200 import ops

    for key in tacker_b200.KEYS:
        info = ops.query(key)
        assert info.regs_per_thread > 0 and info.max_ctas_per_sm >= 1 and info.nparams > 0, key
        if key.startswith(("tzgemm_", "tzconv_", "gptb_tzgemm", "gptb_tzconv")):
            assert info.threads_tensor == 192 and info.tmem_columns == 512 and info.dynamic_smem > 100000
        else:
            assert info.threads_tensor == 0 and info.threads_cd_min == 32
    with pytest.raises(tacker_b200.TackerError):
        ops.query("gptb_hot3d")
