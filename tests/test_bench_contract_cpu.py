"""bench.py's contract, as far as it can be checked without a GPU: the workload table, the clock-sample
parser, and the reference arm (`--impl reference`), which runs the reference's CPU build (or the C oracle)
on the host cores and must print ONE JSON line with the agreed keys."""
import importlib.util
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_module():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_workload_table():
    bench = _bench_module()
    assert bench.WORKLOAD is bench.WORKLOADS["base_seq128"]          # the headline workload is the default
    for name, w in bench.WORKLOADS.items():
        for key in ("model", "seq", "batch", "seed", "scaling", "outputs", "metric", "text"):
            assert key in w, (name, key)
        assert w["scaling"] in ("weak", "strong")
    assert bench.WORKLOADS["base_seq128"]["seq"] == 128 and bench.WORKLOADS["base_seq128"]["batch"] == 256
    assert bench.WORKLOADS["large_seq512"]["scaling"] == "strong"
    assert set(bench.NCU_TRAFFIC_BYTES) >= {"bias_gelu", "bias_residual_ln", "masked_softmax", "embed_ln"}


def test_clock_samples_are_parsed(tmp_path):
    bench = _bench_module()
    sampler = bench.ClockSampler.__new__(bench.ClockSampler)
    sampler.path = str(tmp_path / "clocks.csv")
    with open(sampler.path, "w") as f:
        f.write("0, 345, 1965, 140.2, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active\n")
        f.write("0, 1650, 1965, 980.5, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n")
        f.write("0, 1590, 1965, 990.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n")
        f.write("garbage line\n")

    class Done:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

    sampler.proc = Done()
    sampler.out = open(os.devnull, "w")
    got = sampler.stop()
    assert got["sm_mhz"] == 1620.0 and got["sm_max_mhz"] == 1965.0       # median of the samples under load
    assert got["reasons"] == ["sw_power_cap"] and got["samples"] == 3


@pytest.mark.parametrize("workload", ["base_seq128", "base_seq32_f32"])
def test_reference_arm_prints_one_contract_line(workload):
    env = dict(os.environ, CUBERT_BENCH_CPU_THREADS="4")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "1", "--workload", workload], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                          universal_newlines=True, env=env, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["value"] > 0 and line["unit"] == "sequences/s"
    assert line["higher_is_better"] is True and line["data"] == "synthetic" and line["vs_baseline"] is None
    assert line["metric"] == _bench_module().WORKLOADS[workload]["metric"]
    assert "workload" in line["config"]
    base = line["cpu_baseline"]
    assert base["kind"] in ("reference", "port") and base["cores"] == 4 and base["value"] == line["value"]
    assert "sample" in base
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_a_bench_process_sees_one_gpu_whatever_the_launcher_left_visible():
    """The library builds a replica on every visible GPU, a bench process times one: the process narrows
    CUDA_VISIBLE_DEVICES to its own entry, also when it is the only process on an 8-GPU machine."""
    bench = _bench_module()
    # a single process, WORLD_SIZE unset, eight GPUs visible (explicitly or by default)
    env = {"CUDA_VISIBLE_DEVICES": "0,1,2,3,4,5,6,7"}
    assert bench.narrow_to_one_gpu(env, 0) == "0" and env["CUDA_VISIBLE_DEVICES"] == "0"
    assert env["CUBERT_BENCH_PARENT_VISIBLE"] == "0,1,2,3,4,5,6,7"
    env = {}
    assert bench.narrow_to_one_gpu(env, 0) == "0" and env["CUDA_VISIBLE_DEVICES"] == "0"
    # a launcher that hands out a subset: rank 1 of four on GPUs 4..7
    env = {"CUDA_VISIBLE_DEVICES": "4,5,6,7"}
    assert bench.narrow_to_one_gpu(env, 1) == "5" and env["CUDA_VISIBLE_DEVICES"] == "5"
    # narrowing twice (a re-entered process) keeps the first choice
    assert bench.narrow_to_one_gpu(env, 1) == "5"
    # ranks without a list take their own number; UUID entries pass through
    assert bench.device_for_rank("", 3) == "3" and bench.device_for_rank(None, 0) == "0"
    assert bench.device_for_rank("GPU-aaaa,GPU-bbbb", 1) == "GPU-bbbb"
    assert bench.device_for_rank("2", 5) == "5"


def test_ncu_traffic_is_only_reported_for_what_was_captured():
    """roofline.traffic is a figure from one ncu capture: it must vanish when the workload, the kernel library's
    version or a kernel-selection switch differs from what was captured."""
    bench = _bench_module()
    v = bench.NCU_TRAFFIC_SOURCE["cubk_version"]
    got = bench.ncu_traffic("bias_gelu", "base_seq128", v, True)
    assert got["bytes"] == bench.NCU_TRAFFIC["bias_gelu"]["bytes"] and got["profile"].startswith("profiles/")
    assert os.path.exists(os.path.join(ROOT, got["profile"]))
    assert bench.ncu_traffic("bias_gelu", "large_seq512", v, True) is None
    assert bench.ncu_traffic("bias_gelu", "base_seq128", v + 1, True) is None
    assert bench.ncu_traffic("bias_gelu", "base_seq128", v, False) is None
    assert bench.ncu_traffic("mean_pool", "base_seq128", v, True) is None
    assert bench.switches_at_defaults({"PATH": "/bin"}) and not bench.switches_at_defaults({"CUBERT_KEY_GEMM": "1"})
    from cubert_b200 import kernels
    assert kernels.load().cubk_version() == v, "kernel library version changed: re-capture or clear bench.NCU_TRAFFIC"
