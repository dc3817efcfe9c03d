"""Host-side checks of ``bench.py``: the byte accounting behind the roofline
numbers and the reference arm's JSON line (which runs without a GPU)."""

import importlib.util
import json
import subprocess
import sys

import pytest
import torch

from conftest import REPO


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("rln_bench", REPO / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_algorithmic_bytes_per_row(bench):
    # fp16 branch, float32 normalized, dropout on: (12 + 2 + 1/8) H + 8 and (16 + 2 + 1/8) H + 8
    expected = {128: (1816, 2328), 256: (3624, 4648), 384: (5432, 6968), 512: (7240, 9288),
                768: (10856, 13928), 1024: (14472, 18568)}
    for hidden, (forward, backward) in expected.items():
        assert bench.forward_bytes_per_row(hidden, 2, True) == forward
        assert bench.backward_bytes_per_row(hidden, 2, True) == backward
    # fp32 branch adds 2 bytes per element to each direction, no dropout removes the mask
    assert bench.forward_bytes_per_row(768, 4, True) == 10856 + 2 * 768
    assert bench.backward_bytes_per_row(768, 4, True) == 13928 + 2 * 768
    assert bench.forward_bytes_per_row(768, 2, False) == 10856 - 768 // 8
    # a 16-bit normalized removes 2 bytes per element from each direction
    assert bench.forward_bytes_per_row(768, 2, True, 2) == 9320
    assert bench.backward_bytes_per_row(768, 2, True, 2) == 12392


def test_workload_table(bench):
    rows, hidden, branch_dtype, dropout_p, normalized_dtype = bench.workload("h768_64Mi")
    assert (rows, hidden, branch_dtype, dropout_p) == (87381, 768, torch.float16, 0.1)
    assert normalized_dtype == torch.float32
    assert rows * hidden >= 64 * 2 ** 20 - hidden          # "64 Mi elements"
    assert bench.workload("h768_64Mi_bf16_normalized")[4] == torch.bfloat16
    for name in bench.WORKLOADS:
        fields = bench.workload(name)
        assert len(fields) == 5 and fields[1] in (128, 256, 384, 512, 768, 1024)
        config = bench.workload_config(name, 2)
        assert config["workload"] == name and config["rows_total"] == 2 * fields[0]
        assert "model" not in config
    assert set(bench.NCU_BACKWARD_TRAFFIC_BYTES) <= set(bench.WORKLOADS)


def test_reference_arm_prints_one_json_line():
    completed = subprocess.run(
        [sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--steps", "1",
         "--warmup", "0", "--workload", "c2_3x1367x128_fp32"],
        capture_output=True, text=True, timeout=300, check=True,
    )
    lines = [line for line in completed.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference"
    assert record["unit"] == "rows/s" and record["higher_is_better"] is True
    assert record["value"] > 0 and record["n_gpus"] == 1 and record["steps"] == 1
    assert record["config"]["workload"] == "c2_3x1367x128_fp32"
    # the reference's own package when oracle/build_ref.py has installed it, else the port
    installed = (REPO / "oracle" / "_ref" / "gfx1010_kernels" / "normalization.py").exists()
    assert record["cpu_baseline"]["kind"] == ("reference" if installed else "port")
    assert record["cpu_baseline"]["cores"] >= 1
    assert record["cpu_baseline"]["value"] == record["value"]
    assert record["e2e"] == {
        "value": record["value"], "unit": "rows/s",
        "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
    }
    assert record["gpu_launches"] == 0 and record["vs_baseline"] is None


def test_reference_arm_under_torchrun_prints_on_rank_0_only():
    completed = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
         "--master-addr", "127.0.0.1", "--master-port", "29631",
         str(REPO / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
         "--warmup", "0", "--workload", "c2_5x817x256_fp32"],
        capture_output=True, text=True, timeout=600, check=True,
    )
    lines = [line for line in completed.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference" and record["n_gpus"] == 2
    assert record["config"]["rows_total"] == 2 * 5 * 817


def test_cpu_arm_falls_back_to_the_port_without_the_reference_package(bench, monkeypatch, tmp_path):
    monkeypatch.setattr(bench, "REFERENCE_PACKAGE_DIR", tmp_path)
    times, threads, kind = bench.time_cpu_reference(64, 128, torch.float16, 0.1, 1, 0)
    assert kind == "port" and len(times) == 1 and threads >= 1


def test_clock_summary_names_the_window_it_used(bench):
    sampler = bench.ClockSampler(0)
    sampler.max_mhz = 1965
    sampler.samples = [(1.0, 1900, 0), (2.0, 1800, 0x4), (3.0, 1700, 0x4), (9.0, 1000, 0x1)]
    inner = sampler.summary([("timed regions", 1.5, 3.5), ("whole run", 0.0, 10.0)])
    assert inner["window"] == "timed regions" and inner["samples"] == 2
    assert inner["sm_mhz"] == 1750 and inner["reasons"] == ["sw_power_cap"]
    # a span with fewer than two samples is skipped, and the label says which one was used
    outer = sampler.summary([("timed regions", 2.5, 3.5), ("whole run", 0.0, 10.0)])
    assert outer["window"] == "whole run" and outer["samples"] == 4
    nothing = sampler.summary([("timed regions", 20.0, 30.0)])
    assert nothing["window"] == "all samples of the run" and nothing["samples"] == 4
    empty = bench.ClockSampler(0)
    assert empty.summary([("timed regions", 0.0, 1.0)])["window"] == "no samples"
