"""Command line of the *_perf binaries (csrc/perf/perf_main.cu): every flag of the rccl-tests harness
(common.cpp:1343-1513) is accepted, bad values are refused before any GPU work. Runs without a GPU:
only paths that end before the first CUDA call are exercised."""
import subprocess

import pytest

from rocm_systems_b200.utils import build


@pytest.fixture(scope="module")
def perf_bin():
    outs = build.build_perf()
    by_name = {p.name: p for p in outs}
    assert "all_reduce_perf" in by_name
    return by_name


def test_usage_lists_every_flag(perf_bin):
    out = subprocess.run([str(perf_bin["all_reduce_perf"]), "-h"], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0
    for flag in ["-g", "-b", "-e", "-i", "-f", "-n", "-w", "-m", "-N", "-c", "-o", "-d", "-r", "-z", "-G", "-C", "-a", "-R", "-O", "-T",
                 "-x", "-Z", "-p", "-y", "-q", "-E", "-Y"]:
        assert f"[{flag} " in out.stdout, flag


def test_bad_values_are_refused_before_any_gpu_work(perf_bin):
    exe = str(perf_bin["reduce_scatter_perf"])
    for argv in (["-Y", "bogus"], ["--no-such-flag"], ["-b"]):
        out = subprocess.run([exe, *argv], capture_output=True, text=True, timeout=60)
        assert out.returncode == 1, argv


def test_one_binary_per_collective_and_a_stock_nccl_twin(perf_bin):
    for coll in ["all_reduce", "all_gather", "reduce_scatter", "broadcast", "reduce", "alltoall", "alltoallv", "sendrecv", "gather",
                 "scatter", "hypercube"]:
        assert f"{coll}_perf" in perf_bin
    twins = [n for n in perf_bin if n.endswith("_perf_nccl")]
    assert twins == [] or "all_reduce_perf_nccl" in twins   # present wherever a system nccl.h exists
