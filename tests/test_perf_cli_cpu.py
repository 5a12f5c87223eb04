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


def test_communicator_split_by_environment(perf_bin):
    """NCCL_TESTS_SPLIT_MASK / NCCL_TESTS_SPLIT group the ranks as the reference harness does (common.cpp:1640-1672)."""
    import os

    exe = str(perf_bin["all_gather_perf"])

    def groups(n, **env):
        e = {k: v for k, v in os.environ.items() if not k.startswith("NCCL_TESTS_")}
        e.update(env)
        out = subprocess.run([exe, "--print-split", str(n)], capture_output=True, text=True, env=e, timeout=60).stdout
        rows = [line.split() for line in out.strip().splitlines()]
        return [(int(r[0]), int(r[2]), int(r[4]), int(r[6])) for r in rows]      # proc, colour, rank in group, group size

    assert groups(3) == [(0, 0, 0, 3), (1, 0, 1, 3), (2, 0, 2, 3)]
    assert groups(4, NCCL_TESTS_SPLIT_MASK="0x1") == [(0, 0, 0, 2), (1, 1, 0, 2), (2, 0, 1, 2), (3, 1, 1, 2)]
    assert [g[1] for g in groups(8, NCCL_TESTS_SPLIT="DIV4")] == [0, 0, 0, 0, 1, 1, 1, 1]
    assert [g[1] for g in groups(6, NCCL_TESTS_SPLIT="MOD 3")] == [0, 1, 2, 0, 1, 2]
    assert [g[1] for g in groups(4, NCCL_TESTS_SPLIT="%2")] == [0, 1, 0, 1]
    assert [g[1] for g in groups(4, NCCL_TESTS_SPLIT="AND2")] == [0, 0, 2, 2]
    assert [g[1] for g in groups(4, NCCL_TESTS_SPLIT="|1")] == [1, 1, 3, 3]
