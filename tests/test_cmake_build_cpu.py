"""The CMake build for C / C++ users (rocm_systems_b200/csrc/CMakeLists.txt): configure, build for sm_100a without a
GPU, install, and build examples/allreduce.c in a separate project through find_package(b200coll)."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _run(cmd, timeout=1800):
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, " ".join(map(str, cmd)) + "\n" + (p.stdout + p.stderr)[-4000:]
    return p.stdout


@pytest.mark.skipif(shutil.which("cmake") is None or shutil.which("ninja") is None or not Path("/usr/local/cuda/bin/nvcc").exists(),
                    reason="needs cmake, ninja and nvcc")
def test_configure_build_install_and_consume(tmp_path):
    build, prefix = tmp_path / "build", tmp_path / "prefix"
    _run(["cmake", "-S", str(ROOT / "rocm_systems_b200" / "csrc"), "-B", str(build), "-G", "Ninja", "-DCMAKE_CUDA_COMPILER=/usr/local/cuda/bin/nvcc"])
    _run(["cmake", "--build", str(build), "--target", "b200coll", "all_reduce_perf", "b200coll_sample_tool"])
    assert (build / "libb200coll.so").exists() and (build / "all_reduce_perf").exists()
    out = subprocess.run([str(build / "all_reduce_perf"), "-h"], capture_output=True, text=True)
    assert out.returncode == 0 and "USAGE: all_reduce_perf" in out.stdout
    _run(["cmake", "-DB200COLL_BUILD_PERF=OFF", str(build)])       # the install step then has no unbuilt targets
    _run(["cmake", "--build", str(build)])
    _run(["cmake", "--install", str(build), "--prefix", str(prefix)])
    assert (prefix / "include" / "b200coll" / "nccl.h").exists() and (prefix / "lib" / "cmake" / "b200coll" / "b200collConfig.cmake").exists()
    consumer = tmp_path / "consumer"
    consumer.mkdir()
    (consumer / "CMakeLists.txt").write_text(
        "cmake_minimum_required(VERSION 3.24)\nproject(consumer LANGUAGES C CXX)\nfind_package(b200coll REQUIRED)\n"
        f"add_executable(allreduce {ROOT / 'examples' / 'allreduce.c'})\ntarget_link_libraries(allreduce PRIVATE b200coll::b200coll CUDA::cudart)\n")
    _run(["cmake", "-S", str(consumer), "-B", str(consumer / "b"), "-G", "Ninja", f"-DCMAKE_PREFIX_PATH={prefix}"])
    _run(["cmake", "--build", str(consumer / "b")])
    assert (consumer / "b" / "allreduce").exists()
