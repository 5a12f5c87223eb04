"""Host code under sanitizers: the rendezvous (root thread, per-rank sockets, descriptor passing) is
built with AddressSanitizer + UBSan and with ThreadSanitizer and stressed with several ranks as
threads, random start skew and two communicators back to back. The reference builds its host code
with the same compiler options in CI; a GPU race detector exists on neither side."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "rocm_systems_b200" / "csrc"


def _build(tmp_path, flags, name):
    out = tmp_path / name
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, f"-I{CSRC}", f"-I{CSRC / 'include'}", "-I/usr/local/cuda/include",
           str(ROOT / "tests" / "native" / "bootstrap_stress.cc"), str(CSRC / "core" / "bootstrap.cc"), str(CSRC / "core" / "common.cc"),
           "-o", str(out), "-lpthread"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0 and ("cannot find" in p.stderr or "unrecognized" in p.stderr):
        pytest.skip("this toolchain has no runtime for " + " ".join(flags))
    assert p.returncode == 0, p.stderr[-3000:]
    return out


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
@pytest.mark.parametrize("name,flags,env", [
    ("asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0"}),
    ("tsan", ["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=1"}),
])
def test_bootstrap_under_sanitizer(tmp_path, name, flags, env):
    exe = _build(tmp_path, flags, "stress_" + name)
    e = dict(os.environ, B200COLL_BOOTSTRAP_TIMEOUT_MS="60000")
    e.update(env)
    p = subprocess.run([str(exe), "4", "30"], env=e, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, (p.stdout + p.stderr)[-4000:]
    assert "bootstrap stress OK" in p.stdout
    assert "ERROR: AddressSanitizer" not in p.stderr and "WARNING: ThreadSanitizer" not in p.stderr and "runtime error" not in p.stderr


def _build_units(tmp_path, flags, name):
    out = tmp_path / name
    cuda_lib = Path("/usr/local/cuda/lib64")
    if not (cuda_lib / "libcudart.so").exists():
        pytest.skip("needs the CUDA runtime library to link the marker recorder")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, f"-I{CSRC}", f"-I{CSRC / 'include'}", "-I/usr/local/cuda/include",
           str(ROOT / "tests" / "native" / "host_units.cc"), str(CSRC / "trace" / "markers.cc"), str(CSRC / "core" / "common.cc"),
           "-o", str(out), "-lpthread", f"-L{cuda_lib}", "-lcudart", f"-Wl,-rpath,{cuda_lib}"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0 and ("cannot find" in p.stderr or "unrecognized" in p.stderr):
        pytest.skip("this toolchain has no runtime for " + " ".join(flags))
    assert p.returncode == 0, p.stderr[-3000:]
    return out


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
@pytest.mark.parametrize("name,flags,env,what", [
    ("asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0"}, "all"),
    ("tsan", ["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=1"}, "markers"),
])
def test_json_reader_and_marker_recorder_under_sanitizer(tmp_path, name, flags, env, what):
    """The tuning-table reader on valid, truncated, mutated and absurdly nested texts; the range recorder from 8 threads
    with ranges that end on another thread."""
    exe = _build_units(tmp_path, flags, "units_" + name)
    p = subprocess.run([str(exe), what], env=dict(os.environ, **env), capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, (p.stdout + p.stderr)[-4000:]
    assert "markers OK" in p.stdout and (what != "all" or "json OK" in p.stdout)
    assert "ERROR: AddressSanitizer" not in p.stderr and "WARNING: ThreadSanitizer" not in p.stderr and "runtime error" not in p.stderr
