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


@pytest.mark.skipif(not Path("/usr/local/cuda/bin/nvcc").exists(), reason="needs nvcc")
def test_planner_and_tuning_loader_under_sanitizers(tmp_path):
    """The whole library compiled with ASan + UBSan (host side), then the planner on 20000 random requests, bad
    arguments, the settings listing into short buffers, and tuning files with out-of-range and wrongly typed values."""
    import concurrent.futures as cf
    import sys

    sys.path.insert(0, str(ROOT))
    from rocm_systems_b200.utils import build

    san = "-fPIC,-fsanitize=address,-fsanitize=undefined,-fsanitize=float-cast-overflow,-fno-omit-frame-pointer"

    def compile_one(job):
        src, obj, defs = job
        out = tmp_path / obj.name
        cmd = [build.NVCC, *build.ARCH, "-O1", "-g", "-std=c++17", "-Xcompiler", san, f"-I{CSRC / 'include'}", f"-I{CSRC}", "--expt-relaxed-constexpr", *defs,
               "-c", str(src), "-o", str(out)]
        p = subprocess.run(cmd, capture_output=True, text=True)
        assert p.returncode == 0, p.stderr[-3000:]
        return str(out)

    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(compile_one, build.lib_jobs()))
    exe = tmp_path / "planner_fuzz"
    p = subprocess.run([build.NVCC, *build.ARCH, "-Xcompiler", "-fsanitize=address,-fsanitize=undefined", f"-I{CSRC / 'include'}",
                        str(ROOT / "tests" / "native" / "planner_fuzz.cc"), *objs, "-o", str(exe), "-cudart", "static", "-lpthread", "-ldl", "-lrt",
                        "-Xlinker", "-lasan", "-Xlinker", "-lubsan"], capture_output=True, text=True)
    if p.returncode != 0 and "cannot find" in p.stderr:
        pytest.skip("no sanitizer runtime for this toolchain")
    assert p.returncode == 0, p.stderr[-3000:]
    files = {
        "good.json": '{"entries": [{"coll": "allreduce", "max_bytes": 1048576, "algo": "p2p", "ctas": 8}, {"coll": "allgather", "max_bytes": 1e12, "algo": "nvls", "ctas": 999999}]}',
        "range.json": '{"entries": [{"max_bytes": 1e300, "ctas": 1e30, "nranks": -1e40}, {"coll": "reducescatter", "algo": "ll", "max_bytes": -5}]}',
        "types.json": '{"entries": [{"coll": 5, "max_bytes": "x", "algo": null, "ctas": -3}, 7, "s", {"coll": "all_reduce"}], "extra": [[[[]]]]}',
        "cut.json": '{"entries": [{"coll": "allreduce", "max_bytes": 1e308',
    }
    env = {k: v for k, v in os.environ.items() if not k.startswith(("B200COLL_", "NCCL_"))}
    env.update(ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="halt_on_error=1")
    for name, text in [("", "")] + list(files.items()):
        e = dict(env)
        if name:
            (tmp_path / name).write_text(text)
            e["B200COLL_TUNING_FILE"] = str(tmp_path / name)
        r = subprocess.run([str(exe)], env=e, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and "planner under sanitizers: 0 bad" in r.stdout, (name, (r.stdout + r.stderr)[-3000:])
        assert "AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr, (name, r.stderr[-3000:])


def test_instrumentation_hooks_and_kokkos_connector_under_asan(tmp_path):
    """The entry / exit hooks (lock-free function table, per-thread stacks, symbol-table reader) with their instrumented
    target, and the Kokkos connector with its driver, all built with ASan + UBSan in one process each: no report, same
    results."""
    san = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-g", "-O1", "-std=c++17"]
    exe = tmp_path / "instr_asan"
    p = subprocess.run(["g++", *san, "-finstrument-functions", "-finstrument-functions-exclude-file-list=/usr/include,/usr/lib",
                        str(ROOT / "tests" / "native" / "instrument_target.cc"), str(CSRC / "prof" / "instrument.cc"), "-o", str(exe), "-lpthread", "-ldl"],
                       capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-3000:]
    env = dict(os.environ, B200INSTR_PREFIX=str(tmp_path / "i"), B200INSTR_MIN_US="-1", ASAN_OPTIONS="detect_leaks=0:abort_on_error=0")
    r = subprocess.run([str(exe)], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "instrument target done 3" in r.stdout and "ERROR" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-3000:]
    rows = next(tmp_path.glob("i.*.functions.csv")).read_text()
    assert '"inner(int)",7,' in rows and '"outer()",3,' in rows
    exe = tmp_path / "kk_asan"
    p = subprocess.run(["g++", *san, "-rdynamic", str(ROOT / "tests" / "native" / "kokkosp_driver.cc"), "-o", str(exe), "-ldl", "-lpthread"], capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-3000:]
    lib = tmp_path / "libkk_asan.so"
    p = subprocess.run(["g++", *san, "-fPIC", "-shared", str(CSRC / "trace" / "kokkosp.cc"), "-o", str(lib), "-ldl"], capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-3000:]
    r = subprocess.run([str(exe), str(lib)], env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0"), capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.startswith("ids ") and "ERROR" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-3000:]


def test_causal_profiler_under_asan(tmp_path):
    """The causal profiler (signal handler, thread slots, pthread wrappers, symbol-table reader, experiment loop) built with
    ASan + UBSan and preloaded into its thread-pool target, also built that way: experiments are recorded and no report."""
    san = ["-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-g", "-O1", "-std=c++17", f"-I{CSRC / 'include'}"]
    lib, exe, out = tmp_path / "libcausal_asan.so", tmp_path / "target_asan", tmp_path / "c.coz"
    p = subprocess.run(["g++", *san, "-fPIC", "-shared", str(CSRC / "prof" / "causal.cc"), "-o", str(lib), "-lpthread", "-ldl"], capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-3000:]
    p = subprocess.run(["g++", *san, str(ROOT / "tests" / "native" / "causal_target.cc"), "-o", str(exe), "-lpthread", "-ldl"], capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-3000:]
    asan = subprocess.run(["g++", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    env = dict(os.environ, LD_PRELOAD=f"{asan}:{lib}", ASAN_OPTIONS="verify_asan_link_order=0:detect_leaks=0:abort_on_error=0", B200CAUSAL_FILE=str(out),
               B200CAUSAL_FIXED_SPEEDUP="0,30", B200CAUSAL_EXPERIMENT_SECONDS="0.25")
    r = subprocess.run([str(exe), "120", "80", "1500000", "pool"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "done 120" in r.stdout and "ERROR" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-3000:]
    assert out.read_text().count("experiment\t") >= 2
