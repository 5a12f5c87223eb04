"""In-tree build of the native parts: ``lib/libb200coll.so`` (collective library, sm_100a
kernels), the ``*_perf`` benchmark binaries, and the torch extension.

Everything is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and lands
inside the package directory, so a checkout that was built on a machine without a GPU can be
carried to a GPU machine as is. ``python -m rocm_systems_b200.utils.build`` builds all targets;
``build_all()`` is what ``__graft_entry__.build`` calls.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shlex
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "lib"
BIN = PKG / "bin"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function,-Wno-sign-compare",
          f"-I{CSRC / 'include'}", f"-I{CSRC}", "--expt-relaxed-constexpr"]

REDUCE_TYPES = [
    ("int8_t", "i8", False), ("uint8_t", "u8", False), ("int32_t", "i32", False), ("uint32_t", "u32", False),
    ("int64_t", "i64", False), ("uint64_t", "u64", False), ("__half", "f16", True), ("float", "f32", True),
    ("double", "f64", False), ("__nv_bfloat16", "bf16", True), ("__nv_fp8_e4m3", "e4m3", False),
    ("__nv_fp8_e5m2", "e5m2", False),
]


def _run(cmd: list[str], quiet: bool = False) -> None:
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        sys.stderr.write("FAILED: " + " ".join(shlex.quote(c) for c in cmd) + "\n" + p.stdout + p.stderr + "\n")
        raise RuntimeError(f"build step failed: {cmd[-1]}")
    if not quiet and p.stderr.strip():
        # ptxas -v and warnings
        sys.stderr.write(p.stderr)


def _headers_stamp() -> str:
    h = hashlib.sha1()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".cuh", ".inc"):
            h.update(str(p).encode())
            h.update(str(p.stat().st_mtime_ns).encode())
    return h.hexdigest()[:16]


def _needs(obj: Path, src: Path, stamp: str, extra: str = "") -> bool:
    tag = obj.with_suffix(obj.suffix + ".stamp")
    want = f"{stamp}:{src.stat().st_mtime_ns}:{extra}"
    if obj.exists() and tag.exists() and tag.read_text() == want:
        return False
    return True


def _mark(obj: Path, src: Path, stamp: str, extra: str = "") -> None:
    obj.with_suffix(obj.suffix + ".stamp").write_text(f"{stamp}:{src.stat().st_mtime_ns}:{extra}")


def _compile(src: Path, obj: Path, defs: list[str], stamp: str, verbose_ptxas: bool) -> Path:
    extra = " ".join(defs)
    if _needs(obj, src, stamp, extra):
        cmd = [NVCC, *ARCH, *COMMON, *defs]
        if verbose_ptxas and src.suffix == ".cu":
            cmd += ["-Xptxas", "-v"]
        cmd += ["-c", str(src), "-o", str(obj)]
        _run(cmd, quiet=not verbose_ptxas)
        _mark(obj, src, stamp, extra)
    return obj


def lib_jobs() -> list[tuple[Path, Path, list[str]]]:
    jobs: list[tuple[Path, Path, list[str]]] = []
    for rel in ["core/common.cc", "core/bootstrap.cc", "core/cudrv.cc", "core/mem.cc", "core/comm.cc", "core/api.cc",
                "core/topo.cc", "coll/enqueue.cc", "coll/launch.cu", "coll/emu.cu", "trace/tracer.cc", "trace/markers.cc", "shmem/shmem_host.cc",
                "coll/verifiable.cu", "fused/train_ops.cu", "fused/fsdp_kernels.cu", "fused/gemm_sm100.cu", "fused/gemm_pair_sm100.cu", "fused/tp_fused.cu", "fused/tp_fused_fp8.cu",
                "fused/ep_kernels.cu", "fused/gemm_fp8_sm100.cu", "fused/no_alloc.cu", "shmem/shmem_kernels.cu", "core/health.cc"]:
        src = CSRC / rel
        if not src.exists():
            continue
        jobs.append((src, OBJ / (rel.replace("/", "_") + ".o"), ["-x", "cu"] if src.suffix == ".cc" else []))
    for ctype, tn, nvls in REDUCE_TYPES:
        defs = [f"-DB200_T={ctype}", f"-DB200_TN={tn}"] + (["-DB200_NVLS_OK=1"] if nvls else [])
        jobs.append((CSRC / "coll/reduce_inst.cu", OBJ / f"coll_reduce_inst_{tn}.o", defs))
    return jobs


def build_lib(verbose_ptxas: bool = False, jobs_n: int | None = None) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    stamp = _headers_stamp()
    jobs = lib_jobs()
    with cf.ThreadPoolExecutor(max_workers=jobs_n or os.cpu_count() or 4) as ex:
        objs = list(ex.map(lambda j: _compile(j[0], j[1], j[2], stamp, verbose_ptxas), jobs))
    out = LIB / "libb200coll.so"
    newest = max(o.stat().st_mtime_ns for o in objs)
    if not out.exists() or out.stat().st_mtime_ns < newest:
        _run([NVCC, *ARCH, "-shared", "-o", str(out), *map(str, objs), "-cudart", "static", "-lpthread", "-ldl", "-lrt"])
    return out


def build_sample_tool() -> Path | None:
    """The example profiling tool for the dispatch table, as a shared object of its own."""
    src = CSRC / "trace" / "sample_tool.cc"
    if not src.exists():
        return None
    LIB.mkdir(exist_ok=True)
    out = LIB / "libb200coll_sample_tool.so"
    if not out.exists() or out.stat().st_mtime_ns < src.stat().st_mtime_ns:
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-I{CSRC / 'include'}", "-I/usr/local/cuda/include", str(src), "-o", str(out)])
    return out


def build_prof() -> Path | None:
    """The CUPTI activity tracing library (in-process API and CUDA injection entry point)."""
    src = CSRC / "prof" / "b200prof.cc"
    cuda = Path(NVCC).resolve().parents[1]
    if not src.exists() or not (cuda / "include" / "cupti.h").exists():
        return None
    LIB.mkdir(exist_ok=True)
    out = LIB / "libb200prof.so"
    hdr = CSRC / "include" / "b200coll" / "prof.h"
    if not out.exists() or out.stat().st_mtime_ns < max(src.stat().st_mtime_ns, hdr.stat().st_mtime_ns):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-I{CSRC / 'include'}", f"-I{cuda / 'include'}", str(src), "-o", str(out),
              f"-L{cuda / 'lib64'}", "-lcupti", f"-Wl,-rpath,{cuda / 'lib64'}", "-lpthread"])
    return out


def build_sampler() -> Path | None:
    """The host call-stack sampler (preload library, plain C++, no CUDA)."""
    src = CSRC / "prof" / "sampler.cc"
    if not src.exists():
        return None
    LIB.mkdir(exist_ok=True)
    out = LIB / "libb200sample.so"
    hdr = CSRC / "include" / "b200coll" / "sample.h"
    if not out.exists() or out.stat().st_mtime_ns < max(src.stat().st_mtime_ns, hdr.stat().st_mtime_ns):
        _run(["g++", "-O2", "-g", "-std=c++17", "-fPIC", "-shared", f"-I{CSRC / 'include'}", str(src), "-o", str(out), "-lpthread", "-ldl"])
    return out


def build_kokkosp() -> Path | None:
    """The Kokkos Tools library that turns Kokkos callbacks into marker ranges (plain C++; finds the markers at run time)."""
    src = CSRC / "trace" / "kokkosp.cc"
    if not src.exists():
        return None
    LIB.mkdir(exist_ok=True)
    out = LIB / "libb200kokkosp.so"
    if not out.exists() or out.stat().st_mtime_ns < src.stat().st_mtime_ns:
        _run(["g++", "-O2", "-g", "-std=c++17", "-fPIC", "-shared", str(src), "-o", str(out), "-ldl"])
    return out


def build_ompt() -> Path | None:
    """The OpenMP tool (OMPT) that turns OpenMP regions into marker ranges; needs the OMPT header the CUDA toolkit ships."""
    src = CSRC / "trace" / "ompt.cc"
    cuda_inc = Path(NVCC).resolve().parents[1] / "include"
    if not src.exists() or not (cuda_inc / "Openmp" / "omp-tools.h").exists():
        return None
    LIB.mkdir(exist_ok=True)
    out = LIB / "libb200ompt.so"
    if not out.exists() or out.stat().st_mtime_ns < src.stat().st_mtime_ns:
        _run(["g++", "-O2", "-g", "-std=c++17", "-fPIC", "-shared", f"-I{cuda_inc}", str(src), "-o", str(out), "-ldl"])
    return out


def build_instrument() -> Path | None:
    """Entry / exit hooks for code compiled with -finstrument-functions: function statistics, marker ranges, coverage."""
    src = CSRC / "prof" / "instrument.cc"
    if not src.exists():
        return None
    LIB.mkdir(exist_ok=True)
    out = LIB / "libb200instr.so"
    if not out.exists() or out.stat().st_mtime_ns < src.stat().st_mtime_ns:
        _run(["g++", "-O2", "-g", "-std=c++17", "-fPIC", "-shared", str(src), "-o", str(out), "-ldl"])
    return out


def build_causal() -> Path | None:
    """The causal profiler (preload library, plain C++, no CUDA)."""
    src = CSRC / "prof" / "causal.cc"
    if not src.exists():
        return None
    LIB.mkdir(exist_ok=True)
    out = LIB / "libb200causal.so"
    hdr = CSRC / "include" / "b200coll" / "causal.h"
    if not out.exists() or out.stat().st_mtime_ns < max(src.stat().st_mtime_ns, hdr.stat().st_mtime_ns):
        _run(["g++", "-O2", "-g", "-std=c++17", "-fPIC", "-shared", f"-I{CSRC / 'include'}", str(src), "-o", str(out), "-lpthread", "-ldl"])
    return out


def build_perf(verbose_ptxas: bool = False) -> list[Path]:
    """rccl-tests-style benchmark binaries (one per collective) linked against the library."""
    BIN.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    perf = CSRC / "perf"
    if not (perf / "perf_main.cu").exists():
        return []
    stamp = _headers_stamp()
    lib = build_lib()
    outs = []
    colls = ["all_reduce", "all_gather", "reduce_scatter", "broadcast", "reduce", "alltoall", "alltoallv", "sendrecv",
             "gather", "scatter", "hypercube"]

    def one(coll: str) -> Path:
        out = BIN / f"{coll}_perf"
        src = perf / "perf_main.cu"
        obj = OBJ / f"perf_{coll}.o"
        _compile(src, obj, [f"-DPERF_COLL_{coll.upper()}=1", f'-DPERF_NAME="{coll}"'], stamp, verbose_ptxas)
        if not out.exists() or out.stat().st_mtime_ns < max(obj.stat().st_mtime_ns, lib.stat().st_mtime_ns):
            _run([NVCC, *ARCH, "-o", str(out), str(obj), f"-L{LIB}", "-lb200coll", "-Xlinker", "-rpath,$ORIGIN/../lib",
                  "-lpthread", "-ldl"])
        return out

    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        outs = list(ex.map(one, colls))
    # The same harness against stock NCCL, the baseline every number is compared with.
    nccl_inc = None
    for cand in ["/usr/include/nccl.h"]:
        if os.path.exists(cand):
            nccl_inc = cand
    if nccl_inc and (perf / "perf_main.cu").exists():
        def one_nccl(coll: str) -> Path:
            out = BIN / f"{coll}_perf_nccl"
            src = perf / "perf_main.cu"
            obj = OBJ / f"perf_nccl_{coll}.o"
            _compile(src, obj, [f"-DPERF_COLL_{coll.upper()}=1", f'-DPERF_NAME="{coll}"', "-DPERF_STOCK_NCCL=1"], stamp, False)
            if not out.exists() or out.stat().st_mtime_ns < obj.stat().st_mtime_ns:
                _run([NVCC, *ARCH, "-o", str(out), str(obj), "-lnccl", "-lpthread", "-ldl"])
            return out
        with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
            outs += list(ex.map(one_nccl, ["all_reduce", "all_gather", "reduce_scatter", "broadcast", "alltoall", "sendrecv", "reduce"]))
    return outs


def build_torch_ext() -> Path | None:
    """The c10d backend + op bindings as a Python extension module next to the package."""
    src = CSRC / "torch" / "pg_b200.cpp"
    if not src.exists():
        return None
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    lib = build_lib()
    OBJ.mkdir(exist_ok=True)
    ext_suffix = sysconfig.get_config_var("EXT_SUFFIX")
    out = PKG / f"_C{ext_suffix}"
    stamp = _headers_stamp()
    srcs = [src] + [p for p in sorted((CSRC / "torch").glob("*.cpp")) if p != src]
    objs = []
    incs = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC / 'include'}", f"-I{CSRC}",
                                                    "-I/usr/local/cuda/include"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)

    def one(s: Path) -> Path:
        obj = OBJ / ("torch_" + s.stem + ".o")
        if _needs(obj, s, stamp, "torch" + torch.__version__):
            _run(["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                  f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DUSE_C10D_GLOO", "-DUSE_C10D_NCCL", "-Wno-deprecated-declarations", *incs, "-c", str(s), "-o", str(obj)])
            _mark(obj, s, stamp, "torch" + torch.__version__)
        return obj

    with cf.ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(one, srcs))
    tlib = Path(torch.__file__).parent / "lib"
    newest = max([o.stat().st_mtime_ns for o in objs] + [lib.stat().st_mtime_ns])
    if not out.exists() or out.stat().st_mtime_ns < newest:
        _run(["g++", "-shared", "-o", str(out), *map(str, objs), f"-L{LIB}", "-lb200coll", f"-L{tlib}", "-ltorch", "-ltorch_cpu",
              "-lc10", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{tlib}"])
    return out


def build_all(verbose_ptxas: bool = False) -> dict:
    res = {"lib": str(build_lib(verbose_ptxas))}
    res["perf"] = [str(p) for p in build_perf()]
    tool = build_sample_tool()
    res["sample_tool"] = str(tool) if tool else None
    prof = build_prof()
    res["prof"] = str(prof) if prof else None
    samp = build_sampler()
    res["sampler"] = str(samp) if samp else None
    kk = build_kokkosp()
    res["kokkosp"] = str(kk) if kk else None
    om = build_ompt()
    res["ompt"] = str(om) if om else None
    ins = build_instrument()
    res["instrument"] = str(ins) if ins else None
    causal = build_causal()
    res["causal"] = str(causal) if causal else None
    ext = build_torch_ext()
    res["torch_ext"] = str(ext) if ext else None
    return res


if __name__ == "__main__":
    import json

    print(json.dumps(build_all("-v" in sys.argv), indent=1))
