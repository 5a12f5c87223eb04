"""Host-side behaviour of the C API that needs no GPU: result strings, argument checks that answer
with a result code instead of crashing, group bookkeeping, identifiers, and error text that names
file and line without a build path."""
import ctypes
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

SUCCESS, CUDA_ERR, SYSTEM_ERR, INTERNAL, INVALID_ARG, INVALID_USAGE, REMOTE, IN_PROGRESS = range(8)


@pytest.fixture(scope="module")
def lib():
    from rocm_systems_b200 import _lib

    L = _lib.load()
    L.ncclGetErrorString.restype = ctypes.c_char_p
    L.ncclGetLastError.restype = ctypes.c_char_p
    L.ncclGetLastError.argtypes = [ctypes.c_void_p]
    return L


def test_result_strings(lib):
    texts = [lib.ncclGetErrorString(i).decode() for i in range(9)]
    assert texts[SUCCESS] == "no error" and "invalid argument" in texts[INVALID_ARG] and "invalid usage" in texts[INVALID_USAGE]
    assert "peer" in texts[REMOTE] and "in progress" in texts[IN_PROGRESS] and "unknown" in texts[8]
    assert len(set(texts)) == 9


def test_version_and_unique_ids(lib):
    v = ctypes.c_int()
    assert lib.ncclGetVersion(ctypes.byref(v)) == SUCCESS and v.value == 22005
    assert lib.ncclGetVersion(None) == INVALID_ARG
    U = lib.ncclGetUniqueId.argtypes[0]._type_
    a, b = U(), U()
    assert lib.ncclGetUniqueId(ctypes.byref(a)) == SUCCESS and lib.ncclGetUniqueId(ctypes.byref(b)) == SUCCESS
    ra, rb = ctypes.string_at(ctypes.addressof(a), 128), ctypes.string_at(ctypes.addressof(b), 128)
    assert ra != rb and any(ra) and len(ra) == 128      # every id names its own rendezvous
    assert lib.ncclGetUniqueId(None) == INVALID_ARG


def test_bad_handles_and_arguments_answer_with_codes(lib):
    vp = ctypes.c_void_p
    lib.ncclAllReduce.argtypes = [vp, vp, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, vp, vp]
    lib.ncclSend.argtypes = [vp, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, vp, vp]
    lib.ncclCommCount.argtypes = [vp, ctypes.POINTER(ctypes.c_int)]
    lib.ncclCommDestroy.argtypes = [vp]
    n = ctypes.c_int()
    junk = (ctypes.c_char * 4096)()                      # readable memory that is not a communicator
    assert lib.ncclAllReduce(None, None, 4, 7, 0, None, None) == INVALID_ARG
    assert lib.ncclSend(None, 4, 7, 0, None, None) == INVALID_ARG
    assert lib.ncclCommCount(None, ctypes.byref(n)) == INVALID_ARG
    assert lib.ncclCommCount(ctypes.addressof(junk), ctypes.byref(n)) == INVALID_ARG
    assert b"invalid communicator handle" in lib.ncclGetLastError(None)
    assert lib.ncclCommDestroy(None) == SUCCESS          # like free(NULL)


def test_group_bookkeeping(lib):
    assert lib.ncclGroupEnd() == INVALID_USAGE           # nothing open
    assert lib.ncclGroupStart() == SUCCESS and lib.ncclGroupStart() == SUCCESS      # groups nest
    assert lib.ncclGroupEnd() == SUCCESS and lib.ncclGroupEnd() == SUCCESS
    assert lib.ncclGroupEnd() == INVALID_USAGE


def test_init_argument_checks_and_error_text(lib):
    U = lib.ncclGetUniqueId.argtypes[0]._type_
    u = U()
    lib.ncclGetUniqueId(ctypes.byref(u))
    comm = ctypes.c_void_p()
    assert lib.ncclCommInitRank(ctypes.byref(comm), 0, u, 0) == INVALID_ARG
    assert lib.ncclCommInitRank(ctypes.byref(comm), 9, u, 0) == INVALID_ARG       # one NVSwitch domain: at most 8
    assert lib.ncclCommInitRank(ctypes.byref(comm), 2, u, 5) == INVALID_ARG
    assert lib.ncclCommInitRank(None, 1, u, 0) == INVALID_ARG
    import torch

    if not torch.cuda.is_available():
        rc = lib.ncclCommInitRank(ctypes.byref(comm), 1, u, 0)
        assert rc == CUDA_ERR and not comm.value
        msg = lib.ncclGetLastError(None).decode()
        assert msg.startswith("comm.cc:") and "/" not in msg.split(" ")[0] and "cudaGetDevice" in msg


def test_debug_file_receives_the_log_lines(tmp_path):
    import os
    import subprocess

    code = """
import ctypes
from rocm_systems_b200 import _lib
lib = _lib.load()
lib.ncclCommCount.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
n = ctypes.c_int()
assert lib.ncclCommCount(None, ctypes.byref(n)) == 4
"""
    e = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_DEBUG_FILE=str(tmp_path / "log.%p.txt"))
    p = subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr
    files = list(tmp_path.glob("log.*.txt"))
    assert len(files) == 1 and files[0].name != "log.%p.txt"
    assert "invalid communicator handle" in files[0].read_text() and "invalid communicator handle" not in p.stderr


def test_copy_engine_transfers_are_cut_into_whole_64k_parts_that_cover_the_message():
    from rocm_systems_b200 import shmem

    for nbytes, gang in [(1, 0), (65536, 4), (65537, 4), (8 << 20, 0), (64 << 20, 0), (3 << 20, 8), ((1 << 30) + 12345, 0), (100 << 20, 3), (1 << 20, 64)]:
        parts = shmem.dma_plan(nbytes, gang)
        assert 1 <= len(parts) <= 8
        assert parts[0][0] == 0 and sum(n for _, n in parts) == nbytes
        for (o0, n0), (o1, _) in zip(parts, parts[1:]):
            assert o0 + n0 == o1 and n0 % 65536 == 0 and n0 > 0
        sizes = [n for _, n in parts]
        assert max(sizes) - min(sizes) <= 2 * 65536
    assert len(shmem.dma_plan(1 << 20)) == 1 and len(shmem.dma_plan(8 << 20)) == 2 and len(shmem.dma_plan(64 << 20)) == 4
    assert len(shmem.dma_plan(128 << 10, 8)) == 2            # never more parts than 64 KiB units


def test_every_function_declared_in_a_public_header_is_exported():
    """A user who compiles against csrc/include/b200coll must be able to link: every declared entry point exists in
    libb200coll.so (or, for the activity tracer, libb200prof.so)."""
    import re
    import subprocess
    from pathlib import Path

    from rocm_systems_b200.utils import build

    root = Path(build.CSRC) / "include" / "b200coll"
    declared = set()
    prefixes = r"(?:p?nccl[A-Z]|b200coll[A-Z_]|b200shmem_|b200smi_|b200tx[A-Z]|b200prof[A-Z]|b200ops_|msccl[A-Z])"
    for h in root.glob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        text = re.sub(r"//.*", "", text)
        declared |= {m.group(1) for m in re.finditer(r"\b(" + prefixes + r"\w*)\s*\(", text)}
        declared |= {m.group(1) for m in re.finditer(r"B200COLL_DECL\(\s*[^,]+,\s*(\w+)\s*,", text)}
    declared = {d for d in declared if not d.endswith("_t") and not d.endswith("_fn") and not d.endswith("_cb") and d != "name"}   # "name": the macro's own parameter
    assert len(declared) > 100
    exported = set()
    libs = [build.build_lib()]
    prof = build.build_prof()
    if prof:
        libs.append(prof)
    for lib in libs:
        out = subprocess.check_output(["nm", "-D", "--defined-only", str(lib)], text=True)
        exported |= {line.split()[-1] for line in out.splitlines() if line.strip()}
    missing = sorted(d for d in declared if d not in exported and (prof or not d.startswith("b200prof")))
    assert missing == [], missing


def test_every_native_symbol_the_python_package_calls_exists():
    """ctypes resolves names at call time, so a misspelt entry point in a wrapper that no CPU test calls would only show
    up on a GPU. Every ``.b200...`` / ``.nccl...`` attribute used in the package must be an exported symbol."""
    import re
    import subprocess
    from pathlib import Path

    from rocm_systems_b200.utils import build

    pkg = Path(build.PKG)
    used = {}
    for py in list(pkg.rglob("*.py")) + [pkg.parent / "bench.py"]:
        for m in re.finditer(r"\.((?:b200coll|b200shmem_|b200smi_|b200tx|b200prof|b200ops_|nccl[A-Z])\w*)\b", py.read_text()):
            used.setdefault(m.group(1), py.name)
    assert len(used) > 80
    exported = set()
    libs = [build.build_lib()] + ([build.build_prof()] if build.build_prof() else [])
    for lib in libs:
        out = subprocess.check_output(["nm", "-D", "--defined-only", str(lib)], text=True)
        exported |= {line.split()[-1] for line in out.splitlines() if line.strip()}
    missing = sorted((n, f) for n, f in used.items() if n not in exported)
    assert missing == [], missing


def test_ctypes_signatures_have_the_arity_of_the_c_functions():
    """The number of ``argtypes`` every wrapper module declares equals the parameter count of the C definition."""
    import re
    from pathlib import Path

    from rocm_systems_b200 import _lib, shmem
    from rocm_systems_b200.ops import fp8, train_ops
    from rocm_systems_b200.parallel import ep, tp
    from rocm_systems_b200.utils import build

    lib = _lib.load()
    for setup in (shmem._l, train_ops._lib_ops, fp8._lib, tp._lib_tp, ep._lib_ep):
        setup()                                   # these only declare signatures; nothing touches a GPU
    arity, signatures = {}, {}
    pat = re.compile(r"\b((?:b200coll|b200shmem_|b200ops_)\w*)\s*\(([^(){};]*(?:\([^()]*\)[^(){};]*)*)\)\s*\{")
    for src in list(Path(build.CSRC).rglob("*.cu")) + list(Path(build.CSRC).rglob("*.cc")):
        text = re.sub(r"/\*.*?\*/", "", src.read_text(), flags=re.S)
        text = re.sub(r"//.*", "", text)
        for m in pat.finditer(text):
            params = m.group(2).strip()
            if params and params != "void" and not re.search(r"\b(int|void|size_t|float|char|double|uint\w+|unsigned|long|const|nccl\w+|cuda\w+|b200\w+_t)\b", params):
                continue                          # a call, not a definition
            plist = [] if params in ("", "void") else re.split(r",(?![^()]*\))", params)
            arity[m.group(1)] = len(plist)
            signatures[m.group(1)] = plist
    checked, bad = 0, []
    for name, n in arity.items():
        fn = getattr(lib, name, None)
        if fn is None or fn.argtypes is None:
            continue
        checked += 1
        if len(fn.argtypes) != n:
            bad.append((name, len(fn.argtypes), n))
    assert checked > 60, checked
    assert bad == [], bad

    # ... and every argument has the class (pointer, 32-bit, 64-bit, float, double) of the C parameter.
    import ctypes

    def c_class(param: str) -> str:
        param = re.sub(r"\s*=.*$", "", param.strip())
        if "*" in param or "[" in param or re.search(r"\b(cudaStream_t|ncclComm_t|b200shmem_ctx_t)\b", param):
            return "ptr"
        ctype = " ".join(param.replace("const", " ").split()[:-1])
        if ctype in ("int", "unsigned", "unsigned int", "uint32_t", "int32_t", "ncclDataType_t", "ncclRedOp_t"):
            return "i32"
        if ctype in ("long long", "unsigned long long", "uint64_t", "int64_t", "size_t", "long", "unsigned long"):
            return "i64"
        return {"float": "f32", "double": "f64"}.get(ctype, "?" + ctype)

    def py_class(a) -> str:
        if a in (ctypes.c_void_p, ctypes.c_char_p) or (isinstance(a, type) and issubclass(a, ctypes._Pointer)):
            return "ptr"
        if a in (ctypes.c_int, ctypes.c_uint, ctypes.c_int32, ctypes.c_uint32):
            return "i32"
        if a in (ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_size_t, ctypes.c_uint64, ctypes.c_int64, ctypes.c_long, ctypes.c_ulong):
            return "i64"
        return {ctypes.c_float: "f32", ctypes.c_double: "f64"}.get(a, "?" + str(a))

    mismatched = []
    for name, params in signatures.items():
        fn = getattr(lib, name, None)
        if fn is None or fn.argtypes is None or len(params) != len(fn.argtypes):
            continue
        for i, (cp, at) in enumerate(zip(params, fn.argtypes)):
            if c_class(cp) != py_class(at):
                mismatched.append((name, i, cp.strip(), str(at)))
    assert mismatched == [], mismatched
