"""The public headers have to be usable the way a user would use them: nccl.h from plain C, the
device-initiated API from a user's own CUDA kernel. The examples are compiled (not run) here."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
INC = ROOT / "rocm_systems_b200" / "csrc" / "include"


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_c_example_compiles_as_c(tmp_path):
    p = subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-c", str(ROOT / "examples" / "allreduce.c"), f"-I{INC}", "-I/usr/local/cuda/include",
                        "-o", str(tmp_path / "a.o")], capture_output=True, text=True)
    assert p.returncode == 0, p.stderr


@pytest.mark.skipif(not Path("/usr/local/cuda/bin/nvcc").exists(), reason="needs nvcc")
def test_device_api_example_compiles_for_sm100a(tmp_path):
    p = subprocess.run(["/usr/local/cuda/bin/nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-c", str(ROOT / "examples" / "shmem_ring.cu"),
                        f"-I{INC}", "-o", str(tmp_path / "s.o")], capture_output=True, text=True)
    assert p.returncode == 0, p.stderr


def test_python_example_parses():
    import ast

    for name in ("train_llama_fsdp.py", "tensor_parallel_mlp.py", "moe_expert_parallel.py"):
        ast.parse((ROOT / "examples" / name).read_text())


@pytest.mark.parametrize("example,port,marker,extra", [
    ("pipeline_1f1b.py", 29921, "pipeline_1f1b OK", []),
    ("long_context_attention.py", 29922, "long_context_attention OK", []),
    ("torch_fsdp_llama.py", 29923, "torch_fsdp_llama OK", ["--device", "cpu", "--backend", "gloo", "--steps", "2", "--warmup", "1"]),
])
def test_parallel_examples_run_on_cpu_ranks(example, port, marker, extra):
    import sys

    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), str(ROOT / "examples" / example), *extra], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert marker in p.stdout


def test_python_tracing_example_under_the_launcher(tmp_path):
    """examples/trace_python_step.py under the launcher and the Python tracer: marker ranges of the steps and their phases and
    the Python calls of the example end up in one database, the phases inside their step."""
    import sqlite3
    import sys

    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--marker-trace", "-d", str(tmp_path), "-o", "run", "--",
                        sys.executable, "-m", "rocm_systems_b200.tools.pytrace", "-MR", "trace_python_step", "--", str(ROOT / "examples" / "trace_python_step.py"),
                        "--steps", "3"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert p.returncode == 0 and "trace_python_step OK" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
    db = sqlite3.connect(str(tmp_path / "run.db"))
    got = {(c, n): k for c, n, k in db.execute("select category, name, count(*) from regions group by 1, 2")}
    assert got[("MARKER_API", "forward + backward")] == 3 and got[("MARKER_API", "step 1")] == 1 and got[("PYTHON_FUNCTION", "forward_backward")] == 3
    step = db.execute("select start_ns, end_ns from regions where name = 'step 2'").fetchone()
    inner = db.execute("select start_ns, end_ns from regions where category = 'MARKER_API' and name = 'optimizer' order by start_ns desc limit 1").fetchone()
    assert step[0] <= inner[0] <= inner[1] <= step[1]
