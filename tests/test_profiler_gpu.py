"""Activity tracing on a real device: in-process records and the launcher's injection path."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def test_in_process_kernel_and_memcpy_records():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from rocm_systems_b200.ops import train_ops
    from rocm_systems_b200.utils.profiler import Profiler

    x = torch.randn(512, 4096, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(4096, device="cuda", dtype=torch.bfloat16)
    host = torch.empty(1 << 20, dtype=torch.uint8).pin_memory()
    train_ops.rmsnorm(x, w)  # load the module before tracing starts
    torch.cuda.synchronize()
    with Profiler(kernels=True, memops=True, runtime_api=True) as p:
        for _ in range(3):
            train_ops.rmsnorm(x, w)
        dev = host.cuda(non_blocking=True)
        torch.cuda.synchronize()
        del dev
    ks = p.kernels()
    mine = [k for k in ks if "rmsnorm" in k["name"].lower()]
    assert len(mine) == 3, [k["name"] for k in ks]
    assert all(k["end_ns"] > k["start_ns"] and k["registers"] > 0 and k["block"][0] > 0 for k in mine)
    copies = [m for m in p.memops() if m["op"] == "memcpy" and m["bytes"] == 1 << 20]
    assert copies, p.memops()
    assert any("cudaLaunchKernel" in a["name"] or "LaunchKernel" in a["name"] for a in p.apis())
    s = p.kernel_summary()
    assert sum(v["calls"] for v in s.values()) == len(ks)
    p.clear()
    assert p.kernels() == []


def test_launcher_traces_a_child_process(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    child = ("import torch\nfrom rocm_systems_b200.utils import markers\n"
             "with markers.range('mm'):\n    a = torch.randn(1024, 1024, device='cuda'); b = a @ a; torch.cuda.synchronize()\n")
    e = dict(os.environ, PYTHONPATH=str(ROOT))
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--kernel-trace", "--memory-copy-trace", "--marker-trace", "--summary",
                        "-d", str(tmp_path), "--", sys.executable, "-c", child], env=e, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout + p.stderr
    s = json.loads((tmp_path / "trace_summary.json").read_text())
    assert s["kernels"] and s["kernels"][0]["calls"] >= 1
    assert any(r["name"] == "mm" for r in s["regions"])
