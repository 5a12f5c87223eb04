"""Several ranks of one communicator on ONE GPU, played by one cooperative kernel (csrc/coll/emu.cu): the collective
kernels' multi-rank paths — the flag-in-data family, pipelined staged reduce with bulk asynchronous loads, staged copy, the
scatter-and-forward broadcast and the staged all-to-all (several steps each: the staging is set to 1 MiB),
grouped send/recv through FIFO slots and credits, the fused FSDP reduce-scatter+cast, and the device-initiated layer's
put+signal ring and remote atomics — run where only one GPU is there. The check itself is native (b200collEmuSelftest: small-integer data, every collective in
float / bfloat16 / int32, verified on the host, guard bytes behind every output).

It runs in a child process with every device-side wait limited to 5 s."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu

CODE = """
import ctypes, sys
import torch
from rocm_systems_b200 import _lib
torch.cuda.set_device(0)
torch.zeros(1, device='cuda')
lib = _lib.load()
lib.b200collEmuSelftest.argtypes = [ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_int)]
bad = 0
for nranks, count in [(2, 1000), (4, 1000), (4, 70001), (3, 300007), (4, (1 << 20) + 8), (5, 700001), (8, 400003), (8, 100003)]:
    wrong, status = ctypes.c_longlong(-1), ctypes.c_int(-1)
    rc = lib.b200collEmuSelftest(nranks, count, ctypes.byref(wrong), ctypes.byref(status))
    print(f"ranks {nranks} count {count}: rc {rc} wrong {wrong.value} status {status.value}", flush=True)
    bad += (rc != 0) + (wrong.value != 0) + (status.value != 0)
print("EMULATED RANKS OK" if bad == 0 else "EMULATED RANKS FAILED", flush=True)
sys.exit(1 if bad else 0)
"""


def test_collectives_of_emulated_ranks_on_one_gpu():
    env = dict(os.environ, PYTHONPATH=str(ROOT), B200COLL_EMULATE_RANKS="1", B200COLL_NVLS_ENABLE="0", B200COLL_WAIT_TIMEOUT_MS="5000",
               B200COLL_BUFFSIZE="1M", B200COLL_BOOTSTRAP_TIMEOUT_MS="30000")
    p = subprocess.run([sys.executable, "-c", CODE], env=env, capture_output=True, text=True, timeout=900)
    sys.stdout.write(p.stdout[-3000:])
    sys.stderr.write(p.stderr[-3000:])
    assert p.returncode == 0 and "EMULATED RANKS OK" in p.stdout
