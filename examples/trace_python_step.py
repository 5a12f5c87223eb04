"""A toy training loop on the CPU that shows the host-side tracing pieces together: marker ranges around the phases of a
step, a progress point per step for the causal profiler, and (when run under the Python tracer) a range per Python call.

    python -m rocm_systems_b200.tools.prof --python-trace --python-restrict trace_python_step --stats --summary-per-domain -d out -o run -- \\
        python examples/trace_python_step.py --steps 5
    python -m rocm_systems_b200.tools.tracedb query out/run.db "select category, name, count(*) from regions group by 1, 2"

Nothing here needs a GPU; on one, the same markers line up with kernels and collectives in the same database.
"""
import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402

from rocm_systems_b200.utils import causal, markers  # noqa: E402


def make_batch(n: int, d: int, g: torch.Generator):
    x = torch.randn(n, d, generator=g)
    return x, (x.sum(-1, keepdim=True) > 0).float()


def forward_backward(model, x, y):
    loss = torch.nn.functional.binary_cross_entropy_with_logits(model(x), y)
    loss.backward()
    return float(loss)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--width", type=int, default=64)
    a = ap.parse_args()
    g = torch.Generator().manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(a.width, 128), torch.nn.ReLU(), torch.nn.Linear(128, 1))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    first = last = None
    for step in range(a.steps):
        with markers.range(f"step {step}"):
            with markers.range("data"):
                x, y = make_batch(a.batch, a.width, g)
            with markers.range("forward + backward"):
                last = forward_backward(model, x, y)
            with markers.range("optimizer"):
                opt.step()
                opt.zero_grad()
        first = last if first is None else first
        causal.progress("step")
    print(f"trace_python_step OK: loss {first:.3f} -> {last:.3f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
