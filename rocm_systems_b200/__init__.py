"""rocm_systems_b200 — a Blackwell-native collective-communication and device-initiated
communication stack (NCCL-compatible C API, OpenSHMEM-style device API, torch.distributed
backend, fused compute+communication kernels, tracer, telemetry) with PyTorch as the framework
layer. Native code lives in ``csrc/`` and is built in-tree by ``utils/build.py``.
"""

__version__ = "0.1.0"


def __getattr__(name):
    # Lazy so that `import rocm_systems_b200` works before torch is imported or the library built.
    if name in ("Communicator", "get_unique_id", "init_from_env"):
        from . import comm

        return getattr(comm, name)
    if name in ("LlamaConfig", "LlamaTrainer"):
        from .models import llama

        return getattr(llama, name)
    if name in ("init_process_group", "register_backend"):
        from .parallel import dist

        return getattr(dist, name)
    raise AttributeError(name)
