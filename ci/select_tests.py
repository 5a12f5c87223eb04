#!/usr/bin/env python3
"""Choose what CI has to build and test from the list of changed paths.

The counterpart of the reference's mono-repo tooling (.github/scripts/therock_configure_ci.py and
its subtree detection): there a changed project selects the projects to configure; here a changed
layer of the package selects the test files that cover it and says whether the native code must be
rebuilt and whether a GPU box is needed.

    git diff --name-only origin/main... | python ci/select_tests.py            # JSON on stdout
    python ci/select_tests.py --paths rocm_systems_b200/csrc/coll/kernels.cuh
"""
from __future__ import annotations

import argparse
import fnmatch
import json
import sys
from typing import Iterable, List

# (pattern, cpu tests, gpu tests, needs native rebuild)
RULES = [
    ("rocm_systems_b200/csrc/CMakeLists.txt", ["tests/test_cmake_build_cpu.py"], [], False),
    ("rocm_systems_b200/csrc/core/json.h", ["tests/test_sanitizers_cpu.py", "tests/test_planner_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/core/bootstrap.*", ["tests/test_bootstrap.py", "tests/test_sanitizers_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/core/topo.cc", ["tests/test_smi_fake.py", "tests/test_tools_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/core/health.cc", ["tests/test_smi_fake.py", "tests/test_tools_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/core/*", ["tests/test_api_cpu.py", "tests/test_bootstrap.py", "tests/test_planner_cpu.py", "tests/test_tools_cpu.py"], ["tests/test_gpu_collectives.py"], True),
    ("rocm_systems_b200/csrc/coll/verifiable*", ["tests/test_verifiable_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/coll/*", ["tests/test_planner_cpu.py", "tests/test_protocol_interleavings_cpu.py", "tests/test_protocol_model_cpu.py", "tests/test_staged_emulation_cpu.py"], ["tests/test_gpu_collectives.py", "tests/test_gpu_fused_multi.py", "tests/test_zz_emulated_ranks_gpu.py"], True),
    ("rocm_systems_b200/csrc/include/b200coll/shmem_device.cuh", ["tests/test_shmem_collectives_model_cpu.py", "tests/test_examples_build_cpu.py"], ["tests/test_gpu_fused_multi.py"], True),
    ("rocm_systems_b200/csrc/shmem/*", ["tests/test_api_cpu.py"], ["tests/test_gpu_fused_multi.py", "tests/test_shmem_dma_gpu.py"], True),
    ("rocm_systems_b200/csrc/fused/fsdp_kernels.cu", ["tests/test_fsdp_rscast_emulation_cpu.py", "tests/test_protocol_model_cpu.py"], ["tests/test_gpu_fused_multi.py"], True),
    ("rocm_systems_b200/csrc/fused/gemm_fp8*", ["tests/test_fp8_reference_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/fused/*", ["tests/test_kernel_resources_cpu.py"], ["tests/test_gemm_gpu.py", "tests/test_train_ops_gpu.py", "tests/test_gpu_fused_multi.py", "tests/test_zz_fused_single_gpu.py", "tests/test_zz_no_alloc.py"], True),
    ("rocm_systems_b200/csrc/torch/*", ["tests/test_dist_cpu.py"], ["tests/test_gpu_collectives.py"], True),
    ("rocm_systems_b200/csrc/trace/kokkosp.cc", ["tests/test_kokkosp_cpu.py", "tests/test_sanitizers_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/trace/ompt.cc", ["tests/test_ompt_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/trace/*", ["tests/test_tools_cpu.py", "tests/test_sanitizers_cpu.py", "tests/test_kokkosp_cpu.py", "tests/test_ompt_cpu.py", "tests/test_instrument_cpu.py"], ["tests/test_profiler_gpu.py"], True),
    ("rocm_systems_b200/csrc/prof/sampler.cc", ["tests/test_host_sampler_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/prof/causal.cc", ["tests/test_causal_cpu.py", "tests/test_sanitizers_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/prof/instrument.cc", ["tests/test_instrument_cpu.py", "tests/test_sanitizers_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/prof/*", ["tests/test_tools_cpu.py"], ["tests/test_profiler_gpu.py"], True),
    ("rocm_systems_b200/csrc/perf/*", ["tests/test_verifiable_cpu.py", "tests/test_perf_cli_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/include/b200coll/causal.h", ["tests/test_causal_cpu.py", "tests/test_tools_cpu.py"], [], True),
    ("rocm_systems_b200/csrc/include/*", ["tests/test_bootstrap.py", "tests/test_tools_cpu.py"], ["tests/test_gpu_collectives.py"], True),
    ("rocm_systems_b200/tools/causal.py", ["tests/test_causal_cpu.py"], [], False),
    ("rocm_systems_b200/tools/pytrace.py", ["tests/test_pytrace_cpu.py", "tests/test_tools_cpu.py"], [], False),
    ("rocm_systems_b200/tools/instrument.py", ["tests/test_instrument_cpu.py"], [], False),
    ("rocm_systems_b200/tools/*", ["tests/test_tools_cpu.py", "tests/test_smi_fake.py"], [], False),
    ("rocm_systems_b200/utils/affinity.py", ["tests/test_smi_fake.py"], [], False),
    ("rocm_systems_b200/utils/apidoc.py", ["tests/test_tools_cpu.py"], [], False),
    ("rocm_systems_b200/utils/causal.py", ["tests/test_causal_cpu.py"], [], False),
    ("rocm_systems_b200/parallel/pp.py", ["tests/test_parallel_cpu.py", "tests/test_examples_build_cpu.py"], [], False),
    ("rocm_systems_b200/parallel/cp.py", ["tests/test_parallel_cpu.py", "tests/test_examples_build_cpu.py"], [], False),
    ("rocm_systems_b200/parallel/fsdp.py", ["tests/test_fsdp_layout_cpu.py"], ["tests/test_gpu_fused_multi.py"], False),
    ("rocm_systems_b200/ops/fp8.py", ["tests/test_fp8_reference_cpu.py"], [], False),
    ("rocm_systems_b200/shmem.py", ["tests/test_api_cpu.py"], ["tests/test_shmem_dma_gpu.py"], False),
    ("rocm_systems_b200/parallel/*", ["tests/test_dist_cpu.py"], ["tests/test_gpu_fused_multi.py"], False),
    ("rocm_systems_b200/utils/elastic.py", ["tests/test_elastic_cpu.py"], [], False),
    ("rocm_systems_b200/utils/checkpoint.py", ["tests/test_elastic_cpu.py"], [], False),
    ("rocm_systems_b200/utils/build.py", ["tests"], ["tests"], True),
    ("rocm_systems_b200/*", ["tests"], ["tests"], False),
    ("tests/*", ["{path}"], ["{path}"], False),
    ("bench.py", [], ["tests/test_gpu_fused_multi.py"], False),
    ("examples/causal_pipeline.cc", ["tests/test_causal_cpu.py"], [], False),
    ("examples/*", ["tests/test_examples_build_cpu.py"], [], False),
    ("pyproject.toml", ["tests/test_tools_cpu.py"], [], False),
    ("ci/*", ["tests/test_ci_select.py"], [], False),
    ("Makefile", [], [], False),
    (".github/*", [], [], False),
    ("docs/python_api.md", ["tests/test_tools_cpu.py"], [], False),
    ("docs/c_api.md", ["tests/test_tools_cpu.py"], [], False),
    ("docs/*", [], [], False),
    ("*.md", [], [], False),
    ("profiles/*", [], [], False),
]


def select(paths: Iterable[str]) -> dict:
    cpu: List[str] = []
    gpu: List[str] = []
    rebuild = False
    unknown: List[str] = []
    for p in paths:
        p = p.strip()
        if not p:
            continue
        for pat, c, g, r in RULES:
            if fnmatch.fnmatch(p, pat):
                cpu += [x.format(path=p) for x in c if "{path}" not in x or p.endswith(".py")]
                gpu += [x.format(path=p) for x in g if "{path}" not in x or p.endswith(".py")]
                rebuild |= r
                break
        else:
            unknown.append(p)
    if unknown:  # something no rule knows: be safe, run everything
        cpu, gpu, rebuild = ["tests"], ["tests"], True

    def norm(xs: List[str]) -> List[str]:
        xs = sorted(set(xs))
        return ["tests"] if "tests" in xs else xs

    return {"rebuild_native": rebuild, "cpu_tests": norm(cpu), "gpu_tests": norm(gpu), "needs_gpu": bool(gpu), "unmatched": unknown}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--paths", nargs="*", help="changed paths (default: one per line on stdin)")
    a = ap.parse_args(argv)
    paths = a.paths if a.paths is not None else sys.stdin.read().splitlines()
    print(json.dumps(select(paths), indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
