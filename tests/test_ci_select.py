"""The change-to-tests selection used by CI."""
import importlib.util
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
spec = importlib.util.spec_from_file_location("select_tests", ROOT / "ci" / "select_tests.py")
sel = importlib.util.module_from_spec(spec)
spec.loader.exec_module(sel)


def test_docs_only_changes_need_nothing():
    r = sel.select(["README.md", "profiles/results_8gpu.md"])
    assert r == {"rebuild_native": False, "cpu_tests": [], "gpu_tests": [], "needs_gpu": False, "unmatched": []}


def test_kernel_change_needs_gpu_and_rebuild():
    r = sel.select(["rocm_systems_b200/csrc/coll/kernels.cuh"])
    assert r["rebuild_native"] and r["needs_gpu"] and "tests/test_gpu_collectives.py" in r["gpu_tests"] and r["cpu_tests"] == ["tests/test_planner_cpu.py", "tests/test_protocol_interleavings_cpu.py", "tests/test_protocol_model_cpu.py", "tests/test_staged_emulation_cpu.py"]


def test_specific_rules_win_over_general_ones():
    r = sel.select(["rocm_systems_b200/csrc/core/bootstrap.cc", "rocm_systems_b200/parallel/pp.py"])
    assert r["cpu_tests"] == ["tests/test_bootstrap.py", "tests/test_examples_build_cpu.py", "tests/test_parallel_cpu.py", "tests/test_sanitizers_cpu.py"] and not r["needs_gpu"]


def test_changed_test_file_runs_itself_and_unknown_paths_run_everything():
    assert sel.select(["tests/test_tools_cpu.py"])["cpu_tests"] == ["tests/test_tools_cpu.py"]
    r = sel.select(["setup.cfg"])
    assert r["cpu_tests"] == ["tests"] and r["gpu_tests"] == ["tests"] and r["unmatched"] == ["setup.cfg"]


def test_every_listed_test_file_exists():
    for _, cpu, gpu, _ in sel.RULES:
        for t in cpu + gpu:
            if "{path}" not in t:
                assert (ROOT / t).exists(), t
