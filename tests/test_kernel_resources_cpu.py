"""A budget for what the compiler makes of every kernel (nvcc -Xptxas -v for sm_100a, no GPU needed): no register spills
outside a short list of known ones, and the hot kernels stay inside the register counts their launch shapes need
(512-thread kernels at most 128, the GEMMs one CTA per SM). A change that pushes a kernel over shows up here, before it
shows up as lost bandwidth."""
import pytest

from rocm_systems_b200.utils import ptxas_report


@pytest.fixture(scope="module")
def rows():
    return ptxas_report.collect()


def _base(row):
    return row["name"].split("<")[0].replace("void ", "").strip("` ")


KNOWN_SPILLS = {                      # kernel -> most bytes of spill stores tolerated
    "kReduceScatterCast": 352,        # three unrolled variants for 2, 4 and 8 ranks in one kernel; known, listed as open
    "ep::epRoute": 4,
    "ep::groupedGemmFp8Kernel": 24,   # 128 fp32 accumulators per thread plus the per-expert tile arithmetic: a few tile-level values spill
    # the block-scaled fp8 main loop keeps 64 fp32 accumulators, 32 freshly loaded partial sums and both scale rows live in
    # each promotion thread; a handful of tile-level values (coordinates, limits) go to local memory once per tile
    "gemm8::gemmFp8BlockKernel": 24, "tp8::agGemmFp8Kernel": 16, "tp8::gemmRsFp8Kernel": 16,
    "emu::kRsCast": 512, "emu::kReduce": 128, "emu::kSendRecv": 256,   # the single-GPU emulation: by-value argument blocks live in local memory
}


def test_no_new_register_spills(rows):
    bad = [(r["file"], r["name"], r["spill_stores"]) for r in rows if r["spill_stores"] > KNOWN_SPILLS.get(_base(r), 0)]
    assert bad == [], bad


def test_register_budgets_of_the_hot_kernels(rows):
    limits = {"kStagedReduce": 128, "kStagedCopy": 128, "kLLAllReduce": 64, "kP2p": 64, "gemm::gemmKernel": 128, "tp::agGemmKernel": 128,
              "tp::gemmRsKernel": 128, "ep::groupedGemmKernel": 128, "ep::epDispatch": 128, "ep::epCombine": 128, "adamwKernel": 64,
              "crossEntropyFwdBwd": 64, "rmsnormFwd": 64, "gemm8::gemmFp8BlockKernel": 255}
    seen = set()
    over = []
    for r in rows:
        b = _base(r)
        if b in limits:
            seen.add(b)
            if r["registers"] > limits[b]:
                over.append((b, r["registers"], limits[b]))
    assert over == [], over
    assert seen == set(limits), sorted(set(limits) - seen)          # a renamed kernel must not drop out of the check silently
