"""Turn sweep results into a tuning file for the communication library.

Input: one or more JSON files written by ``rocm_systems_b200.bench.coll_sweep --out``, each taken
with a different forced algorithm (``B200COLL_ALGO=ll|p2p|nvls``) or with none; the algorithm of a
file is read from its ``algo`` field or given as ``NAME=FILE``. Output: the JSON the library loads
through ``B200COLL_TUNING_FILE`` — rows ``{coll, nranks, max_bytes, algo}`` in ascending size, one
row per run of sizes won by the same algorithm (the first row that covers a message wins).

    B200COLL_ALGO=p2p  torchrun ... -m rocm_systems_b200.bench.coll_sweep --no-nccl --out p2p.json
    B200COLL_ALGO=nvls torchrun ... -m rocm_systems_b200.bench.coll_sweep --no-nccl --out nvls.json
    python -m rocm_systems_b200.tools.tune p2p=p2p.json nvls=nvls.json -o tuning.json

The reference has no tuner; this closes the loop its runtime leaves to environment variables
(rocr-runtime flag.h copy-size overrides) for this library's size → algorithm table.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List, Optional, Sequence


def build_table(runs: Dict[str, dict], margin: float = 0.03) -> dict:
    """``runs``: algorithm name -> sweep document. An algorithm has to beat the incumbent of the
    previous size by ``margin`` to take over, which keeps noise from chopping the table up."""
    nranks = {d.get("nranks") for d in runs.values()}
    if len(nranks) != 1:
        raise ValueError(f"the sweeps were taken at different rank counts: {sorted(nranks)}")
    n = nranks.pop()
    per: Dict[str, Dict[int, Dict[str, float]]] = {}
    for algo, doc in runs.items():
        for r in doc["rows"]:
            per.setdefault(r["coll"], {}).setdefault(int(r["bytes"]), {})[algo] = float(r["ours_us"])
    entries: List[dict] = []
    for coll, sizes in per.items():
        incumbent: Optional[str] = None
        run_end = None
        for size in sorted(sizes):
            times = sizes[size]
            best = min(times, key=times.get)
            if incumbent in times and times[incumbent] <= times[best] * (1 + margin):
                best = incumbent
            if best != incumbent and incumbent is not None:
                entries.append({"coll": coll, "nranks": n, "max_bytes": run_end, "algo": incumbent})
            incumbent, run_end = best, size
        if incumbent is not None:
            entries.append({"coll": coll, "nranks": n, "max_bytes": 1 << 62, "algo": incumbent})
    return {"generated_by": "rocm_systems_b200.tools.tune", "entries": entries}


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="tune", description=__doc__.split("\n\n")[0])
    ap.add_argument("sweeps", nargs="+", help="[ALGO=]FILE")
    ap.add_argument("-o", "--output", required=True)
    ap.add_argument("--margin", type=float, default=0.03)
    a = ap.parse_args(argv)
    runs = {}
    for spec in a.sweeps:
        name, _, path = spec.rpartition("=")
        with open(path) as f:
            doc = json.load(f)
        name = name or doc.get("algo") or "auto"
        runs[name] = doc
    table = build_table(runs, a.margin)
    with open(a.output, "w") as f:
        json.dump(table, f, indent=1)
    print(f"{len(table['entries'])} rows -> {a.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
