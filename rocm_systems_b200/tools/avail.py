"""List every setting of the communication library: environment names, current value, default and
meaning — what ``rocprof-sys-avail`` is to the reference's settings
(rocprofiler-systems/source/bin/rocprof-sys-avail) and ``Flag::Refresh`` is to its runtime's
(rocr-runtime/runtime/hsa-runtime/core/util/flag.h:78-299).

    python -m rocm_systems_b200.tools.avail [--json] [--changed]
"""
from __future__ import annotations

import argparse
import ctypes
import json
import sys
from typing import List, Optional, Sequence

from .. import _lib


def settings() -> List[dict]:
    lib = _lib.load()
    lib.b200collDescribeSettings.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    lib.b200collDescribeSettings.restype = ctypes.c_size_t
    need = lib.b200collDescribeSettings(None, 0)
    buf = ctypes.create_string_buffer(need)
    lib.b200collDescribeSettings(buf, need)
    return json.loads(buf.value.decode())


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="avail", description=__doc__.split("\n\n")[0])
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--changed", action="store_true", help="only settings whose value differs from the default")
    a = ap.parse_args(argv)
    rows = settings()
    if a.changed:
        rows = [r for r in rows if _norm(r["value"]) != _norm(r["default"])]
    if a.json:
        print(json.dumps(rows, indent=1))
        return 0
    w = max((len(r["env"][0]) for r in rows), default=10)
    for r in rows:
        alias = f" (also {r['env'][1]})" if len(r["env"]) > 1 else ""
        print(f"{r['env'][0]:<{w}}  = {r['value'] or '\"\"':<12} default {r['default'] or '\"\"':<10} {r['doc']}{alias}")
    return 0


def _norm(v: str) -> str:
    """'64M' and '67108864' are the same value."""
    v = v.strip()
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    if v and v[-1].upper() in mult and v[:-1].replace(".", "", 1).isdigit():
        return str(int(float(v[:-1]) * mult[v[-1].upper()]))
    return v


if __name__ == "__main__":
    sys.exit(main())
