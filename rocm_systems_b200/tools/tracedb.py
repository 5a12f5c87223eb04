"""Trace database: every trace this package produces, in one SQLite file that can be queried,
summarised, merged across ranks and converted.

It plays the role of the reference's ``rocpd`` (rocprofiler-sdk/source/lib/python/rocpd:
``importer``, ``summary``, ``query``, ``csv``/``pftrace`` converters and the schema under
rocprofiler-sdk/source/share/rocprofiler-sdk-rocpd/*.sql) with a schema of its own:

    process(id, pid, rank, hostname, command)
    string(id, value)                                  -- interned names
    kernel_dispatch(process_id, device, stream, name_id, correlation_id, start_ns, end_ns,
                    registers, static_smem, dynamic_smem, grid_x..z, block_x..z, cluster_x..z)
    memory_copy(process_id, device, stream, direction_id, bytes, start_ns, end_ns, src_device, dst_device)
    region(process_id, tid, category_id, name_id, correlation_id, start_ns, end_ns)      -- API calls, markers
    collective(process_id, rank, name_id, correlation_id, count, dtype, bytes, algo, ctas,
               host_start_ns, host_end_ns, device_start_ns, device_end_ns)
    counter_sample(name_id, device, ts_ns, value)                                       -- system sampler

and the views ``kernels``, ``regions``, ``collectives``, ``top_kernels``, ``top_collectives``, ``busy``.

    python -m rocm_systems_b200.tools.tracedb import out/run*.csv -o run.db
    python -m rocm_systems_b200.tools.tracedb summary run.db
    python -m rocm_systems_b200.tools.tracedb query run.db "select * from top_kernels limit 5"
    python -m rocm_systems_b200.tools.tracedb convert run.db --format perfetto -o run.json
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import re
import socket
import sqlite3
import sys
from typing import Iterable, List, Optional, Sequence

SCHEMA = """
create table if not exists process(id integer primary key, pid integer, rank integer, hostname text, command text);
create table if not exists string(id integer primary key, value text unique);
create table if not exists kernel_dispatch(id integer primary key, process_id integer, device integer, stream integer, name_id integer,
    correlation_id integer, start_ns integer, end_ns integer, registers integer, static_smem integer, dynamic_smem integer,
    grid_x integer, grid_y integer, grid_z integer, block_x integer, block_y integer, block_z integer,
    cluster_x integer, cluster_y integer, cluster_z integer);
create table if not exists memory_copy(id integer primary key, process_id integer, device integer, stream integer, direction_id integer,
    bytes integer, start_ns integer, end_ns integer, src_device integer, dst_device integer);
create table if not exists region(id integer primary key, process_id integer, tid integer, category_id integer, name_id integer,
    correlation_id integer, start_ns integer, end_ns integer);
create table if not exists collective(id integer primary key, process_id integer, rank integer, name_id integer, correlation_id integer,
    count integer, dtype text, bytes integer, algo integer, ctas integer, host_start_ns integer, host_end_ns integer,
    device_start_ns integer, device_end_ns integer);
create table if not exists counter_sample(id integer primary key, name_id integer, device integer, ts_ns integer, value real);
create table if not exists host_sample(id integer primary key, process_id integer, tid integer, ts_ns integer, depth integer, clock text,
    leaf_id integer, stack_id integer);
create index if not exists kd_name on kernel_dispatch(name_id);
create index if not exists kd_start on kernel_dispatch(start_ns);
create index if not exists rg_start on region(start_ns);
create view if not exists kernels as
    select k.id, p.pid, p.rank, k.device, k.stream, s.value as name, k.correlation_id, k.start_ns, k.end_ns, k.end_ns - k.start_ns as duration_ns,
           k.registers, k.static_smem, k.dynamic_smem, k.grid_x, k.grid_y, k.grid_z, k.block_x, k.block_y, k.block_z
    from kernel_dispatch k join string s on s.id = k.name_id join process p on p.id = k.process_id;
create view if not exists regions as
    select r.id, p.pid, p.rank, r.tid, c.value as category, s.value as name, r.correlation_id, r.start_ns, r.end_ns, r.end_ns - r.start_ns as duration_ns
    from region r join string s on s.id = r.name_id join string c on c.id = r.category_id join process p on p.id = r.process_id;
create view if not exists collectives as
    select c.id, p.pid, c.rank, s.value as name, c.correlation_id, c.count, c.dtype, c.bytes, c.algo, c.ctas, c.host_start_ns, c.host_end_ns,
           c.device_start_ns, c.device_end_ns, c.device_end_ns - c.device_start_ns as device_ns
    from collective c join string s on s.id = c.name_id join process p on p.id = c.process_id;
create view if not exists top_kernels as
    select name, count(*) as calls, sum(duration_ns) as total_ns, avg(duration_ns) as mean_ns, min(duration_ns) as min_ns, max(duration_ns) as max_ns,
           100.0 * sum(duration_ns) / (select sum(duration_ns) from kernels) as percent
    from kernels group by name order by total_ns desc;
create view if not exists top_collectives as
    select name, bytes, count(*) as calls, sum(device_ns) as total_ns, avg(device_ns) as mean_ns, min(device_ns) as min_ns, max(device_ns) as max_ns,
           case when avg(device_ns) > 0 then bytes / avg(device_ns) else 0 end as algbw_gbps
    from collectives group by name, bytes order by total_ns desc;
create view if not exists busy as
    select p.rank, k.device, count(*) as kernels, sum(k.end_ns - k.start_ns) as kernel_ns, max(k.end_ns) - min(k.start_ns) as span_ns,
           100.0 * sum(k.end_ns - k.start_ns) / max(1, max(k.end_ns) - min(k.start_ns)) as busy_percent
    from kernel_dispatch k join process p on p.id = k.process_id group by p.rank, k.device;
"""


class TraceDB:
    """A trace as an SQLite database (the role of rocpd in the reference, rocprofiler-sdk source/lib/output/sql and
    source/lib/python/rocpd): imports the CSV files the tracers write, merges ranks, answers SQL, summarises, exports
    Perfetto JSON and CSV.
    """

    def __init__(self, path: str):
        self.path = path
        self.db = sqlite3.connect(path)
        self.db.executescript(SCHEMA)
        self._strings: dict = {}

    def close(self) -> None:
        self.db.commit()
        self.db.close()

    def __enter__(self) -> "TraceDB":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    # ---- building ----
    def string_id(self, value: str) -> int:
        sid = self._strings.get(value)
        if sid is None:
            row = self.db.execute("select id from string where value = ?", (value,)).fetchone()
            if row:
                sid = row[0]
            else:
                sid = self.db.execute("insert into string(value) values (?)", (value,)).lastrowid
            self._strings[value] = sid
        return sid

    def process_id(self, pid: int, rank: int = -1, command: str = "") -> int:
        row = self.db.execute("select id, rank from process where pid = ?", (pid,)).fetchone()
        if row:
            if rank >= 0 and row[1] < 0:
                self.db.execute("update process set rank = ? where id = ?", (rank, row[0]))
            return row[0]
        return self.db.execute("insert into process(pid, rank, hostname, command) values (?,?,?,?)",
                               (pid, rank, socket.gethostname(), command)).lastrowid

    def import_csv(self, path: str, command: str = "") -> int:
        """Imports one CSV file of any kind this package writes; the header decides the kind."""
        with open(path, newline="") as f:
            rows = list(csv.DictReader(f))
        if not rows:
            return 0
        cols = set(rows[0].keys())
        m = re.search(r"\.rank(\d+)\.", os.path.basename(path))
        file_rank = int(m.group(1)) if m else -1
        n = 0
        if "Kernel_Name" in cols:
            for r in rows:
                pid = self.process_id(int(r["Process_Id"]), file_rank, command)
                self.db.execute(
                    "insert into kernel_dispatch(process_id, device, stream, name_id, correlation_id, start_ns, end_ns, registers, static_smem,"
                    " dynamic_smem, grid_x, grid_y, grid_z, block_x, block_y, block_z, cluster_x, cluster_y, cluster_z)"
                    " values (?,?,?,?,?,?,?,?,?,?,?,?,?,?,?,?,?,?,?)",
                    (pid, int(r["Agent_Id"]), int(r["Queue_Id"]), self.string_id(r["Kernel_Name"]), int(r["Correlation_Id"]),
                     int(r["Start_Timestamp"]), int(r["End_Timestamp"]), int(r.get("Registers_Per_Thread", 0) or 0),
                     int(r.get("Static_Shared_Memory", 0) or 0), int(r.get("Dynamic_Shared_Memory", 0) or 0),
                     int(r["Grid_Size_X"]), int(r["Grid_Size_Y"]), int(r["Grid_Size_Z"]), int(r["Workgroup_Size_X"]), int(r["Workgroup_Size_Y"]),
                     int(r["Workgroup_Size_Z"]), int(r.get("Cluster_X", 0) or 0), int(r.get("Cluster_Y", 0) or 0), int(r.get("Cluster_Z", 0) or 0)))
                n += 1
        elif {"timestamp_ns", "tid", "stack"} <= cols:  # host call-stack samples (libb200sample.so); the file name carries the pid
            m2 = re.search(r"\.(\d+)\.samples\.csv$", os.path.basename(path))
            pid = self.process_id(int(m2.group(1)) if m2 else 0, file_rank, command)
            for r in rows:
                stack = r["stack"]
                self.db.execute("insert into host_sample(process_id, tid, ts_ns, depth, clock, leaf_id, stack_id) values (?,?,?,?,?,?,?)",
                                (pid, int(r["tid"]), int(r["timestamp_ns"]), int(r["depth"]), r.get("clock", ""), self.string_id(stack.rsplit(";", 1)[-1]),
                                 self.string_id(stack)))
                n += 1
        elif {"Counter", "Device", "Timestamp", "Value"} <= cols:  # system sampler
            for r in rows:
                self.db.execute("insert into counter_sample(name_id, device, ts_ns, value) values (?,?,?,?)",
                                (self.string_id(r["Counter"]), int(r["Device"]), int(r["Timestamp"]), float(r["Value"])))
                n += 1
        elif "Direction" in cols:
            for r in rows:
                pid = self.process_id(int(r["Process_Id"]), file_rank, command)
                self.db.execute("insert into memory_copy(process_id, device, stream, direction_id, bytes, start_ns, end_ns, src_device, dst_device)"
                                " values (?,?,?,?,?,?,?,?,?)",
                                (pid, int(r["Agent_Id"]), int(r["Queue_Id"]), self.string_id(r["Direction"]), int(r["Bytes"]),
                                 int(r["Start_Timestamp"]), int(r["End_Timestamp"]), int(r["Source_Agent_Id"]), int(r["Destination_Agent_Id"])))
                n += 1
        elif "Device_Start" in cols:  # collective trace of the communication library
            for r in rows:
                rank = int(r["Rank"])
                pid = self.process_id(int(r["Process_Id"]), rank, command)
                self.db.execute("insert into collective(process_id, rank, name_id, correlation_id, count, dtype, bytes, algo, ctas, host_start_ns,"
                                " host_end_ns, device_start_ns, device_end_ns) values (?,?,?,?,?,?,?,?,?,?,?,?,?)",
                                (pid, rank, self.string_id(r["Function"]), int(r["Correlation_Id"]), int(r["Count"]), r["Dtype"], int(r["Bytes"]),
                                 int(r["Algo"]), int(r["Ctas"]), int(r["Start_Timestamp"]), int(r["End_Timestamp"]), int(r["Device_Start"]),
                                 int(r["Device_End"])))
                self.db.execute("insert into region(process_id, tid, category_id, name_id, correlation_id, start_ns, end_ns) values (?,?,?,?,?,?,?)",
                                (pid, int(r["Thread_Id"]), self.string_id(r["Domain"]), self.string_id(r["Function"]), int(r["Correlation_Id"]),
                                 int(r["Start_Timestamp"]), int(r["End_Timestamp"])))
                n += 1
        elif {"Domain", "Function", "Start_Timestamp"} <= cols:  # API and marker traces
            for r in rows:
                pid = self.process_id(int(r["Process_Id"]), file_rank, command)
                self.db.execute("insert into region(process_id, tid, category_id, name_id, correlation_id, start_ns, end_ns) values (?,?,?,?,?,?,?)",
                                (pid, int(r["Thread_Id"]), self.string_id(r["Domain"]), self.string_id(r["Function"]), int(r["Correlation_Id"]),
                                 int(r["Start_Timestamp"]), int(r["End_Timestamp"])))
                n += 1
        else:
            raise ValueError(f"{path}: not a trace CSV of this package (columns {sorted(cols)})")
        self.db.commit()
        return n

    # ---- post-processing (what rocprofv3 offers as --kernel-exclude-regex, --truncate-kernels, --collection-period) ----
    def drop_kernels(self, exclude_regex: str) -> int:
        """Deletes kernel rows whose name matches; returns how many went."""
        rx = re.compile(exclude_regex)
        ids = [i for i, v in self.db.execute("select id, value from string") if rx.search(v)]
        n = 0
        for i in ids:
            n += self.db.execute("delete from kernel_dispatch where name_id = ?", (i,)).rowcount
        self.db.commit()
        return n

    @staticmethod
    def short_kernel_name(name: str) -> str:
        """``void ns::kernel<int, Foo<3> >(Args...)`` -> ``kernel``: return type, namespaces, template and call arguments go."""
        depth, out = 0, []
        for ch in name:
            if ch in "<(":
                depth += 1
            elif ch in ">)":
                depth -= 1
            elif depth == 0:
                out.append(ch)
        flat = "".join(out).strip()
        flat = flat.split(" ")[-1] if " " in flat else flat
        return flat.split("::")[-1] or name

    def truncate_kernel_names(self) -> int:
        """Rewrites every kernel name to its short form; instantiations of one template then aggregate in the statistics."""
        names = self.db.execute("select distinct s.id, s.value from string s join kernel_dispatch k on k.name_id = s.id").fetchall()
        changed = 0
        for sid, value in names:
            short = self.short_kernel_name(value)
            if short != value:
                self.db.execute("update kernel_dispatch set name_id = ? where name_id = ?", (self.string_id(short), sid))
                changed += 1
        self.db.commit()
        return changed

    def rename_kernels_by_marker(self) -> int:
        """Gives every kernel the name of the innermost marker range that was open on the launching thread when it was
        launched (what the reference launcher offers as --kernel-rename: a region of the application then shows up as ONE
        row of the kernel statistics). The launch is the runtime / driver API record with the kernel's correlation id (its
        thread and start time); without API records the kernel's device start time inside a range of the same process is
        used instead. Kernels outside every range keep their names. Returns how many were renamed."""
        marker = self.db.execute("select id from string where value = 'MARKER_API'").fetchone()
        if not marker:
            return 0
        ranges = {}   # process_id -> [(start, end, tid, name_id)], innermost first when sorted by start descending
        for pid, tid, name_id, st, en in self.db.execute("select process_id, tid, name_id, start_ns, end_ns from region where category_id = ?", (marker[0],)):
            ranges.setdefault(pid, []).append((st, en, tid, name_id))
        for v in ranges.values():
            v.sort(key=lambda r: -r[0])
        launches = {}  # (process_id, correlation_id) -> (tid, start) of the API call that launched
        for pid, tid, corr, st in self.db.execute("select process_id, tid, correlation_id, start_ns from region where category_id != ? and correlation_id != 0", (marker[0],)):
            launches.setdefault((pid, corr), (tid, st))
        renamed = 0
        for kid, pid, corr, dev_start in self.db.execute("select id, process_id, correlation_id, start_ns from kernel_dispatch").fetchall():
            tid, when = launches.get((pid, corr), (None, dev_start))
            for st, en, rtid, name_id in ranges.get(pid, []):
                if st <= when < en and (tid is None or rtid == tid):
                    self.db.execute("update kernel_dispatch set name_id = ? where id = ?", (name_id, kid))
                    renamed += 1
                    break
        self.db.commit()
        return renamed

    def keep_window(self, delay_ms: float, duration_ms: float) -> int:
        """Keeps only what started within ``duration_ms`` after ``delay_ms`` from the first record; returns rows deleted."""
        starts = [r[0] for r in (self.db.execute("select min(start_ns) from kernel_dispatch").fetchone(), self.db.execute("select min(start_ns) from region").fetchone(),
                                 self.db.execute("select min(host_start_ns) from collective").fetchone(), self.db.execute("select min(start_ns) from memory_copy").fetchone())
                  if r and r[0] is not None]
        if not starts:
            return 0
        lo = min(starts) + int(delay_ms * 1e6)
        hi = lo + int(duration_ms * 1e6) if duration_ms > 0 else 1 << 62
        n = 0
        for table, col in (("kernel_dispatch", "start_ns"), ("memory_copy", "start_ns"), ("region", "start_ns"), ("collective", "host_start_ns")):
            n += self.db.execute(f"delete from {table} where {col} < ? or {col} >= ?", (lo, hi)).rowcount
        n += self.db.execute("delete from counter_sample where ts_ns < ? or ts_ns >= ?", (lo, hi)).rowcount
        n += self.db.execute("delete from host_sample where ts_ns < ? or ts_ns >= ?", (lo, hi)).rowcount
        self.db.commit()
        return n

    @staticmethod
    def parse_iteration_ranges(words: Sequence[str]) -> List[tuple]:
        """``["[1-3]", "5", "[8-]"]`` -> ``[(1, 3), (5, 5), (8, None)]``: 1-based launch numbers, closed ranges, open end."""
        out = []
        for w in words:
            for part in w.strip().strip("[]").split(","):
                part = part.strip()
                if not part:
                    continue
                lo, dash, hi = part.partition("-")
                if not lo.isdigit() or (dash and hi and not hi.isdigit()):
                    raise ValueError(f"not a range of launch numbers: {w!r}")
                out.append((int(lo), int(hi) if hi else (None if dash else int(lo))))
        return out

    def keep_kernel_iterations(self, ranges: Sequence[tuple]) -> int:
        """Numbers the launches of every kernel name 1, 2, 3, ... in order of start (per process) and keeps only those whose
        number falls in one of ``ranges`` (the reference launcher's --kernel-iteration-range: profile the steady state of
        every kernel, not its first launches). Returns how many kernel rows were deleted."""
        seen: dict = {}
        drop = []
        for kid, pid, name_id in self.db.execute("select id, process_id, name_id from kernel_dispatch order by start_ns, id"):
            n = seen[(pid, name_id)] = seen.get((pid, name_id), 0) + 1
            if not any(lo <= n and (hi is None or n <= hi) for lo, hi in ranges):
                drop.append((kid,))
        self.db.executemany("delete from kernel_dispatch where id = ?", drop)
        self.db.commit()
        return len(drop)

    def domain_rows(self) -> List[tuple]:
        """Every timed record as ``(domain, name, duration_ns)``: kernels (KERNEL_DISPATCH), copies (MEMORY_COPY, by
        direction), API and marker regions (their category), collectives (COLLECTIVE, device time)."""
        rows = [("KERNEL_DISPATCH", n, d) for n, d in self.db.execute("select name, duration_ns from kernels")]
        rows += [("MEMORY_COPY", n, d) for n, d in self.db.execute("select s.value, m.end_ns - m.start_ns from memory_copy m join string s on s.id = m.direction_id")]
        rows += [(c, n, d) for c, n, d in self.db.execute("select category, name, duration_ns from regions")]
        rows += [("COLLECTIVE", n, d) for n, d in self.db.execute("select name, device_ns from collectives")]
        return rows

    @staticmethod
    def summarize_rows(rows: Sequence[tuple], top: int, with_domain: bool = False) -> List[dict]:
        acc: dict = {}
        for domain, name, dur in rows:
            key = (domain, name) if with_domain else (name,)
            a = acc.setdefault(key, [0, 0, None, None])
            a[0] += 1
            a[1] += dur or 0
            a[2] = dur if a[2] is None or dur < a[2] else a[2]
            a[3] = dur if a[3] is None or dur > a[3] else a[3]
        total = sum(a[1] for a in acc.values()) or 1
        out = []
        for key, (calls, tot, lo, hi) in sorted(acc.items(), key=lambda kv: -kv[1][1])[:top]:
            row = {"domain": key[0]} if with_domain else {}
            row.update({"name": key[-1], "calls": calls, "total_ns": tot, "mean_ns": tot / calls, "min_ns": lo, "max_ns": hi, "percent": 100.0 * tot / total})
            out.append(row)
        return out

    def domain_summaries(self, top: int = 15, groups: Sequence[str] = ()) -> dict:
        """``{"domains": {domain: rows}, "groups": {pattern: rows}}``: the statistics of every domain on its own (share within
        the domain), and of every requested union of domains (a regular expression on domain names; share within the
        union, rows labelled with their domain) -- the reference launcher's --summary-per-domain and --summary-groups."""
        rows = self.domain_rows()
        domains = sorted({r[0] for r in rows})
        out = {"domains": {d: self.summarize_rows([r for r in rows if r[0] == d], top) for d in domains}, "groups": {}}
        for pattern in groups:
            rx = re.compile(pattern)
            out["groups"][pattern] = self.summarize_rows([r for r in rows if rx.fullmatch(r[0])], top, with_domain=True)
        return out

    def merge(self, other_path: str) -> None:
        """Appends another database (for example another rank's) into this one."""
        src = sqlite3.connect(other_path)
        pmap, smap = {}, {}
        for sid, value in src.execute("select id, value from string"):
            smap[sid] = self.string_id(value)
        for pid_row in src.execute("select id, pid, rank, hostname, command from process"):
            pmap[pid_row[0]] = self.db.execute("insert into process(pid, rank, hostname, command) values (?,?,?,?)", pid_row[1:]).lastrowid
        for row in src.execute("select process_id, device, stream, name_id, correlation_id, start_ns, end_ns, registers, static_smem, dynamic_smem,"
                               " grid_x, grid_y, grid_z, block_x, block_y, block_z, cluster_x, cluster_y, cluster_z from kernel_dispatch"):
            row = list(row)
            row[0], row[3] = pmap[row[0]], smap[row[3]]
            self.db.execute("insert into kernel_dispatch(process_id, device, stream, name_id, correlation_id, start_ns, end_ns, registers,"
                            " static_smem, dynamic_smem, grid_x, grid_y, grid_z, block_x, block_y, block_z, cluster_x, cluster_y, cluster_z)"
                            " values (?,?,?,?,?,?,?,?,?,?,?,?,?,?,?,?,?,?,?)", row)
        for row in src.execute("select process_id, device, stream, direction_id, bytes, start_ns, end_ns, src_device, dst_device from memory_copy"):
            row = list(row)
            row[0], row[3] = pmap[row[0]], smap[row[3]]
            self.db.execute("insert into memory_copy(process_id, device, stream, direction_id, bytes, start_ns, end_ns, src_device, dst_device)"
                            " values (?,?,?,?,?,?,?,?,?)", row)
        for row in src.execute("select process_id, tid, category_id, name_id, correlation_id, start_ns, end_ns from region"):
            row = list(row)
            row[0], row[2], row[3] = pmap[row[0]], smap[row[2]], smap[row[3]]
            self.db.execute("insert into region(process_id, tid, category_id, name_id, correlation_id, start_ns, end_ns) values (?,?,?,?,?,?,?)", row)
        for row in src.execute("select process_id, rank, name_id, correlation_id, count, dtype, bytes, algo, ctas, host_start_ns, host_end_ns,"
                               " device_start_ns, device_end_ns from collective"):
            row = list(row)
            row[0], row[2] = pmap[row[0]], smap[row[2]]
            self.db.execute("insert into collective(process_id, rank, name_id, correlation_id, count, dtype, bytes, algo, ctas, host_start_ns,"
                            " host_end_ns, device_start_ns, device_end_ns) values (?,?,?,?,?,?,?,?,?,?,?,?,?)", row)
        for name_id, device, ts_ns, value in src.execute("select name_id, device, ts_ns, value from counter_sample"):
            self.db.execute("insert into counter_sample(name_id, device, ts_ns, value) values (?,?,?,?)", (smap[name_id], device, ts_ns, value))
        if src.execute("select count(*) from sqlite_master where name = 'host_sample'").fetchone()[0]:
            for row in src.execute("select process_id, tid, ts_ns, depth, clock, leaf_id, stack_id from host_sample"):
                row = list(row)
                row[0], row[5], row[6] = pmap[row[0]], smap[row[5]], smap[row[6]]
                self.db.execute("insert into host_sample(process_id, tid, ts_ns, depth, clock, leaf_id, stack_id) values (?,?,?,?,?,?,?)", row)
        src.close()
        self.db.commit()

    # ---- reading ----
    def query(self, sql: str, params: Sequence = ()) -> tuple:
        cur = self.db.execute(sql, params)
        names = [d[0] for d in cur.description] if cur.description else []
        return names, cur.fetchall()

    def summary(self, top: int = 15) -> dict:
        out = {}
        names, rows = self.query(f"select * from top_kernels limit {int(top)}")
        out["kernels"] = [dict(zip(names, r)) for r in rows]
        names, rows = self.query(f"select * from top_collectives limit {int(top)}")
        out["collectives"] = [dict(zip(names, r)) for r in rows]
        names, rows = self.query("select category, name, count(*) as calls, sum(duration_ns) as total_ns, avg(duration_ns) as mean_ns from regions"
                                 f" group by category, name order by total_ns desc limit {int(top)}")
        out["regions"] = [dict(zip(names, r)) for r in rows]
        names, rows = self.query("select s.value as direction, count(*) as calls, sum(bytes) as bytes, sum(end_ns - start_ns) as total_ns"
                                 " from memory_copy m join string s on s.id = m.direction_id group by s.value order by total_ns desc")
        out["memory_copies"] = [dict(zip(names, r)) for r in rows]
        names, rows = self.query("select * from busy order by rank, device")
        out["busy"] = [dict(zip(names, r)) for r in rows]
        names, rows = self.query("select s.value as counter, c.device, count(*) as samples, min(c.value) as min, avg(c.value) as mean, max(c.value) as max"
                                 " from counter_sample c join string s on s.id = c.name_id group by s.value, c.device order by s.value, c.device")
        out["counters"] = [dict(zip(names, r)) for r in rows]
        out["host_samples"] = self.host_profile(top)
        return out

    def host_profile(self, top: int = 15) -> List[dict]:
        """Functions by the share of host call-stack samples they appear in: ``self`` counts samples whose innermost frame is
        the function, ``inclusive`` samples that have it anywhere on the stack (once per sample, recursion or not)."""
        total = self.db.execute("select count(*) from host_sample").fetchone()[0]
        if not total:
            return []
        self_n: dict = {}
        incl: dict = {}
        for stack, leaf, cnt in self.db.execute("select st.value, lf.value, count(*) from host_sample h join string st on st.id = h.stack_id"
                                                " join string lf on lf.id = h.leaf_id group by h.stack_id"):
            self_n[leaf] = self_n.get(leaf, 0) + cnt
            for fn in set(stack.split(";")):
                incl[fn] = incl.get(fn, 0) + cnt
        rows = sorted(incl.items(), key=lambda kv: (-self_n.get(kv[0], 0), -kv[1], kv[0]))[:top]
        return [{"function": fn, "self": self_n.get(fn, 0), "self_pct": round(100.0 * self_n.get(fn, 0) / total, 2), "inclusive": n,
                 "inclusive_pct": round(100.0 * n / total, 2)} for fn, n in rows]

    def to_folded(self, path: str) -> int:
        """Host samples as folded stacks (``outer;...;leaf count`` per line), the input of flame-graph tools."""
        rows = self.db.execute("select st.value, count(*) from host_sample h join string st on st.id = h.stack_id group by h.stack_id order by 2 desc").fetchall()
        with open(path, "w") as f:
            for stack, cnt in rows:
                f.write(f"{stack} {cnt}\n")
        return len(rows)

    def to_perfetto(self, path: str) -> int:
        """Chrome/Perfetto JSON: one process per rank/pid; threads for host regions, streams for kernels and copies."""
        events: List[dict] = []
        for pid, rank in self.db.execute("select pid, rank from process"):
            events.append({"ph": "M", "pid": pid, "name": "process_name", "args": {"name": f"rank {rank} (pid {pid})" if rank >= 0 else f"pid {pid}"}})
        for pid, dev, stream, name, s, e, gx, bx, regs in self.db.execute(
                "select pid, device, stream, name, start_ns, end_ns, grid_x, block_x, registers from kernels"):
            events.append({"ph": "X", "pid": pid, "tid": f"gpu{dev} stream {stream}", "name": name, "cat": "kernel", "ts": s / 1e3,
                           "dur": max(e - s, 1) / 1e3, "args": {"grid_x": gx, "block_x": bx, "registers": regs}})
        for pid, dev, stream, direction, nbytes, s, e in self.db.execute(
                "select p.pid, m.device, m.stream, st.value, m.bytes, m.start_ns, m.end_ns from memory_copy m join process p on p.id = m.process_id"
                " join string st on st.id = m.direction_id"):
            events.append({"ph": "X", "pid": pid, "tid": f"gpu{dev} stream {stream}", "name": direction, "cat": "memcpy", "ts": s / 1e3,
                           "dur": max(e - s, 1) / 1e3, "args": {"bytes": nbytes}})
        for pid, tid, cat, name, s, e in self.db.execute("select pid, tid, category, name, start_ns, end_ns from regions"):
            events.append({"ph": "X", "pid": pid, "tid": f"{cat} {tid}", "name": name, "cat": cat, "ts": s / 1e3, "dur": max(e - s, 1) / 1e3})
        for pid, rank, name, nbytes, s, e in self.db.execute("select pid, rank, name, bytes, device_start_ns, device_end_ns from collectives"):
            if e > s:
                events.append({"ph": "X", "pid": pid, "tid": "collectives (device)", "name": name, "cat": "collective", "ts": s / 1e3,
                               "dur": (e - s) / 1e3, "args": {"bytes": nbytes, "rank": rank}})
        # Arrows from the host call to the device work it started, by correlation id: a runtime / driver launch to its kernel,
        # a collective call to its device interval (the reference's Perfetto output draws the same flows).
        marker = self.db.execute("select id from string where value = 'MARKER_API'").fetchone()
        flow = 0
        calls: dict = {}
        for ppid, pid, tid, cat, corr, st in self.db.execute(
                "select r.process_id, p.pid, r.tid, c.value, r.correlation_id, r.start_ns from region r join process p on p.id = r.process_id"
                " join string c on c.id = r.category_id where r.correlation_id != 0 and r.category_id != ?", (marker[0] if marker else -1,)):
            calls.setdefault((ppid, corr, cat == "B200COLL_API"), (pid, f"{cat} {tid}", st))
        for ppid, corr, dev, stream, st in self.db.execute("select process_id, correlation_id, device, stream, start_ns from kernel_dispatch where correlation_id != 0"):
            src = calls.get((ppid, corr, False))
            if src and src[2] <= st:
                flow += 1
                events.append({"ph": "s", "id": flow, "pid": src[0], "tid": src[1], "ts": src[2] / 1e3, "name": "launch", "cat": "flow"})
                events.append({"ph": "f", "bp": "e", "id": flow, "pid": src[0], "tid": f"gpu{dev} stream {stream}", "ts": st / 1e3, "name": "launch", "cat": "flow"})
        for ppid, corr, st, en in self.db.execute("select process_id, correlation_id, device_start_ns, device_end_ns from collective where correlation_id != 0"):
            src = calls.get((ppid, corr, True))
            if src and en > st and src[2] <= st:
                flow += 1
                events.append({"ph": "s", "id": flow, "pid": src[0], "tid": src[1], "ts": src[2] / 1e3, "name": "collective", "cat": "flow"})
                events.append({"ph": "f", "bp": "e", "id": flow, "pid": src[0], "tid": "collectives (device)", "ts": st / 1e3, "name": "collective", "cat": "flow"})
        # Communication volume as cumulative counter tracks per rank, classified the way the reference's system profiler does
        # (rocprofiler-systems source/lib/rocprof-sys/library/rocprofiler-sdk/rccl.cpp:105-180): gather-like and reducing
        # collectives and receives count as received bytes, broadcast / reduce-scatter / sends as sent bytes.
        sent_like = ("ncclBroadcast", "ncclBcast", "ncclReduceScatter", "ncclSend", "ncclScatter")
        totals: dict = {}
        for pid, rank, name, nbytes, ts in self.db.execute("select pid, rank, name, bytes, host_start_ns from collectives order by host_start_ns"):
            kind = "Comm Send" if name in sent_like else "Comm Recv"
            key = (pid, kind)
            totals[key] = totals.get(key, 0) + (nbytes or 0)
            events.append({"ph": "C", "pid": pid, "name": f"{kind} (bytes)", "cat": "comm_data", "ts": ts / 1e3, "args": {"value": totals[key]}})
        for name, dev, ts, val in self.db.execute("select s.value, c.device, c.ts_ns, c.value from counter_sample c join string s on s.id = c.name_id"):
            track = name if dev < 0 else f"{name} [{dev}]"
            events.append({"ph": "C", "pid": 0, "name": track, "ts": ts / 1e3, "args": {"value": val}})
        # Host call-stack samples: one instant per sample on the sampled thread's track, named by the innermost frame.
        for pid, tid, ts, leaf, stack in self.db.execute("select p.pid, h.tid, h.ts_ns, lf.value, st.value from host_sample h join process p on p.id = h.process_id"
                                                         " join string lf on lf.id = h.leaf_id join string st on st.id = h.stack_id"):
            events.append({"ph": "i", "s": "t", "pid": pid, "tid": f"samples {tid}", "name": leaf, "cat": "host_sample", "ts": ts / 1e3,
                           "args": {"stack": stack.split(";")}})
        with open(path, "w") as f:
            json.dump({"traceEvents": events, "displayTimeUnit": "ns"}, f)
        return len(events)

    def to_csv(self, prefix: str) -> List[str]:
        written = []
        for view in ("kernels", "regions", "collectives", "top_kernels", "top_collectives", "busy"):
            names, rows = self.query(f"select * from {view}")
            if not rows:
                continue
            path = f"{prefix}_{view}.csv"
            with open(path, "w", newline="") as f:
                w = csv.writer(f, quoting=csv.QUOTE_NONNUMERIC)
                w.writerow(names)
                w.writerows(rows)
            written.append(path)
        return written


def format_table(names: Sequence[str], rows: Iterable[Sequence], max_width: int = 60) -> str:
    def cell(v) -> str:
        if isinstance(v, float):
            return f"{v:.2f}"
        s = str(v)
        return s if len(s) <= max_width else s[:max_width - 1] + "…"

    table = [list(map(str, names))] + [[cell(v) for v in r] for r in rows]
    widths = [max(len(r[i]) for r in table) for i in range(len(names))]
    lines = ["  ".join(c.ljust(w) for c, w in zip(r, widths)) for r in table]
    lines.insert(1, "  ".join("-" * w for w in widths))
    return "\n".join(lines)


def diff(base: "TraceDB", other: "TraceDB", domains: Sequence[str] = ("KERNEL_DISPATCH", "COLLECTIVE", "MEMORY_COPY"), min_change: float = 0.0,
         top: int = 30) -> List[dict]:
    """Two traces of the same program side by side: per (domain, name) the calls, total and mean time in each and the change
    of the total in percent of the base; rows sorted by the absolute change in time, names that exist on one side only
    included. ``min_change`` (percent) hides rows that moved less. The question it answers is the one a timing regression
    asks: which kernel or collective got slower, and by how much of the whole."""
    def table(db):
        acc: dict = {}
        for domain, name, dur in db.domain_rows():
            if domain in domains:
                a = acc.setdefault((domain, name), [0, 0])
                a[0] += 1
                a[1] += dur or 0
        return acc

    a, b = table(base), table(other)
    whole = sum(v[1] for v in a.values()) or 1
    out = []
    for key in set(a) | set(b):
        ca, ta = a.get(key, (0, 0))
        cb, tb = b.get(key, (0, 0))
        change = 100.0 * (tb - ta) / ta if ta else float("inf")
        if ta and abs(change) < min_change:
            continue
        out.append({"domain": key[0], "name": key[1], "base_calls": ca, "calls": cb, "base_total_ns": ta, "total_ns": tb,
                    "base_mean_ns": ta / ca if ca else 0.0, "mean_ns": tb / cb if cb else 0.0, "change_percent": change,
                    "share_of_base_percent": 100.0 * (tb - ta) / whole})
    out.sort(key=lambda r: -abs(r["total_ns"] - r["base_total_ns"]))
    return out[:top]


UNITS = {"nsec": 1.0, "usec": 1e3, "msec": 1e6, "sec": 1e9}


def scale_units(summary, unit: str):
    """The same summary with every ``*_ns`` column divided into ``unit`` and renamed (``total_ns`` -> ``total_usec``)."""
    if unit == "nsec":
        return summary
    div = UNITS[unit]
    if isinstance(summary, dict):
        out = {}
        for k, v in summary.items():
            if isinstance(k, str) and k.endswith("_ns") and isinstance(v, (int, float)):
                out[k[:-3] + "_" + unit] = v / div
            else:
                out[k] = scale_units(v, unit)
        return out
    if isinstance(summary, list):
        return [scale_units(v, unit) for v in summary]
    return summary


def print_summary(summary: dict, file=None) -> None:
    file = file or sys.stdout    # looked up when called: the caller may have redirected it since this module was loaded
    for kind, label in (("domains", "DOMAIN"), ("groups", "GROUP")):
        for key, rows in (summary.get(kind) or {}).items():
            if rows:
                print(f"\n== {label} {key} ==", file=file)
                names = list(rows[0].keys())
                print(format_table(names, [[r[n] for n in names] for r in rows]), file=file)
    titles = {"kernels": "KERNEL_DISPATCH", "collectives": "COLLECTIVES (device time)", "regions": "API / MARKER REGIONS",
              "memory_copies": "MEMORY_COPY", "busy": "DEVICE BUSY", "counters": "SAMPLED COUNTERS", "host_samples": "HOST CALL-STACK SAMPLES"}
    for key, title in titles.items():
        rows = summary.get(key) or []
        if not rows:
            continue
        print(f"\n== {title} ==", file=file)
        names = list(rows[0].keys())
        print(format_table(names, [[r[n] for n in names] for r in rows]), file=file)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="tracedb", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("import", help="CSV trace files -> database")
    p.add_argument("files", nargs="+")
    p.add_argument("-o", "--output", required=True)
    p = sub.add_parser("merge", help="append databases into the first")
    p.add_argument("target")
    p.add_argument("others", nargs="+")
    p = sub.add_parser("summary")
    p.add_argument("db")
    p.add_argument("--top", type=int, default=15)
    p.add_argument("--json", action="store_true")
    p.add_argument("--per-domain", action="store_true", help="statistics of every domain on its own")
    p.add_argument("--groups", nargs="+", default=[], metavar="REGEX", help="statistics over unions of domains")
    p.add_argument("--units", choices=list(UNITS), default="nsec")
    p = sub.add_parser("diff", help="two traces of one program: what got slower or faster, per kernel / collective / copy")
    p.add_argument("base")
    p.add_argument("other")
    p.add_argument("--domains", nargs="+", default=["KERNEL_DISPATCH", "COLLECTIVE", "MEMORY_COPY"])
    p.add_argument("--min-change", type=float, default=0.0, metavar="PERCENT")
    p.add_argument("--top", type=int, default=30)
    p.add_argument("--units", choices=list(UNITS), default="usec")
    p.add_argument("--json", action="store_true")
    p.add_argument("--fail-above", type=float, default=None, metavar="PERCENT", help="exit code 1 when the summed time of the chosen domains grew by more")
    p = sub.add_parser("query")
    p.add_argument("db")
    p.add_argument("sql")
    p.add_argument("--format", choices=["table", "csv", "json"], default="table")
    p = sub.add_parser("convert")
    p.add_argument("db")
    p.add_argument("--format", choices=["perfetto", "csv", "folded"], required=True)
    p.add_argument("-o", "--output", required=True)
    a = ap.parse_args(argv)
    if a.cmd == "import":
        with TraceDB(a.output) as db:
            total = sum(db.import_csv(f) for f in a.files)
        print(f"{total} records -> {a.output}")
    elif a.cmd == "merge":
        with TraceDB(a.target) as db:
            for o in a.others:
                db.merge(o)
    elif a.cmd == "summary":
        with TraceDB(a.db) as db:
            s = db.summary(a.top)
            if a.per_domain or a.groups:
                extra = db.domain_summaries(a.top, a.groups)
                if not a.per_domain:
                    extra["domains"] = {}
                s.update(extra)
        s = scale_units(s, a.units)
        print(json.dumps(s, indent=1)) if a.json else print_summary(s)
    elif a.cmd == "diff":
        with TraceDB(a.base) as x, TraceDB(a.other) as y:
            rows = diff(x, y, a.domains, a.min_change, a.top)
            ta = sum(d for dom, _, d in x.domain_rows() if dom in a.domains)
            tb = sum(d for dom, _, d in y.domain_rows() if dom in a.domains)
        growth = 100.0 * (tb - ta) / ta if ta else 0.0
        if a.json:
            print(json.dumps({"base_total_ns": ta, "total_ns": tb, "change_percent": growth, "rows": rows}, indent=1))
        else:
            scaled = scale_units(rows, a.units)
            if scaled:
                names = list(scaled[0].keys())
                print(format_table(names, [[r[n] for n in names] for r in scaled]))
            print(f"\ntotal of {', '.join(a.domains)}: {ta / UNITS[a.units]:.2f} -> {tb / UNITS[a.units]:.2f} {a.units} ({growth:+.2f} %)")
        if a.fail_above is not None and growth > a.fail_above:
            return 1
    elif a.cmd == "query":
        with TraceDB(a.db) as db:
            names, rows = db.query(a.sql)
        if a.format == "json":
            print(json.dumps([dict(zip(names, r)) for r in rows], indent=1))
        elif a.format == "csv":
            w = csv.writer(sys.stdout)
            w.writerow(names)
            w.writerows(rows)
        else:
            print(format_table(names, rows))
    elif a.cmd == "convert":
        with TraceDB(a.db) as db:
            if a.format == "perfetto":
                print(f"{db.to_perfetto(a.output)} events -> {a.output}")
            elif a.format == "folded":
                print(f"{db.to_folded(a.output)} distinct stacks -> {a.output}")
            else:
                print("\n".join(db.to_csv(a.output)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
