"""Sharded checkpoints of the FSDP engine's optimizer state, and re-sharding to another world size.

Layout: ``<directory>/step-<N>/rank<r>.pt`` (step, world, rank and per unit the fp32 master weights and both AdamW
moments of the rank's slice) and ``<directory>/step-<N>/meta.json`` with the layout. ``meta.json`` is the commit marker
of a step: rank 0 writes it only after every rank's shard of that step is in place (it waits for the files, or for the
``barrier`` the caller passes), and only then removes older steps. A rank that dies in the middle of a save therefore
leaves an uncommitted ``step-<N>`` directory next to the last complete one, and loading picks the newest COMPLETE step.
Every shard carries its step, world and rank and is checked against ``meta.json`` on every load path, so ranks cannot
resume from different steps. Files hold only tensors, numbers and strings and are read with ``weights_only=True``.

Loading into the same world size reads one file per rank; loading into a different one (after a rank was lost, or when
scaling out) concatenates the old shards of each unit in rank order, drops the old padding, and cuts the new rank's
slice — element-wise optimizers make that exact.

The reference has no training state to checkpoint; this is the resume half of its elastic-recovery
story (a communicator is aborted and rebuilt without the lost rank, then the state is reloaded).
"""
from __future__ import annotations

import json
import os
import re
import shutil
import time
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence

import torch

KEYS = ("master", "m", "v")
_STEP_DIR = re.compile(r"^step-(\d+)$")


class CheckpointNotCommitted(RuntimeError):
    """Rank 0 gave up waiting for the other ranks' shards: the step stays uncommitted and older steps stay in place."""


def _step_dir(directory: str, step: int) -> Path:
    return Path(directory) / f"step-{int(step)}"


def _atomic_write(path: Path, write: Callable[[Path], None]) -> None:
    tmp = path.with_name(path.name + ".tmp")
    write(tmp)
    os.replace(tmp, path)  # a reader never sees a half-written file


def save_sharded(state: dict, directory: str, unit_numel: Dict[str, int], barrier: Optional[Callable[[], None]] = None, keep: int = 2,
                 commit_timeout_s: float = 300.0) -> str:
    """Write this rank's ``state`` (as returned by ``FSDPEngine.state_dict``) as its shard of step ``state['step']`` under
    ``directory``. ``unit_numel`` maps unit name to its un-padded element count (needed to re-shard later).

    ``barrier``: a callable every rank runs after its shard is on disk (for example ``torch.distributed.barrier``); when it
    is omitted, rank 0 waits until all ``world`` shard files of the step exist, up to ``commit_timeout_s`` seconds, and
    raises :class:`CheckpointNotCommitted` if they never do. Either way rank 0 then writes ``meta.json`` (the commit) and
    keeps the ``keep`` newest complete steps. The other ranks return as soon as their shard (and the barrier) is done."""
    step, world, rank = int(state["step"]), int(state["world"]), int(state["rank"])
    d = _step_dir(directory, step)
    d.mkdir(parents=True, exist_ok=True)
    path = d / f"rank{rank}.pt"
    _atomic_write(path, lambda t: torch.save(state, t))
    if barrier is not None:
        barrier()
    if rank != 0:
        return str(path)
    deadline = time.monotonic() + commit_timeout_s
    while True:
        missing = [r for r in range(world) if not (d / f"rank{r}.pt").exists()]
        if not missing:
            break
        if barrier is not None or time.monotonic() >= deadline:
            raise CheckpointNotCommitted(f"step {step}: shards of ranks {missing} never appeared under {d}; the step is not committed")
        time.sleep(0.02)
    meta = {"step": step, "world": world, "units": {n: int(k) for n, k in unit_numel.items()}}
    _atomic_write(d / "meta.json", lambda t: t.write_text(json.dumps(meta)))
    done = complete_steps(directory)
    for old in done[:-keep] if keep > 0 else []:
        shutil.rmtree(_step_dir(directory, old), ignore_errors=True)
    for other in all_steps(directory):          # uncommitted left-overs of an earlier, interrupted save
        if other < step and other not in done:
            shutil.rmtree(_step_dir(directory, other), ignore_errors=True)
    return str(path)


def all_steps(directory: str) -> List[int]:
    d = Path(directory)
    if not d.is_dir():
        return []
    return sorted(int(m.group(1)) for m in (_STEP_DIR.match(p.name) for p in d.iterdir() if p.is_dir()) if m)


def complete_steps(directory: str) -> List[int]:
    """Steps whose commit marker exists, oldest first."""
    return [s for s in all_steps(directory) if (_step_dir(directory, s) / "meta.json").exists()]


def latest_dir(directory: str) -> Path:
    """The directory of the newest committed step (``directory`` itself when it holds a ``meta.json``: a step directory
    may be passed directly)."""
    if (Path(directory) / "meta.json").exists():
        return Path(directory)
    done = complete_steps(directory)
    if not done:
        raise FileNotFoundError(f"no committed checkpoint under {directory}")
    return _step_dir(directory, done[-1])


def read_meta(directory: str) -> dict:
    return json.loads((latest_dir(directory) / "meta.json").read_text())


def _load_shard(d: Path, rank: int, meta: dict) -> dict:
    p = d / f"rank{rank}.pt"
    if not p.exists():
        raise FileNotFoundError(f"{p} is missing: the checkpoint of step {meta['step']} is incomplete")
    sd = torch.load(p, map_location="cpu", weights_only=True)
    if sd["step"] != meta["step"] or sd["world"] != meta["world"] or sd["rank"] != rank:
        raise ValueError(f"{p} belongs to step {sd['step']} / world {sd['world']} / rank {sd['rank']}, "
                         f"meta.json says step {meta['step']} / world {meta['world']}, and the file name rank {rank}")
    return sd


def load_shards(directory: str) -> List[dict]:
    d = latest_dir(directory)
    meta = json.loads((d / "meta.json").read_text())
    return [_load_shard(d, r, meta) for r in range(meta["world"])]


def reshard_unit(shards: Sequence[torch.Tensor], numel: int, new_rank: int, new_shard_numel: int) -> torch.Tensor:
    """The slice ``[new_rank * new_shard_numel, (new_rank + 1) * new_shard_numel)`` of the unit whose
    old shards are ``shards`` (rank order); positions at or beyond ``numel`` are padding and read 0."""
    flat = torch.cat([s.reshape(-1) for s in shards])[:numel]
    lo, hi = new_rank * new_shard_numel, (new_rank + 1) * new_shard_numel
    out = torch.zeros(new_shard_numel, dtype=flat.dtype)
    if lo < numel:
        n = min(hi, numel) - lo
        out[:n] = flat[lo:lo + n]
    return out


def reshard(shards: List[dict], meta: dict, new_rank: int, new_world: int, new_shard_numel: Dict[str, int]) -> dict:
    """A state dict for rank ``new_rank`` of ``new_world`` built from all old shards."""
    units = {}
    for name, numel in meta["units"].items():
        units[name] = {k: reshard_unit([sd["units"][name][k] for sd in shards], numel, new_rank, new_shard_numel[name]) for k in KEYS}
    return {"step": meta["step"], "world": new_world, "rank": new_rank, "units": units}


def load_for(directory: str, rank: int, world: int, shard_numel: Dict[str, int]) -> dict:
    """The state dict rank ``rank`` of ``world`` should load from the newest committed step: its own file when the
    checkpoint was written by the same world size, a re-sharded one otherwise."""
    d = latest_dir(directory)
    meta = json.loads((d / "meta.json").read_text())
    if meta["world"] == world:
        sd = _load_shard(d, rank, meta)
        if all(sd["units"][n]["master"].numel() == shard_numel[n] for n in meta["units"]):
            return sd
    return reshard(load_shards(str(d)), meta, rank, world, shard_numel)


def save_engine(engine, directory: str, barrier: Optional[Callable[[], None]] = None, keep: int = 2) -> str:
    """Convenience for ``FSDPEngine``: this rank's shard plus the layout; see :func:`save_sharded` for the commit rule."""
    return save_sharded(engine.state_dict(), directory, {u.name: u.numel for u in engine.units}, barrier=barrier, keep=keep)


def load_engine(engine, directory: str) -> None:
    sd = load_for(directory, engine.rank, engine.world, {u.name: u.shard_numel for u in engine.units})
    engine.load_state_dict(sd)
