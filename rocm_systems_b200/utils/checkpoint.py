"""Sharded checkpoints of the FSDP engine's optimizer state, and re-sharding to another world size.

Every rank writes its own shard file (`rank<r>.pt`: step, world, rank and per unit the fp32 master
weights and both AdamW moments of its slice) plus, on rank 0, `meta.json` with the layout. Loading
into the same world size reads one file per rank; loading into a different one (after a rank was
lost, or when scaling out) concatenates the old shards of each unit in rank order, drops the old
padding, and cuts the new rank's slice — element-wise optimizers make that exact.

The reference has no training state to checkpoint; this is the resume half of its elastic-recovery
story (a communicator is aborted and rebuilt without the lost rank, then the state is reloaded).
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, List, Sequence

import torch

KEYS = ("master", "m", "v")


def save_sharded(state: dict, directory: str, unit_numel: Dict[str, int]) -> str:
    """Write this rank's ``state`` (as returned by ``FSDPEngine.state_dict``) under ``directory``.
    ``unit_numel`` maps unit name to its un-padded element count (needed to re-shard later)."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    path = d / f"rank{state['rank']}.pt"
    tmp = path.with_suffix(".tmp")
    torch.save(state, tmp)
    os.replace(tmp, path)  # a reader never sees a half-written shard
    if state["rank"] == 0:
        meta = {"step": state["step"], "world": state["world"], "units": {n: int(k) for n, k in unit_numel.items()}}
        mtmp = d / "meta.json.tmp"
        mtmp.write_text(json.dumps(meta))
        os.replace(mtmp, d / "meta.json")
    return str(path)


def read_meta(directory: str) -> dict:
    return json.loads((Path(directory) / "meta.json").read_text())


def load_shards(directory: str) -> List[dict]:
    meta = read_meta(directory)
    out = []
    for r in range(meta["world"]):
        p = Path(directory) / f"rank{r}.pt"
        if not p.exists():
            raise FileNotFoundError(f"{p} is missing: the checkpoint of step {meta['step']} is incomplete")
        sd = torch.load(p, map_location="cpu", weights_only=False)
        if sd["step"] != meta["step"] or sd["world"] != meta["world"]:
            raise ValueError(f"{p} belongs to step {sd['step']} / world {sd['world']}, meta.json says {meta['step']} / {meta['world']}")
        out.append(sd)
    return out


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
    """The state dict rank ``rank`` of ``world`` should load: its own file when the checkpoint was
    written by the same world size, a re-sharded one otherwise."""
    meta = read_meta(directory)
    if meta["world"] == world:
        sd = torch.load(Path(directory) / f"rank{rank}.pt", map_location="cpu", weights_only=False)
        if all(sd["units"][n]["master"].numel() == shard_numel[n] for n in meta["units"]):
            return sd
    return reshard(load_shards(directory), meta, rank, world, shard_numel)


def save_engine(engine, directory: str) -> str:
    """Convenience for ``FSDPEngine``: this rank's shard plus the layout."""
    return save_sharded(engine.state_dict(), directory, {u.name: u.numel for u in engine.units})


def load_engine(engine, directory: str) -> None:
    sd = load_for(directory, engine.rank, engine.world, {u.name: u.shard_numel for u in engine.units})
    engine.load_state_dict(sd)
