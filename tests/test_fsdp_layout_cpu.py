"""The FSDP engine's flat-buffer layout and the checkpoint helpers on CPU tensors: shard sizes,
alignment gaps, parameter views, and a save / re-shard / load round trip through the same
state-dict format the engine uses."""
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from rocm_systems_b200.parallel.fsdp import FlatUnit, ParamSpec  # noqa: E402
from rocm_systems_b200.utils import checkpoint  # noqa: E402

SPECS = [ParamSpec("w", (5, 7), std=0.02), ParamSpec("n", (7,), "ones"), ParamSpec("v", (3, 3), std=0.5)]


def _units(world, seed=3):
    return [FlatUnit("u", SPECS, r, world, torch.device("cpu"), seed) for r in range(world)]


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_shards_tile_the_flat_buffer(world):
    us = _units(world)
    u0 = us[0]
    assert u0.padded == u0.shard_numel * world and u0.padded >= u0.numel
    assert all(u.shard_numel == u0.shard_numel and u.master.numel() == u0.shard_numel for u in us)
    flat = torch.cat([u.master for u in us])
    # every rank drew the same full-precision values: the concatenation equals the one-rank layout
    ref = _units(1)[0].master
    assert torch.equal(flat[:u0.numel], ref[:u0.numel])
    # the norm weights are ones, the gaps and the tail are zeros
    o = u0.offsets["n"]
    assert torch.equal(flat[o:o + 7], torch.ones(7))
    for a, b in u0.gaps:
        assert torch.equal(flat[a:b], torch.zeros(b - a))
    covered = sum(s.numel for s in SPECS) + sum(b - a for a, b in u0.gaps)
    assert covered == u0.padded                                     # parameters and gaps account for every element


def test_parameter_views_alias_the_full_buffer():
    u = _units(1)[0]
    assert u.params["w"].shape == (5, 7) and u.params["n"].shape == (7,)
    u.full[u.offsets["v"]] = 42.0
    assert u.params["v"].flatten()[0].item() == 42.0                # a view, not a copy
    assert all(p.requires_grad for p in u.params.values())


class _Engine:
    """What checkpoint.save_engine / load_engine need of an engine, over CPU units."""

    def __init__(self, unit, rank, world):
        self.units, self.rank, self.world, self.step_count = [unit], rank, world, 0

    def state_dict(self):
        return {"step": self.step_count, "world": self.world, "rank": self.rank,
                "units": {u.name: {"master": u.master.clone(), "m": u.m.clone(), "v": u.v.clone()} for u in self.units}}

    def load_state_dict(self, sd):
        assert sd["world"] == self.world and sd["rank"] == self.rank
        self.step_count = sd["step"]
        for u in self.units:
            for k in checkpoint.KEYS:
                getattr(u, k).copy_(sd["units"][u.name][k])


@pytest.mark.parametrize("old_world,new_world", [(4, 4), (4, 2), (3, 8), (8, 1)])
def test_checkpoint_round_trip_across_world_sizes(tmp_path, old_world, new_world):
    olds = [_Engine(u, r, old_world) for r, u in enumerate(_units(old_world))]
    for e in reversed(olds):                  # rank 0 last: it commits the step once every shard is there
        e.step_count = 17
        e.units[0].m.uniform_(-1, 1)
        e.units[0].v.uniform_(0, 1)
        checkpoint.save_engine(e, str(tmp_path))
    want = {k: torch.cat([getattr(e.units[0], k) for e in olds])[:olds[0].units[0].numel] for k in checkpoint.KEYS}
    news = [_Engine(u, r, new_world) for r, u in enumerate(_units(new_world, seed=99))]      # other initial values
    for e in news:
        checkpoint.load_engine(e, str(tmp_path))
        assert e.step_count == 17
    for k in checkpoint.KEYS:
        got = torch.cat([getattr(e.units[0], k) for e in news])
        assert torch.equal(got[:want[k].numel()], want[k])
        assert torch.equal(got[want[k].numel():], torch.zeros(got.numel() - want[k].numel()))   # padding reads zero


def test_model_table_and_parameter_counts():
    from rocm_systems_b200.models.llama import LlamaConfig

    assert abs(LlamaConfig.by_name("llama3-8b").param_count() / 1e9 - 8.03) < 0.01
    assert abs(LlamaConfig.by_name("llama3-70b").param_count() / 1e9 - 70.55) < 0.05
    assert abs(LlamaConfig.by_name("llama2-7b").param_count() / 1e9 - 6.74) < 0.01
    assert abs(LlamaConfig.by_name("llama3.2-1b").param_count() / 1e9 - 1.50) < 0.01      # untied embeddings: 1.24 B + the output matrix
    with pytest.raises(KeyError):
        LlamaConfig.by_name("nope")
    m8 = LlamaConfig.llama3_8b().memory_per_gpu_gib(8, 4096)
    m1 = LlamaConfig.llama3_8b().memory_per_gpu_gib(1, 4096)
    assert abs(m1["state"] - 14 * 8.03e9 / 2**30) < 0.5 and abs(m8["state"] * 8 - m1["state"]) < 1e-6
    assert m1["total"] < 180                                                   # the benchmark's configuration fits one 180 GB GPU
    big = LlamaConfig.llama3_70b()
    assert big.memory_per_gpu_gib(8, 8192)["total"] > 180 > big.memory_per_gpu_gib(8, 2048)["total"]   # 70B on 8 GPUs: 2048 tokens per micro-batch fit, 8192 do not


def test_learning_rate_schedules():
    from rocm_systems_b200.utils import schedule

    s = schedule.warmup_cosine(peak=1.0, warmup=10, total=110, floor=0.1)
    assert s(0) == pytest.approx(0.1) and s(9) == pytest.approx(1.0) and s(10) == pytest.approx(1.0)
    assert s(60) == pytest.approx(0.55) and s(110) == pytest.approx(0.1) and s(10_000) == pytest.approx(0.1)
    assert all(s(i) >= s(i + 1) for i in range(10, 120))
    lin = schedule.warmup_linear(1.0, 0, 100)
    assert lin(0) == 1.0 and lin(50) == pytest.approx(0.5) and lin(100) == 0.0
    wsd = schedule.warmup_stable_decay(2.0, 5, 50, 100, floor=0.0)
    assert wsd(4) == pytest.approx(2.0) and wsd(49) == 2.0 and wsd(75) == pytest.approx(1.0) and wsd(100) == 0.0
    with pytest.raises(ValueError):
        schedule.warmup_cosine(1.0, 10, 10)
