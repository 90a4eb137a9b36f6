"""Failure paths of the owner-rank exchange, made on the host with CPU / gloo ranks (no GPU is involved, nothing hangs:
every collective runs under a short process-group timeout).

* a shard-size table that does not add up to the parameter is refused when the plan is built;
* a rank whose local slice is shorter than the size it announced makes the exchange raise on every rank - at once on
  the faulty rank, within the timeout on its peers;
* a rank that leaves between two steps makes the survivors' next exchange raise within the timeout instead of waiting
  for ever.
"""

import datetime
import math
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import heavyball_b200 as hb
from heavyball_b200.parallel import fsdp

TIMEOUT_S = 6


def test_plan_rejects_sizes_that_do_not_sum_to_the_parameter():
    p = torch.nn.Parameter(torch.zeros(10))
    info = fsdp.ShapeInfo((4, 5), 0, 20, owner=0, param_idx=0, sizes=[10, 7])  # 17 != 20
    with pytest.raises(RuntimeError, match="sum to 17, expected 20"):
        fsdp._Plan([(p, info)], rank=0, ws=2)


def _sharded_muon(rank, world, shape=(8, 6), lie=0):
    """Every rank holds half of one matrix; ``lie`` makes this rank's real slice shorter than announced."""
    total = math.prod(shape)
    half = total // world
    sizes = [half] * world
    full = torch.arange(total, dtype=torch.float32) / total
    mine = full[rank * half : (rank + 1) * half - lie].clone()
    p = torch.nn.Parameter(mine)
    info = fsdp.ShapeInfo(shape, rank * half, total, owner=0, param_idx=0, sizes=sizes)
    return p, hb.Muon([p], lr=1e-2, orig_shapes={id(p): info})


def _record(path, rank, what):
    with open(f"{path}.{rank}", "w") as fh:
        fh.write(what)


def _worker(rank, world, store_path, scenario, result_path):
    dist.init_process_group("gloo", store=dist.FileStore(store_path, world), rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=TIMEOUT_S))  # fmt: skip
    started = time.time()
    try:
        if scenario == "short_payload":
            p, opt = _sharded_muon(rank, world, lie=2 if rank == 1 else 0)
            p.grad = torch.ones_like(p)
            opt.step()
            _record(result_path, rank, "no error")
        elif scenario == "rank_leaves":
            p, opt = _sharded_muon(rank, world)
            p.grad = torch.ones_like(p)
            opt.step()  # a complete step with everybody present
            if rank == 1:
                _record(result_path, rank, "left")
                return  # leaves between steps: nothing of its own is in flight
            p.grad = torch.ones_like(p)
            opt.step()
            _record(result_path, rank, "no error")
    except Exception as err:  # noqa: BLE001 - the test inspects what was raised
        _record(result_path, rank, f"{type(err).__name__} after {time.time() - started:.1f}s: {str(err)[:200]}")
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(scenario, world=2):
    with tempfile.TemporaryDirectory() as tmp:
        store, result = os.path.join(tmp, "store"), os.path.join(tmp, "result")
        t0 = time.time()
        mp.spawn(_worker, args=(world, store, scenario, result), nprocs=world, join=True)
        took = time.time() - t0
        return [open(f"{result}.{r}").read() for r in range(world)], took


def test_short_payload_raises_on_every_rank_within_the_timeout():
    out, took = _run("short_payload")
    assert all("Error" in o for o in out), out
    assert took < 4 * TIMEOUT_S + 30, took


def test_survivor_raises_when_a_rank_leaves_between_steps():
    out, took = _run("rank_leaves")
    assert out[1] == "left"
    assert "Error" in out[0], out
    assert took < 4 * TIMEOUT_S + 30, took

