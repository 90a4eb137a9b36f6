"""Host-side guards: slab-membership checks of the peer kernels' inputs, rank-invariant kernel seeds, and the
checkpoint round trip of user-defined preconditioner schedules."""

import pytest
import torch

import heavyball_b200 as hb
from heavyball_b200 import lowering
from heavyball_b200.parallel.ddp import check_slab_view
from heavyball_b200.utils import pickle_compat


def test_slab_view_check_accepts_views_and_rejects_everything_else():
    slab, n = 1 << 20, 4096
    f32, bf16 = torch.float32, torch.bfloat16
    check_slab_view("gradient", slab + 64, n, f32, slab, 1 << 16, f32, 64)  # inside, right offset
    with pytest.raises(RuntimeError, match="dtype"):
        check_slab_view("gradient", slab + 64, n, bf16, slab, 1 << 16, f32, 64)
    with pytest.raises(RuntimeError, match="does not live in the symmetric slab"):
        check_slab_view("gradient", slab - 16, n, f32, slab, 1 << 16, f32)  # starts before the slab
    with pytest.raises(RuntimeError, match="does not live in the symmetric slab"):
        check_slab_view("parameter", slab + (1 << 16) - 8, n, f32, slab, 1 << 16, f32)  # runs past the end
    with pytest.raises(RuntimeError, match="expected 64"):
        check_slab_view("parameter", slab + 128, n, f32, slab, 1 << 16, f32, 64)  # inside, wrong segment


def _seeds(opt, steps=3):
    out = []
    for gi, group in enumerate(opt.param_groups):
        for step in range(1, steps + 1):
            group["step"] = step
            out += [lowering._seed(opt, group, launch) for launch in range(3)]
            group["step"] = None
    return out


def test_kernel_seeds_depend_only_on_seed_group_position_step_and_launch():
    def make(order):
        params = [torch.nn.Parameter(torch.zeros(4)) for _ in range(3)]
        junk = [object() for _ in range(order * 7)]  # shifts heap addresses between the two constructions
        opt = hb.AdamW([{"params": params[:1]}, {"params": params[1:]}], lr=1e-3)
        del junk
        return opt

    torch.manual_seed(1234)
    a = _seeds(make(0))
    torch.manual_seed(1234)
    b = _seeds(make(3))
    assert a == b
    assert len(set(a)) == len(a)  # and they differ by group, step and launch
    torch.manual_seed(99)
    assert _seeds(make(0)) != a


def custom_schedule(step):  # module level: pickle refers to it by name
    return 0.25


def test_user_schedule_round_trips_only_when_allowed():
    p = torch.nn.Parameter(torch.randn(4, 4))
    opt = hb.SOAP([p], lr=1e-2)
    opt.precond_schedule = custom_schedule
    sd = opt.state_dict()
    fresh = hb.SOAP([torch.nn.Parameter(torch.randn(4, 4))], lr=1e-2)
    before = fresh.precond_schedule
    with pytest.warns(UserWarning, match="not on the allow-list"):
        fresh.load_state_dict(sd)  # refused: keeps its own schedule, everything else loads
    assert fresh.precond_schedule == before
    pickle_compat.allow_global(custom_schedule)
    try:
        fresh.load_state_dict(sd)
        assert fresh.precond_schedule is custom_schedule
    finally:
        pickle_compat.allowed_globals.clear()
