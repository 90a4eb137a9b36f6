"""The allocation-free cautious AdamW entry point against the regular (allocating) caution path.

Some callers of the optimizer kernels cannot allocate device memory while stepping (fixed memory
budgets, a device handed to another allocator, C clients without a tensor library); for them the library exports one C
symbol whose scratch lives in a fixed in-library array.  This test calls that exported symbol through
ctypes twice in a row - the second call reuses the array the first one dirtied - and checks parameters
and both moments against ``ops.fused_chain``'s two-phase caution path on identical inputs.

Collected last on purpose (file name), so a stop-at-first-failure run has exercised everything else.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular_path(p, g, m, v, *, lr, b1, b2, eps, wd):
    from heavyball_b200 import ops

    scratch = [torch.empty_like(p)]
    masked = torch.zeros(1, dtype=torch.int32, device=p.device)
    ops.fused_chain(g=[g], u=scratch, s0=[m], s1=[v], masked=masked, count_caution=1, algo=ops.ADAM, n_state=2,
                    out_mode=ops.OUT_UPDATE, dt_g=ops.F32, dt_u=ops.F32, dt_s=ops.F32, dt_p=ops.NONE, b1=b1, b2=b2,
                    eps=eps)  # fmt: skip
    ops.fused_chain(p=[p], u=scratch, masked=masked, algo=ops.IDENTITY, u_is_input=1, caution_apply=1,
                    out_mode=ops.OUT_PARAM, dt_u=ops.F32, dt_p=ops.F32, dt_g=ops.NONE, dt_s=ops.NONE, lr=lr, wd=wd)  # fmt: skip


@pytest.mark.parametrize("numel", [1, 4097, 1 << 20])
def test_noalloc_matches_regular_path_twice(numel):
    from heavyball_b200.ops import noalloc

    torch.manual_seed(numel)
    dev = "cuda"
    p0 = torch.randn(numel, device=dev)
    state = {k: [p0.clone(), torch.zeros(numel, device=dev), torch.zeros(numel, device=dev)] for k in ("a", "b")}
    hyper = dict(lr=1e-2, eps=1e-8, wd=0.1)
    for step in (1, 2):
        g = torch.randn(numel, device=dev)
        b1 = 1 - (1 - 0.9) / (1 - 0.9**step)
        b2 = 1 - (1 - 0.99) / (1 - 0.99**step)
        pa, ma, va = state["a"]
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        reserved_before = torch.cuda.memory_reserved()
        noalloc.cautious_adamw_step(pa, g, ma, va, lr=hyper["lr"], beta1=b1, beta2=b2, eps=hyper["eps"],
                                    weight_decay=hyper["wd"])  # fmt: skip
        torch.cuda.synchronize()
        if step == 2:  # the first call on a device may load the kernels' module; from then on nothing may move
            assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free step changed free device memory"
        assert torch.cuda.memory_reserved() == reserved_before
        pb, mb, vb = state["b"]
        _regular_path(pb, g, mb, vb, lr=hyper["lr"], b1=b1, b2=b2, eps=hyper["eps"], wd=hyper["wd"])
        torch.cuda.synchronize()
        for got, want in zip(state["a"], state["b"]):
            torch.testing.assert_close(got, want, rtol=2e-5, atol=2e-6)
    assert not torch.equal(state["a"][0], p0)


def test_noalloc_refuses_oversize():
    from heavyball_b200.ops import noalloc

    n = noalloc.MAX_ELEMS + 1
    t = [torch.zeros(n, device="cuda") for _ in range(4)]
    with pytest.raises(ValueError, match="exceeds the fixed scratch capacity"):
        noalloc.cautious_adamw_step(*t, lr=1e-3, beta1=0.9, beta2=0.99, eps=1e-8)
