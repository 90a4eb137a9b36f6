"""Checkpoint migration CLI: version detection, class renames, flat 1.x -> nested layout, end to end."""

import torch

import heavyball_b200 as hb
from heavyball_b200 import migrate


def _v1_state():
    return {
        "state": {0: {"update_by_adam_exp_avg": torch.ones(3, 2), "update_by_adam_exp_avg_sq": torch.full((3, 2), 2.0),
                      "is_initialized": [0]},
                  1: {"update_by_adam_exp_avg": [torch.ones(2)], "update_by_adam_exp_avg_sq": [torch.ones(2)]}},
        "param_groups": [{"params": [0, 1], "lr": 1e-3, "betas": [0.9, 0.99], "eps": 1e-8, "weight_decay": 0.0,
                          "foreach": True, "stochastic_schedule": False, "warmup_steps": 0, "caution": False}],
    }  # fmt: skip


def test_version_detection():
    assert migrate._detect_version(_v1_state()) == 1
    v2 = {"state": {0: {0: {"k": torch.ones(1)}}}, "param_groups": [{"params": [0], "foreach": True}]}
    assert migrate._detect_version(v2) == 2
    v3 = {"state": {0: {0: {"k": torch.ones(1)}}}, "param_groups": [{"params": [0], "multi_tensor": True}]}
    assert migrate._detect_version(v3) == 3
    assert migrate._detect_version({"state": {}, "param_groups": [{"params": [], "multi_tensor": True}]}) == 3


def test_former_class_names_resolve():
    assert len(migrate._CLASS_RENAMES) == 41
    for old, new in migrate._CLASS_RENAMES.items():
        assert hasattr(hb, new), (old, new)
    assert migrate._load_optimizer_class("heavyball.ForeachCachedDelayedPSGDKron") is hb.PSGDKron
    assert migrate._load_optimizer_class("PaLMForeachSOAP") is hb.SOAP


def test_v1_to_current_layout():
    out = migrate.migrate_state_dict(_v1_state(), "heavyball.ForeachAdamW")
    st = out["state"][0][0]
    assert set(st) == {"update_by_adam_exp_avg_0", "update_by_adam_exp_avg_sq_0", "is_initialized"}
    assert st["is_initialized"] == [0] and torch.equal(st["update_by_adam_exp_avg_sq_0"], torch.full((3, 2), 2.0))
    assert out["state"][1][0]["update_by_adam_exp_avg_0"].shape == (2,)
    g = out["param_groups"][0]
    assert g["multi_tensor"] is True and "foreach" not in g and "stochastic_schedule" not in g
    assert "inner_group" in out["heavyball"]


def test_v2_groups_are_modernised_and_v3_untouched():
    v2 = {"state": {0: {0: {"update_by_adam_exp_avg_0": torch.ones(1)}}},
          "param_groups": [{"params": [0], "foreach": False, "stochastic_schedule": True}],
          "heavyball": {"precond_rng": b"x", "inner_group": {"stochastic_schedule": None}}}  # fmt: skip
    out = migrate.migrate_state_dict(v2, "AdamW")
    assert out["param_groups"][0] == {"params": [0], "multi_tensor": False}
    assert out["heavyball"] == {"inner_group": {}}
    v3 = {"state": {}, "param_groups": [{"params": [], "multi_tensor": True}]}
    assert migrate.migrate_state_dict(v3, "AdamW") == v3


def test_cli_end_to_end_then_load(tmp_path, capsys):
    path = tmp_path / "ckpt.pt"
    torch.save({"model": {}, "train": {"optimizer": _v1_state()}}, path)
    assert migrate.main([str(path), "heavyball.ForeachAdamW", "--state-key", "train.optimizer", "--dry-run"]) == 0
    assert "Dry run" in capsys.readouterr().out
    out = tmp_path / "new.pt"
    assert migrate.main([str(path), "heavyball.ForeachAdamW", "--state-key", "train.optimizer", "-o", str(out)]) == 0
    sd = torch.load(out, weights_only=False)["train"]["optimizer"]
    params = [torch.nn.Parameter(torch.zeros(3, 2)), torch.nn.Parameter(torch.zeros(2))]
    opt = hb.AdamW(params, lr=1e-3)
    opt.load_state_dict(sd)
    for p in params:
        p.grad = torch.ones_like(p)
    opt.step()
    assert torch.isfinite(params[0]).all() and opt.state[params[0]][0]["update_by_adam_exp_avg_0"].mean() > 0.9
