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


# ---------------------------------------------------------------------------------------- names

import pytest  # noqa: E402

_RENAMES = sorted(migrate._CLASS_RENAMES.items())
_CURRENT = ["AdamW", "SOAP", "PSGDKron", "Muon", "SFAdamW", "LaProp", "ADOPT"]


@pytest.mark.parametrize("old,new", _RENAMES)
def test_every_former_name_loads_its_successor(old, new):
    assert migrate._resolve_class_name(old) == new
    assert migrate._load_optimizer_class(f"heavyball.{old}") is getattr(hb, new)
    assert migrate._load_optimizer_class(old) is getattr(hb, new)  # bare name: the package is implied


@pytest.mark.parametrize("name", _CURRENT)
def test_current_names_pass_through(name):
    assert migrate._resolve_class_name(name) == name
    assert migrate._load_optimizer_class(f"heavyball.{name}") is getattr(hb, name)
    assert migrate._load_optimizer_class(f"heavyball_b200.{name}") is getattr(hb, name)


def test_unknown_class_is_an_error():
    with pytest.raises(ValueError, match="not found"):
        migrate._load_optimizer_class("heavyball.NoSuchOptimizer")
    with pytest.raises(ModuleNotFoundError):
        migrate._load_optimizer_class("no_such_package_anywhere.AdamW")


# ---------------------------------------------------------------------------------------- small helpers


@pytest.mark.parametrize("value,want", [(None, set()), (3, {3}), ([1, 2, 2], {1, 2}), ((0,), {0}), ({4, 5}, {4, 5})])
def test_initialised_markers_become_sets(value, want):
    assert migrate._as_set(value) == want


@pytest.mark.parametrize("entry,shape,dtype", [
    ({"a": torch.zeros(3, 2, dtype=torch.bfloat16)}, (3, 2), torch.bfloat16),
    ({"step": torch.zeros((), dtype=torch.int64), "m": torch.zeros(5)}, (5,), torch.float32),
    ({"views": [torch.zeros(2, 2, dtype=torch.float64), torch.zeros(7)]}, (2, 2), torch.float64),
    ({"scalar": torch.zeros(())}, (1,), torch.float32),
    ({"is_initialized": [0]}, (1,), torch.float32),
    ({}, (1,), torch.float32),
])  # fmt: skip
def test_placeholder_shape_comes_from_the_first_real_buffer(entry, shape, dtype):
    assert migrate._first_tensor_meta(entry) == (shape, dtype)


@pytest.mark.parametrize("group,want", [
    ({"params": [0], "foreach": True}, {"params": [0], "multi_tensor": True}),
    ({"params": [0], "foreach": False, "stochastic_schedule": True}, {"params": [0], "multi_tensor": False}),
    ({"params": [0], "multi_tensor": True, "lr": 0.1}, {"params": [0], "multi_tensor": True, "lr": 0.1}),
    ({"params": [], "stochastic_schedule": None}, {"params": []}),
])  # fmt: skip
def test_group_options_are_modernised(group, want):
    sd = {"state": {}, "param_groups": [dict(group)]}
    migrate._modernise_groups_and_meta(sd)
    assert sd["param_groups"][0] == want


@pytest.mark.parametrize("stale", [("precond_rng",), ("stochastic_schedule",), ("precond_rng", "stochastic_schedule")])
def test_stale_metadata_is_dropped_and_the_rest_kept(stale):
    meta = {"inner_group": {"stochastic_schedule": None, "keep": 1}, "use_ema": False, **{k: b"x" for k in stale}}
    sd = {"state": {}, "param_groups": [{"params": [], "foreach": True}], "heavyball": meta}
    migrate._modernise_groups_and_meta(sd)
    assert sd["heavyball"] == {"inner_group": {"keep": 1}, "use_ema": False}


def test_missing_metadata_block_is_tolerated():
    sd = {"state": {}, "param_groups": [{"params": [], "foreach": True}]}
    migrate._modernise_groups_and_meta(sd)
    assert "heavyball" not in sd and sd["param_groups"][0] == {"params": [], "multi_tensor": True}


# ---------------------------------------------------------------------------------------- locating the state


def test_state_is_found_under_single_and_nested_keys():
    sd = {"state": {}, "param_groups": []}
    assert migrate._locate({"optimizer": sd}, ["optimizer"]) is sd
    assert migrate._locate({"a": {"b": {"c": sd}}}, ["a", "b", "c"]) is sd


def test_missing_key_and_wrong_target_are_errors():
    with pytest.raises(KeyError, match="not found"):
        migrate._locate({"optimizer": {}}, ["trainer", "optimizer"])
    with pytest.raises(ValueError, match="not an optimizer state"):
        migrate._locate({"optimizer": {"weights": 1}}, ["optimizer"])
    with pytest.raises(ValueError, match="not an optimizer state"):
        migrate._locate({"optimizer": [1, 2]}, ["optimizer"])


# ---------------------------------------------------------------------------------------- entries


@pytest.mark.parametrize("n_views", [1, 2, 5])
def test_flat_entry_is_spread_over_its_views(n_views):
    key_map = [("update_by_adam_exp_avg", "update_by_adam_exp_avg_0", 0), ("update_by_adam_exp_avg_sq", "update_by_adam_exp_avg_sq_0", 0)]
    m = [torch.full((2,), float(i)) for i in range(n_views)]
    v = [torch.full((2,), 10.0 + i) for i in range(n_views)]
    entry = {"update_by_adam_exp_avg": m if n_views > 1 else m[0], "update_by_adam_exp_avg_sq": v if n_views > 1 else v[0]}
    out = migrate._migrate_entry(entry, key_map)
    assert sorted(out) == list(range(n_views))
    for i in range(n_views):
        assert torch.equal(out[i]["update_by_adam_exp_avg_0"], m[i]) and torch.equal(out[i]["update_by_adam_exp_avg_sq_0"], v[i])
        assert out[i]["is_initialized"] == [0]


def test_entry_without_known_keys_keeps_its_content():
    out = migrate._migrate_entry({"custom": torch.ones(2), "note": "x"}, [("a", "a_0", 0)])
    assert set(out[0]) == {"custom", "note"} and "is_initialized" not in out[0]
    assert migrate._migrate_entry({}, []) == {}


def test_entry_with_several_transforms_marks_each_index():
    key_map = [("exp_avg_exp_avg", "exp_avg_exp_avg_0", 0), ("scale_by_psgd_Q", "scale_by_psgd_Q_1", 1)]
    entry = {"exp_avg_exp_avg": torch.ones(3), "scale_by_psgd_Q": torch.eye(3), "is_initialized": [7]}
    out = migrate._migrate_entry(entry, key_map)
    assert out[0]["is_initialized"] == [0, 1, 7]
    assert torch.equal(out[0]["scale_by_psgd_Q_1"], torch.eye(3))


# ---------------------------------------------------------------------------------------- whole state dicts


def _v2_state(n_params=2, groups=1):
    state = {i: {0: {"update_by_adam_exp_avg_0": torch.full((2,), float(i)), "is_initialized": [0]}} for i in range(n_params)}
    per = max(1, n_params // groups)
    pgs = [{"params": list(range(g * per, n_params if g == groups - 1 else (g + 1) * per)), "foreach": True,
            "stochastic_schedule": False, "lr": 0.1 * (g + 1)} for g in range(groups)]  # fmt: skip
    return {"state": state, "param_groups": pgs, "heavyball": {"precond_rng": b"r", "inner_group": {"stochastic_schedule": None}}}


@pytest.mark.parametrize("n_params,groups", [(1, 1), (3, 1), (4, 2), (5, 3)])
def test_nested_former_layout_only_changes_options(n_params, groups):
    old = _v2_state(n_params, groups)
    out = migrate.migrate_state_dict(old, "heavyball.ForeachAdamW")
    assert migrate._detect_version(out) == 3
    assert [g["params"] for g in out["param_groups"]] == [g["params"] for g in old["param_groups"]]
    assert all("foreach" not in g and "stochastic_schedule" not in g and g["multi_tensor"] is True for g in out["param_groups"])
    assert [g["lr"] for g in out["param_groups"]] == [g["lr"] for g in old["param_groups"]]
    for i in range(n_params):
        assert torch.equal(out["state"][i][0]["update_by_adam_exp_avg_0"], torch.full((2,), float(i)))
    assert out["heavyball"] == {"inner_group": {}}


def test_migration_is_idempotent():
    once = migrate.migrate_state_dict(_v1_state(), "heavyball.ForeachAdamW")
    twice = migrate.migrate_state_dict(once, "heavyball.AdamW")
    assert twice["param_groups"] == once["param_groups"] and set(twice["state"]) == set(once["state"])
    for pid in once["state"]:
        for view in once["state"][pid]:
            for k, v in once["state"][pid][view].items():
                w = twice["state"][pid][view][k]
                assert torch.equal(v, w) if isinstance(v, torch.Tensor) else v == w


@pytest.mark.parametrize("shape", [(4,), (2, 3), (2, 3, 4)])
@pytest.mark.parametrize("n_params", [1, 3])
def test_flat_layout_of_any_shape_and_count(shape, n_params):
    state = {i: {"update_by_adam_exp_avg": torch.full(shape, 1.0 + i), "update_by_adam_exp_avg_sq": torch.full(shape, 2.0),
                 "is_initialized": [0]} for i in range(n_params)}  # fmt: skip
    old = {"state": state, "param_groups": [{"params": list(range(n_params)), "lr": 1e-3, "betas": [0.9, 0.99], "eps": 1e-8,
                                             "weight_decay": 0.0, "foreach": True, "warmup_steps": 0, "caution": False}]}  # fmt: skip
    out = migrate.migrate_state_dict(old, "ForeachAdamW")
    params = [torch.nn.Parameter(torch.zeros(shape)) for _ in range(n_params)]
    opt = hb.AdamW(params, lr=1e-3)
    opt.load_state_dict(out)
    for i, p in enumerate(params):
        assert torch.equal(opt.state[p][0]["update_by_adam_exp_avg_0"], torch.full(shape, 1.0 + i))
        p.grad = torch.ones_like(p)
    opt.step()
    assert all(torch.isfinite(p).all() for p in params)


# ---------------------------------------------------------------------------------------- command line


def test_cli_overwrites_the_input_when_no_output_is_given(tmp_path):
    path = tmp_path / "ckpt.pt"
    torch.save({"optimizer": _v1_state()}, path)
    assert migrate.main([str(path), "heavyball.ForeachAdamW"]) == 0
    assert migrate._detect_version(torch.load(path, weights_only=False)["optimizer"]) == 3


def test_cli_dry_run_leaves_the_file_alone(tmp_path):
    path = tmp_path / "ckpt.pt"
    torch.save({"optimizer": _v1_state()}, path)
    before = path.read_bytes()
    assert migrate.main([str(path), "heavyball.ForeachAdamW", "--dry-run"]) == 0
    assert path.read_bytes() == before


@pytest.mark.parametrize("key", ["optimizer", "model.optimizer", "a.b.c"])
def test_cli_state_key_paths(tmp_path, key):
    root = node = {}
    parts = key.split(".")
    for part in parts[:-1]:
        node = node.setdefault(part, {})
    node[parts[-1]] = _v1_state()
    root["other"] = {"epoch": 3}
    path, out = tmp_path / "ckpt.pt", tmp_path / "out.pt"
    torch.save(root, path)
    assert migrate.main([str(path), "heavyball.ForeachAdamW", "--state-key", key, "-o", str(out)]) == 0
    loaded = torch.load(out, weights_only=False)
    assert loaded["other"] == {"epoch": 3}
    for part in parts:
        loaded = loaded[part]
    assert migrate._detect_version(loaded) == 3


def test_cli_current_layout_is_left_as_it_is(tmp_path):
    params = [torch.nn.Parameter(torch.randn(3, 2))]
    opt = hb.AdamW(params, lr=1e-3)
    params[0].grad = torch.ones_like(params[0])
    opt.step()
    path, out = tmp_path / "ckpt.pt", tmp_path / "out.pt"
    torch.save({"optimizer": opt.state_dict()}, path)
    assert migrate.main([str(path), "heavyball.AdamW", "-o", str(out)]) == 0
    a, b = torch.load(path, weights_only=False)["optimizer"], torch.load(out, weights_only=False)["optimizer"]
    assert a["param_groups"] == b["param_groups"] and set(a["state"]) == set(b["state"])
