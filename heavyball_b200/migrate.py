"""Checkpoint migration: bring optimizer state dicts written by HeavyBall 1.x / 2.x to the current layout.

    python -m heavyball_b200.migrate CHECKPOINT OPTIMIZER_CLASS [--state-key optimizer] [-o OUT] [--dry-run]

Layouts (parity: ``scripts/migrate_optimizer_state.py:101-313`` of the reference):

* **1.x** - ``state[param]`` is flat: ``{"<fn>_<slot>": tensor | [tensor per view], ...}``.  It becomes
  ``state[param][view][f"{fn}_{slot}_{transform_idx}"]`` with the indices of the current class's chain,
  plus an ``is_initialized`` list per view.
* **2.x** - already nested per view, but param groups say ``foreach``; renamed to ``multi_tensor`` and
  stale keys (``stochastic_schedule``, ``precond_rng``) are dropped.
* **3.x** - ``multi_tensor`` present: returned unchanged.

Old class names (``ForeachAdamW``, ``PaLMForeachSOAP``, ``CachedDelayedPSGDKron`` ...) resolve to the class
that replaced them.  Uses only ``argparse`` (no CLI framework dependency).
"""

from __future__ import annotations

import argparse
import importlib
import sys
from typing import Any, Dict, List, Sequence, Tuple

import torch

# current class -> names it was known under in earlier releases
_FORMER_NAMES = {
    "AdamW": ["ForeachAdamW"],
    "NAdam": ["ForeachNAdam"],
    "AdEMAMix": ["ForeachAdEMAMix"],
    "AdamC": ["ForeachAdamC"],
    "RMSprop": ["ForeachRMSprop"],
    "SFAdamW": ["ForeachSFAdamW", "PaLMForeachSFAdamW", "PaLMSFAdamW"],
    "ADOPT": ["ForeachADOPT"],
    "Muon": ["ForeachMuon"],
    "LaProp": ["ForeachLaProp"],
    "SOAP": [
        "ForeachSOAP", "PaLMForeachSOAP", "PrecondScheduleForeachSOAP", "PrecondSchedulePaLMForeachSOAP", "PaLMSOAP",
        "PalmForEachSoap", "PrecondScheduleSOAP", "PrecondSchedulePaLMSOAP",
    ],
    "SOAPNAdam": ["ForeachSOAPNAdam"],
    "SOAPAdEMAMix": ["ForeachSOAPAdEMAMix"],
    "SignLaProp": ["ForeachSignLaProp"],
    "SOLP": ["ForeachSOLP"],
    "PSGDKron": [
        "ForeachPSGDKron", "ForeachPurePSGD", "ForeachCachedPSGDKron", "ForeachCachedDelayedPSGDKron",
        "ForeachDelayedPSGD", "ForeachCachedNewtonPSGD", "NewtonHybrid2PSGDKron", "PurePSGD", "DelayedPSGD",
        "CachedPSGDKron", "CachedDelayedPSGDKron", "NewtonPSGDKron",
    ],
    "PSGDLRA": [
        "ForeachPSGDLRA", "ForeachDelayedPSGDLRA", "ForeachNewtonPSGDLRA", "NewtonHybrid2PSGDLRA", "DelayedPSGDLRA",
        "NewtonPSGDLRA",
    ],
}  # fmt: skip
_CLASS_RENAMES = {old: new for new, olds in _FORMER_NAMES.items() for old in olds}
_REMOVED_GROUP_KEYS = frozenset({"stochastic_schedule"})
_REMOVED_META_KEYS = frozenset({"stochastic_schedule", "precond_rng"})
_PACKAGE_ALIASES = {"heavyball": "heavyball_b200"}


def _resolve_class_name(name: str) -> str:
    return _CLASS_RENAMES.get(name, name)


def _load_optimizer_class(qualified: str):
    module_name, _, cls_name = qualified.rpartition(".")
    module_name = _PACKAGE_ALIASES.get(module_name or "heavyball", module_name or "heavyball")
    cls_name = _resolve_class_name(cls_name)
    module = importlib.import_module(module_name)
    if not hasattr(module, cls_name):
        raise ValueError(f"Optimizer class '{module_name}.{cls_name}' not found")
    return getattr(module, cls_name)


def _detect_version(sd: Dict[str, Any]) -> int:
    nested = None
    for entry in sd.get("state", {}).values():
        if isinstance(entry, dict):
            nested = any(isinstance(v, dict) for v in entry.values())
            break
    modern_groups = any(isinstance(g, dict) and "multi_tensor" in g for g in sd.get("param_groups", []))
    if nested is False:
        return 1
    if nested:
        return 3 if modern_groups else 2
    return 3 if modern_groups else 1


def _first_tensor_meta(entry: Dict[str, Any]) -> Tuple[Tuple[int, ...], torch.dtype]:
    """Shape and dtype for a placeholder parameter: taken from the first floating-point buffer of the saved state
    (step counters and other integer entries say nothing about the parameter)."""
    fallback = None
    for v in entry.values():
        t = v if isinstance(v, torch.Tensor) else (v[0] if isinstance(v, (list, tuple)) and v and isinstance(v[0], torch.Tensor) else None)
        if t is None:
            continue
        if t.is_floating_point() and t.ndim > 0:
            return tuple(t.shape), t.dtype
        if fallback is None and t.is_floating_point():
            fallback = ((1,), t.dtype)
    return fallback or ((1,), torch.float32)


def _instantiate(opt_cls, sd: Dict[str, Any]):
    """Builds the current optimizer class over placeholder parameters shaped like the saved state, so that
    its chain (and therefore its transform indices) can be inspected."""
    groups = sd["param_groups"]
    if not groups:
        raise ValueError("No parameter groups found in optimizer state")
    n = max(pid for g in groups for pid in g.get("params", [-1])) + 1
    params = []
    for pid in range(n):
        shape, dtype = _first_tensor_meta(sd["state"].get(pid, {}))
        params.append(torch.nn.Parameter(torch.zeros(shape, dtype=dtype)))
    built = []
    for g in groups:
        opts = {}
        for k, v in g.items():
            if k == "params" or k in _REMOVED_GROUP_KEYS:
                continue
            k = "multi_tensor" if k == "foreach" else k
            opts[k] = tuple(v) if isinstance(v, list) and k in ("betas", "weight_decay_steps") else v
        built.append({"params": [params[pid] for pid in g.get("params", [])], **opts})
    return opt_cls(built)


def _key_map(optimizer) -> List[Tuple[str, str, int]]:
    """(old flat key, new indexed key, transform index) for every state slot of the optimizer's chain."""
    from . import chainable as C

    out, seen = [], set()
    for tr in C._walk_fns(getattr(optimizer, "_fns", [])):
        for layer in tr.layers:
            for slot, new_key in layer.keys.items():
                item = (f"{tr.fn_name}_{slot}", new_key, layer.index)
                if item not in seen:
                    seen.add(item)
                    out.append(item)
    return out


def _as_set(v) -> set:
    if isinstance(v, set):
        return v
    if isinstance(v, (list, tuple)):
        return set(v)
    return set() if v is None else {v}


def _migrate_entry(entry: Dict[str, Any], key_map) -> Dict[int, Dict[str, Any]]:
    views: Dict[int, Dict[str, Any]] = {}
    done: Dict[int, set] = {}

    def put(key, value, idx):
        per_view = value if (isinstance(value, (list, tuple)) and value and all(isinstance(t, torch.Tensor) for t in value)) else [value]
        for view, item in enumerate(per_view):
            views.setdefault(view, {})[key] = item
            if idx is not None:
                done.setdefault(view, set()).add(idx)

    rest = dict(entry)
    for old, new, idx in key_map:
        if old in rest:
            put(new, rest.pop(old), idx)
    for key, value in rest.items():
        if key == "is_initialized":
            done.setdefault(0, set()).update(_as_set(value))
        else:
            put(key, value, None)
    for view, bucket in views.items():
        if done.get(view):
            bucket["is_initialized"] = sorted(done[view])
    return views


def _modernise_groups_and_meta(sd: Dict[str, Any]) -> None:
    for g in sd.get("param_groups", []):
        if isinstance(g, dict):
            if "foreach" in g:
                g["multi_tensor"] = g.pop("foreach")
            for k in _REMOVED_GROUP_KEYS:
                g.pop(k, None)
    meta = sd.get("heavyball", {})
    for k in _REMOVED_META_KEYS:
        meta.pop(k, None)
        meta.get("inner_group", {}).pop(k, None)


def migrate_state_dict(old: Dict[str, Any], optimizer_class: str) -> Dict[str, Any]:
    version = _detect_version(old)
    if version == 3:
        return dict(old)
    if version == 2:
        out = dict(old)
    else:
        optimizer = _instantiate(_load_optimizer_class(optimizer_class), old)
        out = dict(optimizer.state_dict())
        key_map = _key_map(optimizer)
        out["param_groups"] = old["param_groups"]
        out["state"] = {pid: {int(v): dict(b) for v, b in _migrate_entry(e, key_map).items()} for pid, e in old["state"].items()}
        out.setdefault("heavyball", {}).setdefault("inner_group", {})
    _modernise_groups_and_meta(out)
    return out


def _locate(root: Dict[str, Any], path: Sequence[str]) -> Dict[str, Any]:
    node = root
    for key in path:
        if key not in node:
            raise KeyError(f"Key '{'.'.join(path)}' not found in checkpoint")
        node = node[key]
    if not isinstance(node, dict) or "state" not in node or "param_groups" not in node:
        raise ValueError(f"Target at '{'.'.join(path)}' is not an optimizer state dict")
    return node


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="heavyball_b200.migrate", description=__doc__.split("\n\n")[0])
    ap.add_argument("checkpoint", help="checkpoint file (.pt / .pth) containing the optimizer state")
    ap.add_argument("optimizer_class", help="e.g. heavyball.AdamW; former names such as ForeachAdamW are resolved")
    ap.add_argument("--state-key", default="optimizer", help="dot-separated path to the optimizer state inside the file")
    ap.add_argument("--output", "-o", default=None, help="where to write (default: overwrite the input)")
    ap.add_argument("--dry-run", action="store_true", help="migrate in memory only")
    args = ap.parse_args(argv)

    data = torch.load(args.checkpoint, map_location="cpu", weights_only=False)
    target = _locate(data, [k for k in args.state_key.split(".") if k])
    migrated = migrate_state_dict(target, args.optimizer_class)
    target.clear()
    target.update(migrated)
    if args.dry_run:
        print("Dry run complete; no file written.")
        return 0
    out = args.output or args.checkpoint
    torch.save(data, out)
    print(f"Migrated checkpoint written to {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
