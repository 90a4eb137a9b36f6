"""Chainable transform engine.

An optimizer is a sequence of *transforms* ``fn(state, group, update, grad, param) -> update``.  A
transform is a plain function wrapped in a stack of *guard layers* (allocate zero state, snapshot the
parameter, run an initialiser, squeeze size-1 dims, bucket same-shape tensors, ...).  Here a transform
is one :class:`FunctionTransform` object holding a flat list of layers; decorators prepend layers
instead of nesting wrapper objects.  Every layer owns one *transform index*; state lives in
``optimizer.state[param][view]`` under ``f"{fn_name}_{slot}_{index}"``.

Checkpoint compatibility with the reference depends on reproducing its index numbering
(``heavyball/chainable.py:2347-2382``): siblings are numbered last-to-first, a transform's layers
outermost-first, ``Route`` / ``Parallel`` children as one flattened sibling list.
:func:`set_indices` implements exactly that order.

Behavioural parity targets: guards ``heavyball/chainable.py:37-640``; transform library
``heavyball/chainable.py:642-1940``; ``chain`` ``heavyball/chainable.py:2278-2323``; ``ChainOpt`` /
``BaseOpt`` / mode switches ``heavyball/chainable.py:2385-2748``.  The sharded-parameter
repartitioning those classes call lives in ``heavyball_b200.parallel.fsdp``.

On CUDA, ``ChainOpt`` first offers each step to ``heavyball_b200.lowering``: chains made of known
transforms execute as a few multi-tensor sm_100a kernel launches per group; anything else (CPU,
user-defined transforms, exotic dtypes) runs through the PyTorch definitions in this file.
"""

from __future__ import annotations

import contextlib
import copy
import functools
import math
import warnings
from collections.abc import Iterable as _Iterable
from typing import Iterable, List, Literal, Optional, Union

import torch
from torch import Tensor

from . import utils

use_default = utils.use_default
_SKIP = object()


# ======================================================================================== state helpers


def _key_in_state(state, key):
    if isinstance(key, str):
        return key in state
    return all(isinstance(k, (tuple, list)) or k in state for k in key)


def _guard_in_state(state, key, template_fn):
    if not _key_in_state(state, key):
        state[key] = template_fn()
    return state[key]


def _storage_dtype(group):
    return getattr(torch, group.get("storage_dtype", "float32"))


def _zero_guard(state, key, ref, dtype):
    return _guard_in_state(state, key, lambda: torch.zeros_like(ref, dtype=dtype, memory_format=torch.preserve_format))


def _states_of(state, param):
    return state if isinstance(state, list) else [state(p) for p in param]


def _mark(st, idx):
    done = st.get("is_initialized")
    if not isinstance(done, set):  # absent, or a list written by an older checkpoint
        done = st["is_initialized"] = set(done or ())
    done.add(idx)


class ECCConfig:
    """``"bf16+8" | "bf16+16" | "fp16+8" | "fp16+16"``: 16-bit primary plus integer correction."""

    __slots__ = ("primary_dtype", "corr_dtype")
    _MODES = {
        "bf16+8": (torch.bfloat16, torch.int8),
        "bf16+16": (torch.bfloat16, torch.int16),
        "fp16+8": (torch.float16, torch.int8),
        "fp16+16": (torch.float16, torch.int16),
    }

    def __init__(self, mode):
        self.primary_dtype, self.corr_dtype = self._MODES[mode]

    @property
    def smax(self):
        return utils._ULPState._SMAX[self.corr_dtype]

    def init_correction(self, correction, fp32, narrow):
        utils._ULPState(correction, self.smax).compute_correction(fp32, narrow)

    @classmethod
    def from_group(cls, group, key="ecc"):
        mode = group.get(key)
        return cls(mode) if mode else None

    def init_state(self, state, key, ref):
        _zero_guard(state, key, ref, self.primary_dtype)
        _zero_guard(state, key + "::ecc", ref, self.corr_dtype)

    @contextlib.contextmanager
    def attached(self, tensors, corrections):
        smax = self.smax
        for t, c in zip(tensors, corrections):
            t._ecc = utils._ULPState(c, smax)
        try:
            yield
        finally:
            for t in tensors:
                t.__dict__.pop("_ecc", None)


# ======================================================================================== guard layers


class Layer:
    """One guard level.  ``slots`` are the state names it owns; ``index`` is its transform index."""

    slots: tuple = ()
    needs_init = True
    terminal = False

    def __init__(self):
        self.index = None
        self.keys = {}

    def bind(self, fn_name, index):
        self.index = index
        self.keys = {n: f"{fn_name}_{n}_{index}" for n in self.slots}

    def key(self, name):
        return self.keys[name]

    # -- default protocol: lazily initialise per-parameter state, then hand the slot lists inward
    def init(self, st, group, update, grad, param, *args, **kwargs):
        return None

    def forward(self, tr, depth, state, group, update, grad, param, slot_lists, *args, **kwargs):
        return tr._invoke(depth + 1, state, group, update, grad, param, *args, *slot_lists, **kwargs)

    def run(self, tr, depth, state, group, update, grad, param, *args, **kwargs):
        states = _states_of(state, param)
        skip = False
        for st, per in zip(states, zip(update, grad, param, *args)):
            if self.index not in st.get("is_initialized", ()):
                if self.init(st, group, *per, **kwargs) is _SKIP:
                    skip = True
                _mark(st, self.index)
        if skip:
            return _SKIP
        slot_lists = [[st.get(self.keys[n]) for st in states] for n in self.slots]
        return self.forward(tr, depth, state, group, update, grad, param, slot_lists, *args, **kwargs)


class ZeroSlots(Layer):
    """Zero-initialised buffers shaped like the parameter (``storage_dtype``, or an ECC pair)."""

    def __init__(self, names):
        super().__init__()
        self.slots = tuple(names)

    def init(self, st, group, update, grad, param, *args, **kwargs):
        ecc = ECCConfig.from_group(group)
        for n in self.slots:
            if ecc is None:
                _zero_guard(st, self.keys[n], param, _storage_dtype(group))
            else:
                ecc.init_state(st, self.keys[n], param)

    def _slab_init(self, states, group, param):
        """When several parameters are initialised in one call, each slot's buffers are carved out
        of one zeroed slab (16-byte aligned segments) instead of being allocated one by one, so a
        group's state is contiguous in memory for the multi-tensor kernels."""
        todo = [
            (st, p) for st, p in zip(states, param)
            if self.index not in st.get("is_initialized", ()) and p.is_contiguous()
        ]  # fmt: skip
        if len(todo) < 2 or len({(p.device, p.dtype) for _, p in todo}) != 1:
            return
        ecc = ECCConfig.from_group(group)
        kinds = [("", _storage_dtype(group))] if ecc is None else [("", ecc.primary_dtype), ("::ecc", ecc.corr_dtype)]
        sizes = [(p.numel() + 15) // 16 * 16 for _, p in todo]
        dev = todo[0][1].device
        for n in self.slots:
            for suffix, dtype in kinds:
                key = self.keys[n] + suffix
                if any(key in st for st, _ in todo):
                    continue
                slab = torch.zeros(sum(sizes), dtype=dtype, device=dev)
                off = 0
                for (st, p), size in zip(todo, sizes):
                    st[key] = slab[off : off + p.numel()].view(p.shape)
                    off += size

    def run(self, tr, depth, state, group, update, grad, param, *args, **kwargs):
        if len(param) > 1 and group.get("slab_state", True):
            self._slab_init(_states_of(state, param), group, param)
        return super().run(tr, depth, state, group, update, grad, param, *args, **kwargs)

    def forward(self, tr, depth, state, group, update, grad, param, slot_lists, *args, **kwargs):
        ecc = ECCConfig.from_group(group)
        if ecc is None:
            return tr._invoke(depth + 1, state, group, update, grad, param, *args, *slot_lists, **kwargs)
        states = _states_of(state, param)
        with contextlib.ExitStack() as stack:
            for n, prim in zip(self.slots, slot_lists):
                stack.enter_context(ecc.attached(prim, [st[self.keys[n] + "::ecc"] for st in states]))
            return tr._invoke(depth + 1, state, group, update, grad, param, *args, *slot_lists, **kwargs)


class CopySlots(Layer):
    """Buffers initialised as a clone of one of the call arguments (2 = the parameter)."""

    def __init__(self, index, names):
        super().__init__()
        self.source = index
        self.slots = tuple(names)

    def init(self, st, group, update, grad, param, *args, **kwargs):
        src = [update, grad, param, *args][self.source]
        for n in self.slots:
            st[self.keys[n]] = torch.clone(src)


class InitSlots(Layer):
    """State produced by a user initialiser that writes plain names into the state dict; they are
    renamed to indexed keys.  With ``skip_first`` the initialising step makes no update."""

    def __init__(self, names, init_fn, skip_first=True):
        super().__init__()
        self.slots = tuple(names)
        self.init_fn = init_fn
        self.skip_first = skip_first

    def init(self, st, group, update, grad, param, *args, **kwargs):
        self.init_fn(st, group, update, grad, param, **kwargs)
        for n in self.slots:
            st[self.keys[n]] = st.pop(n, None)
        return _SKIP if self.skip_first else None


class AccumSlots(Layer):
    """Optional accumulation of the preconditioner input between preconditioner updates
    (``precond_grad_accum``); hands the tensor to fit on to the inner function."""

    slots = ("precond_grad_accum",)

    def bind(self, fn_name, index):
        super().bind(fn_name, index)
        self.counter = f"_{fn_name}_steps_taken_{index}"

    def init(self, st, group, update, grad, param, *args, **kwargs):
        if group.get("precond_grad_accum", False):
            _zero_guard(st, self.keys["precond_grad_accum"], param, _storage_dtype(group))

    def forward(self, tr, depth, state, group, update, grad, param, slot_lists, *args, **kwargs):
        base = update if group.get("momentum_into_precond_update", True) else grad
        nxt = functools.partial(tr._invoke, depth + 1, state, group, update, grad, param, *args)
        if not group.get("precond_grad_accum", False):
            return nxt(base, **kwargs)
        (acc,) = slot_lists
        taken = group.get(self.counter, 0)
        if not group["is_preconditioning"]:
            group[self.counter] = taken + 1
            utils.stochastic_add_(acc, base)
            return nxt(base, **kwargs)
        if not taken:
            return nxt(base, **kwargs)
        group[self.counter] = taken + 1
        utils.stochastic_add_(acc, base)
        utils.stochastic_multiply_(acc, 1 / group[self.counter])
        out = nxt(acc, **kwargs)
        if group.get(self.counter, 0) != 0:
            group[self.counter] = 0
            utils.zero_(acc)
        return out


class Warmup(Layer):
    """Runs ``warmup_fns[k]`` instead of the transform on its k-th call (no update those steps)."""

    def __init__(self, warmup_fns):
        super().__init__()
        self.warmup_fns = list(warmup_fns)

    def bind(self, fn_name, index):
        super().bind(fn_name, index)
        self.counter = f"_warmup_{index}"

    def run(self, tr, depth, state, group, update, grad, param, *args, **kwargs):
        states = _states_of(state, param)
        done = min(st.get(self.counter, 0) for st in states)
        if done < len(self.warmup_fns):
            fn = self.warmup_fns[done]
            for st, per in zip(states, zip(update, grad, param, *args)):
                fn(st, group, *per, **kwargs)
                st[self.counter] = st.get(self.counter, 0) + 1
            return _SKIP
        for st in states:
            _mark(st, self.index)
        return tr._invoke(depth + 1, state, group, update, grad, param, *args, **kwargs)


class Tag(Layer):
    """Attaches attributes (``needs_full_param=True``) to the transform; otherwise transparent."""

    def __init__(self, **tags):
        super().__init__()
        self.tags = tags


def _view_like(src, target):
    v = src.view_as(target)
    ecc = getattr(src, "_ecc", None)
    if ecc is not None:
        v._ecc = ecc
    return v


def _squeeze_inner(u: Tensor) -> Tensor:
    ones = tuple(i for i in range(1, u.ndim) if u.shape[i] == 1)
    return u.squeeze(ones) if ones else u


class Squeeze(Layer):
    """Drops size-1 dims (except the leading slot dim) for the inner function, restores on return."""

    needs_init = False

    def run(self, tr, depth, state, group, update, grad, param, *args, **kwargs):
        shapes = [u.shape for u in update]
        update = [_squeeze_inner(u) for u in update]
        relist = lambda xs: [_view_like(x, u) for x, u in zip(xs, update)]  # noqa: E731
        is_tensor_list = lambda a: isinstance(a, (list, tuple)) and len(a) and isinstance(a[0], Tensor)  # noqa: E731
        args = [relist(a) if is_tensor_list(a) else a for a in args]
        kwargs = {k: relist(a) if is_tensor_list(a) else a for k, a in kwargs.items()}
        out = tr._invoke(depth + 1, state, group, update, relist(grad), relist(param), *args, **kwargs)
        if out is _SKIP or out is None:
            return out
        return [o.view(s) for o, s in zip(out, shapes)]


def _stack_value(vals):
    """Combine per-member state values into one batched value: tensors with a leading slot dim are
    concatenated on it, 0-d tensors shared, lists / tuples recursed, sets united."""
    first = next((v for v in vals if v is not None), None)
    if first is None:
        return None
    if isinstance(first, Tensor):
        if first.ndim == 0:
            return first.clone()
        return torch.cat([v if isinstance(v, Tensor) else torch.zeros_like(first) for v in vals], 0)
    if isinstance(first, tuple):
        return tuple(_stack_value([v[i] if isinstance(v, tuple) else None for v in vals]) for i in range(len(first)))
    if isinstance(first, list):
        return [
            _stack_value([v[i] if isinstance(v, list) and i < len(v) else None for v in vals]) for i in range(len(first))
        ]
    if isinstance(first, set):
        return set().union(*[v for v in vals if isinstance(v, set)])
    return first


def _unstack_value(val, i, n):
    if isinstance(val, Tensor):
        if val.ndim >= 1 and val.shape[0] == n:
            return val[i : i + 1].clone()
        return val.clone()
    if isinstance(val, tuple):
        return tuple(_unstack_value(v, i, n) for v in val)
    if isinstance(val, list):
        return [_unstack_value(v, i, n) for v in val]
    if isinstance(val, set):
        return val.copy()
    return val


class Bucket(Layer):
    """Runs the inner layers once per group of same-(shape, dtype, device, owner) tensors, with
    parameters, gradients, updates and state batched along a new leading slot dimension.  Per-member
    state keeps a leading dim of 1, which is also the checkpoint layout."""

    needs_init = False

    def inner_keys(self, tr, depth):
        keys = set()
        for layer in tr.layers[depth + 1 :]:
            keys.update(layer.keys.values())
        return keys | {k + "::ecc" for k in keys}

    def run(self, tr, depth, state, group, update, grad, param, *args, **kwargs):
        states = _states_of(state, param)
        shapes = group.get("_orig_shapes") or {}
        keys = self.inner_keys(tr, depth)

        buckets = {}
        for i, p in enumerate(param):
            info = shapes.get(id(p))
            sig = (tuple(p.shape), p.dtype, p.device, info.owner if info is not None else None)
            buckets.setdefault(sig, []).append(i)

        out = [None] * len(param)
        skipped = False
        for members in buckets.values():
            fresh = [i for i in members if keys.isdisjoint(states[i])]
            ready = [i for i in members if not keys.isdisjoint(states[i])]
            for sub in (fresh, ready):
                if not sub:
                    continue
                n = len(sub)
                sts = [states[i] for i in sub]
                batch = lambda xs: xs[0][None] if n == 1 else torch.stack(xs, 0)  # noqa: E731
                ps = [param[i] for i in sub]
                slab_p = batch(ps)
                eccs = [getattr(p, "_ecc", None) for p in ps]
                if eccs[0] is not None:
                    slab_p._ecc = utils._ULPState(batch([e.correction for e in eccs]), eccs[0].smax)
                slab_state = {k: v for k in keys if (v := _stack_value([m.get(k) for m in sts])) is not None}
                slab_state["is_initialized"] = set().union(*[m.get("is_initialized") or () for m in sts])

                res = tr._invoke(
                    depth + 1, [slab_state], group, [batch([update[i] for i in sub])], [batch([grad[i] for i in sub])],
                    [slab_p], *args, **kwargs,
                )  # fmt: skip

                for j, m in enumerate(sts):
                    for k, v in slab_state.items():
                        m[k] = _unstack_value(v, j, n)
                if res is _SKIP:
                    skipped = True
                    if n > 1:  # a one-member slab aliases the parameter; larger slabs are copies
                        for j, p in enumerate(ps):
                            p.copy_(slab_p[j])
                        if eccs[0] is not None:
                            for j, e in enumerate(eccs):
                                e.correction.copy_(slab_p._ecc.correction[j])
                    continue
                for j, i in enumerate(sub):
                    out[i] = res[0][j]
        return _SKIP if skipped else out


class Stateless(Layer):
    """Terminal layer: the function takes ``(group, update, grad, param, *state_lists)``."""

    needs_init = False
    terminal = True

    def run(self, tr, depth, state, group, update, grad, param, *args, **kwargs):
        return tr.fn(group, update, grad, param, *args, **kwargs)


class PerTensor(Layer):
    """Terminal layer: the function takes single tensors and is called once per parameter."""

    terminal = True

    def run(self, tr, depth, state, group, update, grad, param, *args, **kwargs):
        for st in _states_of(state, param):
            _mark(st, self.index)
        outs, skipped = [], False
        for per in zip(update, grad, param, *args):
            r = tr.fn(group, *per, **kwargs)
            if r is _SKIP:
                skipped = True
            else:
                outs.append(r)
        return _SKIP if skipped else outs


# ======================================================================================== transform object


class FunctionTransform:
    """A function plus its guard layers (outermost first)."""

    def __init__(self, fn, layers=(), names=None):
        self.fn = fn
        self.layers = list(layers)
        self.fn_name = getattr(fn, "__name__", repr(fn))
        self.__name__ = self.fn_name
        self._under_bucket = False

    # ---- composition
    def wrapped(self, layer):
        return FunctionTransform(self.fn, [layer, *copy.deepcopy(self.layers)])

    def get_fn(self):
        return self.fn

    # ---- attributes contributed by Tag layers
    def __getattr__(self, item):
        if item.startswith("__") or item in ("fn", "layers"):
            raise AttributeError(item)
        for layer in self.__dict__.get("layers", ()):
            if isinstance(layer, Tag) and item in layer.tags:
                return layer.tags[item]
        raise AttributeError(item)

    # ---- indices and keys
    @property
    def transform_idx(self):
        return self.layers[0].index if self.layers else None

    @property
    def names(self):
        return [n for layer in self.layers for n in layer.slots]

    @property
    def _val_names(self):
        return {n: k for layer in self.layers for n, k in layer.keys.items()}

    def val_name(self, name):
        return self._val_names[name]

    def assign(self, start, retain):
        """Gives every unnumbered layer the next free index; returns the next free index."""
        self.__dict__.pop("_mark_indices", None)  # derived from the layer indices by the kernel lowering
        seen_bucket = False
        for layer in self.layers:
            if not retain or layer.index is None:
                layer.bind(self.fn_name, start)
                start += 1
            layer.under_bucket = seen_bucket
            seen_bucket = seen_bucket or isinstance(layer, Bucket)
        return start

    # ---- execution
    def _invoke(self, depth, state, group, update, grad, param, *args, **kwargs):
        if depth == len(self.layers):
            return self.fn(state, group, update, grad, param, *args, **kwargs)
        return self.layers[depth].run(self, depth, state, group, update, grad, param, *args, **kwargs)

    def __call__(self, state, group, update, grad, param, *args, **kwargs):
        return self._invoke(0, state, group, update, grad, param, *args, **kwargs)

    def __repr__(self):
        inner = ", ".join(type(layer).__name__ for layer in self.layers)
        return f"FunctionTransform({self.fn_name}: [{inner}], transform_idx={self.transform_idx})"


def _as_transform(fn):
    return fn if isinstance(fn, FunctionTransform) else FunctionTransform(fn)


def _layer_decorator(make_layer):
    def deco(fn):
        return _as_transform(fn).wrapped(make_layer())

    return deco


def zero_guard(*names):
    return _layer_decorator(lambda: ZeroSlots(names))


def copy_guard(index, *names):
    return _layer_decorator(lambda: CopySlots(index, names))


def general_guard(*names, init_fn, skip_first: bool = True):
    return _layer_decorator(lambda: InitSlots(names, init_fn, skip_first))


def warmup_guard(*warmup_fns):
    return _layer_decorator(lambda: Warmup(warmup_fns))


def no_state(fn):
    return _as_transform(fn).wrapped(Stateless())


def no_state_no_multi_tensor(fn):
    return _as_transform(fn).wrapped(PerTensor())


def needs_full_param(fn):
    return _as_transform(fn).wrapped(Tag(needs_full_param=True))


def bucket_aware(fn):
    return _as_transform(fn).wrapped(Bucket())


def SqueezeGrad(fn):
    return _as_transform(fn).wrapped(Squeeze())


def PrecondGradAccumGuard(fn):
    return _as_transform(fn).wrapped(AccumSlots())


def TagGuard(fn, **tags):
    return _as_transform(fn).wrapped(Tag(**tags))


# class-style aliases kept for code that constructs guards directly
def ZeroGuard(fn, names):
    return zero_guard(*names)(fn)


def CopyGuard(fn, index, names):
    return copy_guard(index, *names)(fn)


def GeneralGuard(fn, names, init_fn, skip_first: bool = True):
    return general_guard(*names, init_fn=init_fn, skip_first=skip_first)(fn)


def WarmupGuard(fn, warmup_fns):
    return warmup_guard(*warmup_fns)(fn)


NoState = no_state
NoStateNoMultiTensor = no_state_no_multi_tensor
BucketGuard = bucket_aware


# ======================================================================================== combinators


def _enforce_uniform_skip(flags):
    flags = list(flags)
    if not flags or not any(flags):
        return False
    if all(flags):
        return True
    raise ValueError("All branches must uniformly skip or not skip updates")


def _normalize_chain(fns):
    if fns is None:
        return None
    return fns if isinstance(fns, (list, tuple)) else (fns,)


def _inner_chain(state, group, update, grad, param, *fns):
    skip = False
    for fn in fns:
        new = fn(state, group, update, grad, param)
        if new is _SKIP:
            skip = True
        elif new is None:
            return None, skip
        else:
            update = new
    return update, skip


class Parallel:
    """Runs several sub-chains on clones of the update and merges their results."""

    def __init__(self, branches: List[List[callable]], merge_fn: callable):
        self.branches = branches
        self.merge_fn = merge_fn

    def __call__(self, state, group, update, grad, param):
        outs, skips = [], []
        for branch in self.branches:
            fresh = [torch.clone(u, memory_format=torch.preserve_format) for u in update]
            u, skip = _inner_chain(state, group, fresh, grad, param, *branch)
            outs.append(u)
            skips.append(skip)
        if _enforce_uniform_skip(skips):
            return _SKIP
        return self.merge_fn(outs)


class Route:
    """Sends each parameter through the first sub-chain whose predicate accepts it (``default``
    otherwise; ``None`` = pass-through).  All used routes must agree on skipping the final update."""

    def __init__(self, *routes, default=None):
        self.routes = [(pred, _normalize_chain(fns)) for pred, fns in routes]
        self.default = _normalize_chain(default)

    def __call__(self, state, group, update, grad, param):
        states = _states_of(state, param)
        taken, plan = set(), []
        for pred, fns in self.routes:
            idx = [i for i, p in enumerate(param) if i not in taken and pred(p)]
            taken.update(idx)
            plan.append((idx, fns))
        rest = [i for i in range(len(param)) if i not in taken]
        if rest:
            plan.append((rest, self.default))

        pick = lambda xs, idx: [xs[i] for i in idx]  # noqa: E731
        out, skips = [None] * len(param), []
        for idx, fns in plan:
            if not idx:
                continue
            if fns is None:
                u, skip = pick(update, idx), False
            else:
                u, skip = _inner_chain(pick(states, idx), group, pick(update, idx), pick(grad, idx), pick(param, idx), *fns)
            skips.append(skip)
            if u is not None:
                for i, ui in zip(idx, u):
                    out[i] = ui
        return _SKIP if _enforce_uniform_skip(skips) else out


def route(*routes, default=None):
    return Route(*routes, default=default)


# ======================================================================================== index assignment


def _children(obj):
    """Direct sub-nodes in the reference's visiting order (siblings are later visited in reverse)."""
    if isinstance(obj, functools.partial):
        return [obj.func]
    if isinstance(obj, Parallel):
        return [f for branch in obj.branches for f in branch]
    if isinstance(obj, Route):
        kids = [f for _, fns in obj.routes for f in fns]
        return kids + list(obj.default or ())
    if isinstance(obj, _Iterable) and not isinstance(obj, (str, bytes, bytearray)):
        return list(obj)
    return []


def _walk_fns(obj):
    """Yields every :class:`FunctionTransform` below ``obj`` in numbering order."""
    if isinstance(obj, FunctionTransform):
        yield obj
        return
    for child in reversed(_children(obj)):
        yield from _walk_fns(child)


def set_indices(fns: Iterable[callable], retain: bool = True, offset: int = 0):
    if retain and offset:
        raise ValueError("offset cannot be retained")
    if retain:
        used = [layer.index for tr in _walk_fns(fns) for layer in tr.layers if layer.index is not None]
        offset = max(used, default=-1) + 1
    new_fns = [copy.deepcopy(fn) for fn in fns]
    for tr in _walk_fns(new_fns):
        offset = tr.assign(offset, retain)
    return new_fns


# ======================================================================================== chain driver


def _final_update(group, param, update, grad):
    utils.update_param_(
        param, update, group["lr"], group["weight_decay"], caution=group["caution"],
        cautious_decay=group.get("cautious_weight_decay", False), grad=grad,
    )  # fmt: skip


def chain(state: list, group, grad, param, *fns):
    """Runs the transforms on a private copy of the gradients; unless one of them already wrote the
    parameters (signalled by ``_SKIP``), applies ``p <- p (1 - wd lr) - lr u`` at the end."""
    update = [torch.clone(g, memory_format=torch.preserve_format) for g in grad]
    ecc = ECCConfig.from_group(group, key="param_ecc")
    ctx = contextlib.nullcontext() if ecc is None else ecc.attached(param, [st["param::ecc"] for st in state])
    with ctx:
        update, skip = _inner_chain(state, group, update, grad, param, *fns)
        if not skip and update is not None:
            _final_update(group, param, update, grad)


# ======================================================================================== transform library
# Order of decorators = order of layers = order of indices.  Functions below are deliberately thin:
# the arithmetic lives in heavyball_b200.utils.


def _cwd(group):
    return group.get("cautious_weight_decay", False)


@zero_guard("mars_old_grad")
@no_state
def mars(group, update, grad, param, mars_old_grad):
    # argument order follows the reference call site (heavyball/chainable.py:645): the coefficient
    # is -beta1 * mars_gamma / (1 - mars_gamma)
    utils.mars_correction(update, mars_old_grad, group["mars_gamma"], utils.get_beta1(group))
    utils.copy_stochastic_list_(grad, update)
    return update


@zero_guard("exp_avg")
@no_state
def exp_avg(group, update, grad, param, exp_avg):
    return utils.scale_by_exp_avg_(exp_avg, update, utils.beta_debias(utils.get_beta1(group), group["step"]))


@copy_guard(2, "init")
@no_state
def weight_decay_to_init(group, update, grad, param, init):
    utils.stochastic_lerp_(param, init, group["weight_decay_to_ema"] * group["lr"])
    return update


def identity(state, group, update, grad, param):
    return update


@no_state
def apply_update(group, update, grad, param):
    _final_update(group, param, update, grad)
    return _SKIP


def _ema_decay_args(group):
    return utils.beta_debias(group["ema_beta"], group["step"]), group["weight_decay_to_ema"] * group["lr"]


@zero_guard("exp_avg")
@no_state
def weight_decay_to_ema(group, update, grad, param, exp_avg):
    utils.weight_decay_to_ema_(param, exp_avg, *_ema_decay_args(group))
    return update


@zero_guard("exp_avg")
@no_state
def l1_weight_decay_to_ema(group, update, grad, param, exp_avg):
    utils.l1_weight_decay_to_ema_(param, exp_avg, *_ema_decay_args(group))
    return update


@zero_guard("exp_avg_sq")
@no_state
def scale_by_exp_avg_sq(group, update, grad, param, exp_avg_sq):
    return utils.scale_by_exp_avg_sq_(
        exp_avg_sq, update, utils.beta_debias(utils.get_beta2(group), group["step"]), group["eps"]
    )


def _betas_step(group, shift=0):
    return utils.get_beta1(group), utils.get_beta2(group), group["step"] + shift


@zero_guard("exp_avg", "exp_avg_sq")
@no_state
def scale_by_adam(group, update, grad, param, exp_avg, exp_avg_sq):
    return utils.adam_(exp_avg, exp_avg_sq, update, *_betas_step(group), group["eps"])


def _fused_adam(group, update, grad, param, exp_avg, exp_avg_sq, decay):
    utils.fused_adam_(
        param, exp_avg, exp_avg_sq, update, grad, *_betas_step(group), group["lr"], group["eps"], decay,
        group["caution"], _cwd(group),
    )  # fmt: skip
    return _SKIP


@zero_guard("exp_avg", "exp_avg_sq")
@no_state
def update_by_adam(group, update, grad, param, exp_avg, exp_avg_sq):
    return _fused_adam(group, update, grad, param, exp_avg, exp_avg_sq, group["weight_decay"])


@zero_guard("exp_avg", "exp_avg_sq")
@no_state
def update_by_adamc(group, update, grad, param, exp_avg, exp_avg_sq):
    decay = group["lr"] * group["weight_decay"] / group["max_lr"]
    return _fused_adam(group, update, grad, param, exp_avg, exp_avg_sq, decay)


def _init_mu_product(state, group, update, grad, param, **kwargs):
    state["mu_product"] = torch.ones((), dtype=_storage_dtype(group), device=param.device)


@zero_guard("exp_avg", "exp_avg_sq")
@general_guard("mu_product", init_fn=_init_mu_product, skip_first=False)
@no_state
def scale_by_nadam(group, update, grad, param, exp_avg, exp_avg_sq, mu_product):
    utils.nadam_(
        param, exp_avg, exp_avg_sq, mu_product, update, *_betas_step(group), group["momentum_decay"], group["eps"],
        group["weight_decay"], group.get("decoupled_weight_decay", False),
    )  # fmt: skip
    return update


@zero_guard("exp_avg", "exp_avg_sq")
@general_guard("mu_product", init_fn=_init_mu_product, skip_first=False)
@no_state
def update_by_nadam(group, update, grad, param, exp_avg, exp_avg_sq, mu_product):
    utils.fused_nadam_(
        param, exp_avg, exp_avg_sq, mu_product, update, grad, *_betas_step(group), group["lr"], group["eps"],
        group["momentum_decay"], group["weight_decay"], group.get("decoupled_weight_decay", False),
        group["caution"], _cwd(group),
    )  # fmt: skip
    return _SKIP


def _ademamix_extra(group):
    return group["alpha"], group.get("beta3_warmup"), group.get("alpha_warmup")


@zero_guard("exp_avg_fast", "exp_avg_slow", "exp_avg_sq")
@no_state
def scale_by_ademamix(group, update, grad, param, exp_avg_fast, exp_avg_slow, exp_avg_sq):
    return utils.ademamix_(
        exp_avg_fast, exp_avg_slow, exp_avg_sq, update, group["betas"], group["step"], group["eps"],
        *_ademamix_extra(group),
    )  # fmt: skip


@zero_guard("exp_avg_fast", "exp_avg_slow", "exp_avg_sq")
@no_state
def update_by_ademamix(group, update, grad, param, exp_avg_fast, exp_avg_slow, exp_avg_sq):
    alpha, b3w, aw = _ademamix_extra(group)
    utils.fused_ademamix_(
        param, exp_avg_fast, exp_avg_slow, exp_avg_sq, update, grad, group["betas"], group["step"], group["lr"],
        group["eps"], group["weight_decay"], alpha, group["caution"], _cwd(group), b3w, aw,
    )  # fmt: skip
    return _SKIP


@zero_guard("exp_avg", "exp_avg_sq")
@no_state
def scale_by_laprop(group, update, grad, param, exp_avg, exp_avg_sq):
    return utils.laprop_(exp_avg, exp_avg_sq, update, *_betas_step(group))


@zero_guard("exp_avg", "exp_avg_sq")
@no_state
def update_by_laprop(group, update, grad, param, exp_avg, exp_avg_sq):
    utils.fused_laprop_(
        param, exp_avg, exp_avg_sq, update, grad, *_betas_step(group), group["lr"], group["weight_decay"],
        group["caution"], _cwd(group),
    )  # fmt: skip
    return _SKIP


@needs_full_param
@no_state
def orthogonalize_grad_to_param(group, update, grad, param):
    return utils.orthogonalize_grad_to_param(param, update, group["eps"])


def _sf_weight(group):
    step = max(utils.as_int(group["step"]), 1)
    return abs(group["lr"]) ** group["weight_lr_power"] * step ** group["r"]


@copy_guard(2, "z")
@no_state
def update_by_schedule_free(group, update, grad, param, z):
    # the running weight sum advances once per optimizer step, not once per parameter
    if group.get("_sf_step") != utils.as_int(group["step"]):
        group["weight_sum"] = group.get("weight_sum", 0) + _sf_weight(group)
        group["_sf_step"] = utils.as_int(group["step"])
    total = group["weight_sum"]
    ckp1 = _sf_weight(group) / total if total != 0 else 0
    update, param, z, grad = utils.list_guard(update, param, z, grad)
    utils._compilable_schedule_free_(
        param, z, ckp1, update, group["lr"], utils.get_beta1(group), group["weight_decay"], grad, group["caution"],
        _cwd(group),
    )  # fmt: skip
    return _SKIP


@needs_full_param
@copy_guard(2, "z")
@zero_guard("exp_avg")
@no_state
def update_by_msam(group, update, grad, param, z, exp_avg):
    utils.msam_(
        group["lr"], utils.beta_debias(utils.get_beta1(group), group["step"]), param, z, update, grad, exp_avg,
        group["caution"], group["weight_decay"], group["sam_step_size"], _cwd(group),
    )  # fmt: skip
    return _SKIP


def _adopt_warmup_1(state, group, update, grad, param, exp_avg, exp_avg_sq):
    utils.scale_by_exp_avg_sq_([exp_avg_sq], [update], 0, group["eps"])


@zero_guard("exp_avg", "exp_avg_sq")
@warmup_guard(_adopt_warmup_1)
@no_state
def update_by_adopt(group, update, grad, param, exp_avg, exp_avg_sq):
    utils.fused_adopt_(
        param, update, grad, exp_avg_sq, exp_avg, *_betas_step(group, -1), group["lr"], group["eps"],
        group["weight_decay"], group["caution"], _cwd(group),
    )  # fmt: skip
    return _SKIP


@zero_guard("exp_avg", "exp_avg_sq")
@warmup_guard(_adopt_warmup_1)
@no_state
def scale_by_adopt(group, update, grad, param, exp_avg, exp_avg_sq):
    return utils.adopt(update, exp_avg_sq, exp_avg, *_betas_step(group, -1))


def _suds_warmup_1(state, group, update, grad, param, exp_avg, exp_avg_sq, fisher_approx):
    utils.copy_stochastic_(fisher_approx, update / update.norm().clamp(min=1e-8))


@needs_full_param
@zero_guard("exp_avg", "exp_avg_sq", "fisher_approx")
@warmup_guard(_suds_warmup_1)
@no_state_no_multi_tensor
def scale_by_suds(group, update, grad, param, exp_avg, exp_avg_sq, fisher_approx):
    """Adam in the eigenbasis of a rank-1 curvature sketch ``lambda I + sigma v v^T`` (Householder
    rotation), with ``v`` tracked by Oja's rule."""
    direction = fisher_approx.flatten().to(update.dtype)
    rotated, w = utils.eigvecs_product_rank1(update.flatten(), direction)
    rotated = utils.adam_(exp_avg, exp_avg_sq, rotated.view_as(exp_avg), *_betas_step(group, -1))[0]
    out, _ = utils.eigvecs_product_rank1(rotated.flatten(), fisher_approx.flatten(), w)
    new_dir = utils.oja_update(direction, update.flatten(), group["precond_lr"])
    utils.copy_stochastic_(fisher_approx, new_dir.view_as(fisher_approx))
    return out


@zero_guard("exp_avg", "exp_avg_sq")
@no_state
def scale_by_unscaled_adam(group, update, grad, param, exp_avg, exp_avg_sq):
    return utils.unscaled_adam_(exp_avg, exp_avg_sq, update, *_betas_step(group))


@needs_full_param
@no_state_no_multi_tensor
def orthogonalize_update(group, update, grad, param, scale_mode: str = "scale"):
    if update.dim() < 2:
        return update
    flat = update.flatten(1, -1)
    utils.inplace_orthogonal_(flat, out=flat, scale_mode=scale_mode)
    return flat.reshape(update.shape)


@zero_guard("momentum")
@no_state
def nesterov_momentum(group, updates, grads, params, momentum):
    return utils.nesterov_momentum(momentum, updates, utils.get_beta1(group))


@zero_guard("momentum")
@no_state
def nesterov_ema(group, updates, grads, params, momentum):
    return utils.nesterov_ema(momentum, updates, utils.get_beta1(group))


@zero_guard("momentum")
@no_state
def heavyball_momentum(group, updates, grads, params, momentum):
    return utils.heavyball_momentum(momentum, updates, utils.get_beta1(group))


def _store_init_norm(state, group, update, grad, param):
    state["init_norm"] = param.to(_storage_dtype(group)).norm()


@needs_full_param
@general_guard("init_norm", init_fn=_store_init_norm, skip_first=False)
@no_state
def update_by_hyperball(group, update, grad, param, init_norm):
    utils.hyperball_step_(
        param, update, init_norm, group["lr"], group["weight_decay"], group["caution"], grad, _cwd(group)
    )
    return _SKIP


def _store_std(state, group, update, grad, param):
    state["init_std"] = torch.std(param.to(_storage_dtype(group)))


@needs_full_param
@general_guard("init_std", init_fn=_store_std, skip_first=False)
@no_state
def mup_approx(group, updates, grads, params, init_std):
    pairs = [(u, s) for u, s in zip(updates, init_std) if u.ndim > 1]
    if pairs:
        us, ss = zip(*pairs)
        utils.stochastic_multiply_(list(us), list(ss))
    return updates


def _init_delta(state, group, update, grad, param, log_space: bool, full: bool = False):
    val = math.log(group["initial_d"]) if log_space else group["initial_d"]
    if full:
        state["delta"] = torch.full_like(param, val)
    else:
        state["delta"] = torch.full((), val, dtype=param.dtype, device=param.device)


_init_full_delta = functools.partial(_init_delta, full=True)


@needs_full_param
@zero_guard("state")
@general_guard("delta", init_fn=functools.partial(_init_delta, log_space=False), skip_first=False)
@no_state
def scale_by_d_adaptation(group, update, grad, param, state, delta):
    utils.d_adaptation(grad, update, state, delta)
    return update


@needs_full_param
@zero_guard("state")
@general_guard("delta", init_fn=functools.partial(_init_delta, log_space=True), skip_first=False)
@no_state
def scale_by_lr_adaptation(group, update, grad, param, state, delta):
    utils.lr_adaptation(grad, update, state, delta, group["lr_lr"])
    return update


@zero_guard("state")
@general_guard("delta", init_fn=functools.partial(_init_full_delta, log_space=True), skip_first=False)
@no_state
def scale_by_pointwise_lr_adaptation(group, update, grad, param, state, delta):
    utils.pointwise_lr_adaptation(grad, update, state, delta, group["lr_lr"])
    return update


def _init_scion_state(state, group, update, grad, param):
    state["scion_state"] = {"initialized": False}


@needs_full_param
@general_guard("scion_state", init_fn=_init_scion_state, skip_first=False)
@no_state
def scion_auto_norm(group, update, grad, param, scion_state):
    scale = group.get("scale", 1.0)
    position = {id(p): i for i, p in enumerate(group["params"])}
    for ctx, p in zip(scion_state, param):
        if not ctx["initialized"]:
            utils.scion_auto_init_param_(p, scale, seed=position.get(id(p), 0))
            ctx["initialized"] = True
    return utils.scion_auto_lmo_(update, scale)


@needs_full_param
@no_state
def sign(group, update, grad, param, graft: bool = True):
    return utils.sign_(update, graft)


@no_state
def global_clip(group, update, grad, param, clip_fn: Optional[callable] = None):
    assert clip_fn is not None
    return clip_fn(update)


def palm_beta2(state, group, update, grad, param):
    """PaLM schedule: ``beta2 = 1 - step^-beta2_scale``."""
    betas = group["betas"]
    group["betas"] = (utils.get_beta1(group), 1 - utils.as_int(group["step"]) ** -group["beta2_scale"], *betas[2:])
    group["_palm_active"] = True
    return update


def apply_to_idx(fn, idx):
    """Wraps ``fn(list_of_tensors)`` (or its name in ``utils``) as a transform acting on argument
    ``idx`` of ``(state, group, update, grad, param)``."""
    name = fn
    if isinstance(fn, str):
        fn = getattr(utils, fn, None)
        if fn is None or not callable(fn):
            raise ValueError(f"Unknown function '{name}'")

    def _fn(state, group, update, grad, param):
        return fn([state, group, update, grad, param][idx])

    _fn.__name__ = _fn.__qualname__ = f"apply_{getattr(fn, '__name__', repr(fn))}_to_{idx}"
    _fn.wrapped_fn = fn
    return _fn


# ---------------------------------------------------------------------------------------- SOAP family


def _init_soap(state, group, update, grad, param):
    utils.init_preconditioner(
        grad, state, group["max_precond_dim"], group["precondition_1d"], group.get("init_factor", 0.0)
    )


def _apply_soap_preconditioner(group, update, Q, GG, *exp_avgs, use_kl=False, eps=1e-8, exp_avg_sq=None, heavy=False):
    """Accumulates Kronecker statistics from this step's update and, on refresh steps, advances the
    eigenbases and rotates the moment buffers."""
    beta = utils.beta_debias(group["shampoo_beta"], group["step"])
    max_dim, p1d = group["max_precond_dim"], group["precondition_1d"]
    sqs = exp_avg_sq or [None] * len(update)
    for u, q, gg, sq, *moments in zip(update, Q, GG, sqs, *exp_avgs):
        g = utils.promote(u)
        if use_kl:
            utils.update_ggt_kl(g, gg, q, max_dim, p1d, beta, eps, heavy=heavy)
        else:
            utils.update_ggt(g, gg, max_dim, p1d, beta)
        if group["is_preconditioning"]:
            utils.get_orthogonal_matrix_QR(gg, q, *moments, exp_avg_sq=sq if heavy else None, heavy=heavy)


def _inner_adam(group, g, st):
    return utils.adam_(st["exp_avg"], st["exp_avg_sq"], g, *_betas_step(group, -1), group["eps"])


def _inner_laprop(group, g, st):
    return utils.laprop_(st["exp_avg"], st["exp_avg_sq"], g, *_betas_step(group, -1))


def _inner_nadam(group, g, st):
    return utils.nadam_(
        g, st["exp_avg"], st["exp_avg_sq"], st["mu_product"], g, *_betas_step(group, -1), group["momentum_decay"],
        group["eps"], 0.0, False,
    )  # fmt: skip


def _inner_ademamix(group, g, st):
    return utils.ademamix_(
        st["exp_avg_fast"], st["exp_avg_slow"], st["exp_avg_sq"], g, group["betas"], group["step"] - 1, group["eps"],
        *_ademamix_extra(group),
    )  # fmt: skip


def _make_soap(name, slots, inner, rotated, *, kl=False, heavy=False, mu=False):
    """Builds one member of the SOAP family: project into the eigenbasis, run ``inner`` there,
    project back, then update statistics / eigenbasis.  ``rotated`` names the moment buffers that
    follow the basis when it is refreshed."""
    arg_names = [*slots, *(["mu_product"] if mu else []), "Q", "GG"]

    def body(group, update, grad, param, *state_lists):
        st = dict(zip(arg_names, state_lists))
        projected = [utils.project(utils.promote(u), q, False) for u, q in zip(update, st["Q"])]
        precond = inner(group, projected, st)
        precond = [utils.project(p, q, True) for p, q in zip(precond, st["Q"])]
        extra = {"use_kl": True, "eps": group["eps"]} if kl else {}
        if heavy:
            extra.update(exp_avg_sq=st["exp_avg_sq"], heavy=True)
        _apply_soap_preconditioner(group, update, st["Q"], st["GG"], *[st[r] for r in rotated], **extra)
        return precond

    body.__name__ = body.__qualname__ = name
    tr = no_state(body)
    tr = general_guard("Q", "GG", init_fn=_init_soap)(tr)
    if mu:
        tr = general_guard("mu_product", init_fn=_init_mu_product, skip_first=False)(tr)
    return needs_full_param(bucket_aware(zero_guard(*slots)(tr)))


_ADAM_SLOTS = ("exp_avg", "exp_avg_sq")
_MIX_SLOTS = ("exp_avg_fast", "exp_avg_slow", "exp_avg_sq")
scale_by_soap = _make_soap("scale_by_soap", _ADAM_SLOTS, _inner_adam, ("exp_avg",))
scale_by_kl_soap = _make_soap("scale_by_kl_soap", _ADAM_SLOTS, _inner_adam, ("exp_avg",), kl=True)
scale_by_soap_nadam = _make_soap("scale_by_soap_nadam", _ADAM_SLOTS, _inner_nadam, ("exp_avg",), mu=True)
scale_by_soap_laprop = _make_soap("scale_by_soap_laprop", _ADAM_SLOTS, _inner_laprop, ("exp_avg",))
scale_by_soap_ademamix = _make_soap(
    "scale_by_soap_ademamix", _MIX_SLOTS, _inner_ademamix, ("exp_avg_slow", "exp_avg_fast")
)
scale_by_heavy_soap = _make_soap("scale_by_heavy_soap", _ADAM_SLOTS, _inner_adam, ("exp_avg",), heavy=True)
scale_by_heavy_kl_soap = _make_soap(
    "scale_by_heavy_kl_soap", _ADAM_SLOTS, _inner_adam, ("exp_avg",), kl=True, heavy=True
)
scale_by_heavy_soap_nadam = _make_soap(
    "scale_by_heavy_soap_nadam", _ADAM_SLOTS, _inner_nadam, ("exp_avg",), mu=True, heavy=True
)
scale_by_heavy_soap_laprop = _make_soap(
    "scale_by_heavy_soap_laprop", _ADAM_SLOTS, _inner_laprop, ("exp_avg",), heavy=True
)
scale_by_heavy_soap_ademamix = _make_soap(
    "scale_by_heavy_soap_ademamix", _MIX_SLOTS, _inner_ademamix, ("exp_avg_slow", "exp_avg_fast"), heavy=True
)


def _make_kl_shampoo(name, heavy):
    def body(group, update, grad, param, exp_avg, Q, GG):
        utils.stochastic_lerp_(exp_avg, update, 1 - utils.get_beta1(group))
        precond = [utils.kl_shampoo_precondition(e, q, gg, group["eps"]) for e, q, gg in zip(exp_avg, Q, GG)]
        damp = group.get("dampening", 0.0)
        accum = [utils.dampen_grad(u, damp)[1] for u in update] if damp > 0 else update
        _apply_soap_preconditioner(group, accum, Q, GG, use_kl=True, eps=group["eps"], heavy=heavy)
        for gg in GG:
            live = [m for m in gg if isinstance(m, Tensor)]
            if len(live) >= 2:
                utils.psgd_balance_Q(live)
        return precond

    body.__name__ = body.__qualname__ = name
    tr = general_guard("Q", "GG", init_fn=_init_soap)(no_state(body))
    return needs_full_param(bucket_aware(zero_guard("exp_avg")(tr)))


scale_by_kl_shampoo = _make_kl_shampoo("scale_by_kl_shampoo", False)
scale_by_heavy_kl_shampoo = _make_kl_shampoo("scale_by_heavy_kl_shampoo", True)


# ---------------------------------------------------------------------------------------- PSGD family


def _fresh_Q(group, grad, hessian_vector=None, vector=None):
    return utils.init_Q_exprs(
        grad, group["precond_init_scale"], group["precond_init_scale_scale"], group["precond_init_scale_power"],
        group["max_size_triangular"], group["min_ndim_triangular"], group["memory_save_mode"], hessian_vector, vector,
        dtype=getattr(torch, group["q_dtype"]),
    )  # fmt: skip


def _fresh_bounds(state, grad, Q, param):
    state["running_lower_bound"] = [torch.zeros((grad.shape[0],), device=q.device, dtype=torch.float64) for q in Q]
    state["step"] = torch.zeros((), device=param.device, dtype=torch.float64)


def _init_psgd_kron(state, group, update, grad, param, cached: bool = False, prob: Optional[callable] = None):
    tmp = utils.get_temporary(group, param) or {}
    Q = _fresh_Q(group, grad, tmp.get("hessian_vector"), tmp.get("vector"))
    state["Q"] = utils.triu_to_line(Q) if group["store_triu_as_line"] else Q
    _fresh_bounds(state, grad, Q, param)
    if cached:
        state["Q_cache"] = [torch.empty_like(q) for q in Q]


def _init_psgd_pro_kron(state, group, update, grad, param, cached: bool = False, prob: Optional[callable] = None):
    Q = _fresh_Q(group, grad)
    state["Q"] = Q
    _fresh_bounds(state, grad, Q, param)
    if cached:
        state["Q_cache"] = [torch.empty_like(q) for q in Q]


def _init_psgd_eigen_kron(state, group, update, grad, param, prob: Optional[callable] = None):
    tmp = utils.get_temporary(group, param) or {}
    Q = _fresh_Q(group, grad, tmp.get("hessian_vector"), tmp.get("vector"))
    _fresh_bounds(state, grad, Q, param)
    _update_psgd_precond(
        False, None, group, param, update, Q, state["running_lower_bound"], state["step"], prob, store_triu_as_line=False
    )
    state["Q"] = utils.triu_to_line(Q) if group["store_triu_as_line"] else Q
    state["Q_basis"] = utils.init_psgd_eigenbasis(Q)


def _init_psgd_lra(state, group, update, grad, param, cached: bool = False, prob: Optional[callable] = None):
    tmp = utils.get_temporary(group, param) or {}
    state["U"], state["V"], state["d"] = utils.init_lra(
        grad, group["param_count"], group["precond_init_scale"], group["precond_init_scale_scale"],
        group["precond_init_scale_power"], group["rank"], tmp.get("hessian_vector"), tmp.get("vector"),
        dtype=getattr(torch, group["q_dtype"]),
    )  # fmt: skip


def _fill_q_cache(Q_cache, Q):
    for i, q in enumerate(Q):
        if Q_cache[i] is None:
            Q_cache[i] = torch.empty_like(q)
        if q.ndim == 3:
            torch.matmul(q.mT, q, out=Q_cache[i])
        else:
            torch.mul(q, q, out=Q_cache[i])


def _decide_cache(group, cached, prob):
    prob = utils.precond_update_prob_schedule() if prob is None else prob
    p = prob if isinstance(prob, float) else prob(group["step"])
    group["is_cached"] = use = bool(cached and p < 0.5)
    return use


def _update_psgd_precond(cached, Q_cache, group, param, grad, Q, running_lower_bound, step, prob=None,
                         store_triu_as_line=None):  # fmt: skip
    if store_triu_as_line is None:
        store_triu_as_line = group["store_triu_as_line"]
    if not group["is_preconditioning"]:
        return
    if (utils.get_temporary(group, param) or {}).get("vector") is None:
        vector, hessian_vector = utils.dampen_grad(grad, group["dampening"])
    else:
        vector, hessian_vector = utils.take_temporary(group, param, "vector", "hessian_vector")
    utils.psgd_update_precond(
        hessian_vector, group["precond_lr"], Q, store_triu_as_line, utils.get_beta2(group), vector,
        running_lower_bound, group["lower_bound_beta"], group["precond_update_power_iterations"],
    )  # fmt: skip
    del vector, hessian_vector
    if _decide_cache(group, cached, prob):
        _fill_q_cache(Q_cache, utils.line_to_triu(Q) if store_triu_as_line else Q)


def _update_psgd_pro_precond(cached, Q_cache, group, param, grad, Q, running_lower_bound, step, prob=None):
    if not group["is_preconditioning"]:
        return
    utils.psgd_pro_update_precond(
        grad, group["precond_lr"], Q, running_lower_bound, group["lower_bound_beta"],
        group["precond_update_power_iterations"], group["dampening"],
    )  # fmt: skip
    if _decide_cache(group, cached, prob):
        _fill_q_cache(Q_cache, Q)


def _use_cache(group, Q_cache):
    return not group.get("sqrt", False) and group.get("is_cached", False) and Q_cache[0] is not None


def _cached_psgd_precond_grad(group, update, Q, Q_cache, grad):
    if _use_cache(group, Q_cache):
        return utils.precond_grad_cached_(ea=update, cached_q=Q_cache, caution=False, grad=grad)
    return utils.psgd_precond_grad(
        ea=update, preconds=Q, caution=False, grad=grad, store_triu_as_line=group["store_triu_as_line"],
        sqrt=group.get("sqrt", False),
    )  # fmt: skip


def _fused_cached_psgd_precond_grad(group, grad, param, update, Q, Q_cache):
    common = dict(
        ea=update, caution=group["caution"], grad=grad, param=param, lr=group["lr"], decay=group["weight_decay"],
        cautious_decay=_cwd(group),
    )  # fmt: skip
    if _use_cache(group, Q_cache):
        utils.fused_precond_grad_cached_(cached_q=Q_cache, **common)
    else:
        utils.fused_psgd_precond_grad(
            preconds=Q, store_triu_as_line=group["store_triu_as_line"], sqrt=group.get("sqrt", False), **common
        )


def _make_psgd(name, *, init_fn, fit, fused, delayed):
    """``fit`` refreshes Q (on preconditioner steps); ``delayed`` applies the old Q before fitting;
    ``fused`` writes the parameter instead of returning the preconditioned update."""

    def body(group, update, grad, param, update_to_precond, Q, Q_cache, running_lower_bound: List[Tensor],
             step: Tensor, cached: bool = False, prob: Optional[callable] = None):  # fmt: skip
        do_fit = lambda: fit(cached, Q_cache, group, param, update_to_precond, Q, running_lower_bound, step, prob)  # noqa: E731
        if not delayed:
            do_fit()
        if fused:
            _fused_cached_psgd_precond_grad(group, update, param, update, Q, Q_cache)
            out = _SKIP
        else:
            out = _cached_psgd_precond_grad(group, update, Q, Q_cache, grad)
        if delayed:
            do_fit()
        return out

    body.__name__ = body.__qualname__ = name
    tr = no_state_no_multi_tensor(body)
    tr = general_guard("Q", "Q_cache", "running_lower_bound", "step", init_fn=init_fn, skip_first=False)(tr)
    return needs_full_param(bucket_aware(SqueezeGrad(PrecondGradAccumGuard(tr))))


scale_by_psgd = _make_psgd("scale_by_psgd", init_fn=_init_psgd_kron, fit=_update_psgd_precond, fused=False, delayed=False)
scale_by_delayed_psgd = _make_psgd(
    "scale_by_delayed_psgd", init_fn=_init_psgd_kron, fit=_update_psgd_precond, fused=False, delayed=True
)
update_by_psgd = _make_psgd("update_by_psgd", init_fn=_init_psgd_kron, fit=_update_psgd_precond, fused=True, delayed=False)
update_by_delayed_psgd = _make_psgd(
    "update_by_delayed_psgd", init_fn=_init_psgd_kron, fit=_update_psgd_precond, fused=True, delayed=True
)
scale_by_psgd_pro = _make_psgd(
    "scale_by_psgd_pro", init_fn=_init_psgd_pro_kron, fit=_update_psgd_pro_precond, fused=False, delayed=False
)
update_by_psgd_pro = _make_psgd(
    "update_by_psgd_pro", init_fn=_init_psgd_pro_kron, fit=_update_psgd_pro_precond, fused=True, delayed=False
)


@needs_full_param
@bucket_aware
@SqueezeGrad
@PrecondGradAccumGuard
@zero_guard("exp_avg", "exp_avg_sq")
@general_guard("Q", "Q_basis", "running_lower_bound", "step", init_fn=_init_psgd_eigen_kron, skip_first=True)
@no_state_no_multi_tensor
def scale_by_lather(group, update, grad, param, update_to_precond, exp_avg, exp_avg_sq, Q, Q_basis,
                    running_lower_bound: List[Tensor], step: Tensor, prob: Optional[callable] = None):  # fmt: skip
    """Adam in the eigenbasis of the PSGD preconditioner ``Q^T Q``."""
    projected = utils.project(utils.promote(update), Q_basis, False)
    precond = utils.adam_(exp_avg, exp_avg_sq, projected, *_betas_step(group), group["eps"])[0]
    precond = utils.project(precond, Q_basis, True)
    if group["is_preconditioning"]:
        _update_psgd_precond(False, None, group, param, update_to_precond, Q, running_lower_bound, step, prob)
        dense = utils.line_to_triu(Q) if group["store_triu_as_line"] else Q
        utils.update_psgd_eigenbasis(dense, Q_basis, exp_avg)
    return precond


def _update_lra(group, U, V, d, params, grads, delayed: bool):
    if not group["is_preconditioning"]:
        return utils.multi_flatten((U, 1), (V, 1), (d, 0))
    if (utils.get_temporary(group, params[0]) or {}).get("hessian_vector") is not None:
        pairs = [utils.take_temporary(group, p, "vector", "hessian_vector") for p in params]
        vector = utils.flatten([v for v, _ in pairs])
        hessian_vector = utils.flatten([hv for _, hv in pairs])
    else:
        vector, hessian_vector = utils.dampen_multiple(grads)
    k = group["precond_step"] = group.get("precond_step", -1) + 1
    return utils.update_lra_precond_(U, V, d, vector, hessian_vector, group["eps"], group["precond_lr"], delayed, bool(k % 2))


def _make_lra(name, *, fused, delayed):
    def body(group, update, grad, param, update_to_precond, U, V, d):
        u, v, dd = _update_lra(group, U, V, d, param, update_to_precond, delayed)
        if fused:
            utils.apply_lra_update(
                param, update, u, v, dd, group["lr"], group["weight_decay"], group["caution"], grad, _cwd(group)
            )
            return _SKIP
        return utils.extract_from_flat_update(param, utils.lra_precond(u, v, dd, utils.flatten(update)))

    body.__name__ = body.__qualname__ = name
    tr = general_guard("U", "V", "d", init_fn=_init_psgd_lra, skip_first=False)(no_state(body))
    return needs_full_param(SqueezeGrad(PrecondGradAccumGuard(tr)))


scale_by_psgd_lra = _make_lra("scale_by_psgd_lra", fused=False, delayed=False)
update_by_psgd_lra = _make_lra("update_by_psgd_lra", fused=True, delayed=False)
scale_by_delayed_psgd_lra = _make_lra("scale_by_delayed_psgd_lra", fused=False, delayed=True)
update_by_delayed_psgd_lra = _make_lra("update_by_delayed_psgd_lra", fused=True, delayed=True)


# ======================================================================================== optimizer classes


def _build_defaults(locals_dict):
    """Turns a constructor's ``locals()`` into ``(params, defaults)``: renames deprecated kwargs,
    rejects removed and unknown ones."""
    d = dict(locals_dict)
    d.pop("self", None)
    params = d.pop("params")
    kwargs = d.pop("kwargs")
    for old, new in _RENAMED_KWARGS.items():
        if old in kwargs:
            warnings.warn(
                f"'{old}' was renamed to '{new}' in HeavyBall 3.0. Pass '{new}' instead.", FutureWarning, stacklevel=4
            )
            d[new] = kwargs.pop(old)
    gone = _REMOVED_KWARGS & kwargs.keys()
    if gone:
        raise TypeError(f"Removed in HeavyBall 3.0: {', '.join(sorted(gone))}. See docs/heavyball3.md for migration details.")
    unknown = kwargs.keys() - _PASSTHROUGH_KWARGS
    if unknown:
        raise TypeError(f"unknown keyword arguments: {sorted(unknown)}")
    d.update(kwargs)
    return params, d


_PASSTHROUGH_KWARGS = frozenset({"orig_shapes", *utils.StatefulOptimizer._INSTANCE_ATTRS})
_RENAMED_KWARGS = {"foreach": "multi_tensor"}
_REMOVED_KWARGS = frozenset({"stochastic_schedule", "normalize_grads", "correct_bias", "inverse_free", "adaptive"})


_TENSOR_GROUP_KEYS = ("prev_lr", "weight_sum")


class ChainOpt(utils.StatefulOptimizer):
    promote: bool = False
    global_defaults = {"caution": False, "lr": 1, "warmup_steps": 0, "weight_decay": 0, "eps": 1e-8}

    def __init__(self, params, defaults, *fns):
        from .parallel import fsdp as _fsdp

        orig = defaults.pop("orig_shapes", None)
        self._orig_shapes = (
            None if orig is None else {k: _fsdp.ShapeInfo(v) if isinstance(v, tuple) else v for k, v in orig.items()}
        )
        base = dict(self.global_defaults)
        base.update({k: v for k, v in defaults.items() if v is not use_default})
        self._local_shards = _fsdp.LocalShards()
        params = self._local_shards.localize(params)  # fully_shard (DTensor) parameters -> plain local-row proxies
        if self._local_shards:
            self._orig_shapes = {**(self._orig_shapes or {}), **self._local_shards.infos}
        super().__init__(params, base)
        self.fns = fns
        self._lowered = None
        self.register_load_state_dict_post_hook(ChainOpt._restore_ecc_dtypes)
        self.register_load_state_dict_post_hook(ChainOpt._scalarize_group_keys)
        self._init_param_ecc()

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        sd = super().state_dict()
        for g in sd["param_groups"]:
            if g.get("_palm_active") and "betas" in g:  # the PaLM schedule stores beta2 as a 0-d tensor
                b = g["betas"]
                g["betas"] = (b[0], torch.tensor(float(b[1]), dtype=torch.float32), *b[2:])
            for k in [k for k in g if k.startswith("_")]:
                del g[k]
            for k in _TENSOR_GROUP_KEYS:  # host scalars here, 0-d tensors in the checkpoint format
                if isinstance(g.get(k), (int, float)) and not isinstance(g.get(k), bool):
                    g[k] = torch.tensor(float(g[k]), dtype=torch.float32)
        return sd

    @staticmethod
    def _scalarize_group_keys(optimizer, *args):
        for g in optimizer.param_groups:
            for k in _TENSOR_GROUP_KEYS:
                if isinstance(g.get(k), Tensor):
                    g[k] = float(g[k])
            if any(isinstance(b, Tensor) for b in g.get("betas", ())):
                g["betas"] = tuple(float(b) if isinstance(b, Tensor) else b for b in g["betas"])

    # ------------------------------------------------------------------ parameter ECC
    def _init_param_ecc(self):
        for group in self.param_groups:
            self._init_param_ecc_group(group)

    def _init_param_ecc_group(self, group):
        """``param_ecc``: parameters are narrowed to the 16-bit primary dtype in place and the
        rounding residual is kept in ``state[...]["param::ecc"]``."""
        ecc = ECCConfig.from_group(group, key="param_ecc")
        if ecc is None:
            return
        for p in group["params"]:
            wide = None
            if p.dtype != ecc.primary_dtype:
                wide = p.data.float()
                p.data = p.data.to(ecc.primary_dtype)
                for old in self.mapping.pop(p, ()):
                    self.mapping_inverse.pop(utils._tensor_key(old), None)
            if p not in self.mapping:
                self._register_views(p, utils.merge_group(group, p))
            wide_views = None if wide is None else utils.merge_group(group, wide)
            for i, pv in enumerate(self.mapping[p]):
                st = self.state_(pv)
                if "param::ecc" in st:
                    continue
                st["param::ecc"] = torch.zeros_like(pv, dtype=ecc.corr_dtype)
                if wide_views is not None:
                    ecc.init_correction(st["param::ecc"], wide_views[i], pv.data)

    def add_param_group(self, param_group):
        shards = getattr(self, "_local_shards", None)
        if shards is not None and any(_is_dtensor(p) for p in _as_list(param_group.get("params", ()))):
            param_group = shards.localize([param_group])[0]
            self._orig_shapes = {**(self._orig_shapes or {}), **shards.infos}
        super().add_param_group(param_group)
        if getattr(self, "_fns", None) is not None:  # groups added after construction; the constructor does all of its own at once
            self._init_param_ecc_group(self.param_groups[-1])

    def zero_grad(self, set_to_none: bool = True):
        super().zero_grad(set_to_none)
        if getattr(self, "_local_shards", None):
            self._local_shards.clear_grads()

    def step(self, closure=None):
        if self._local_shards:
            self._local_shards.refresh()
        return super().step(closure)

    @staticmethod
    def _restore_ecc_dtypes(optimizer, *args):
        """``load_state_dict`` casts every state tensor to the parameter dtype; put ECC primaries and
        corrections back to their storage dtypes and rebuild missing parameter corrections."""
        for group in optimizer.param_groups:
            ecc = ECCConfig.from_group(group, key="ecc")
            pecc = ECCConfig.from_group(group, key="param_ecc")
            if ecc is None and pecc is None:
                continue
            for p in group["params"]:
                for view_state in (optimizer.state.get(p) or {}).values():
                    if not isinstance(view_state, dict):
                        continue
                    for k, v in list(view_state.items()):
                        if not isinstance(v, Tensor):
                            continue
                        cfg = pecc if (k == "param" or k.startswith("param::")) else ecc
                        if cfg is None:
                            continue
                        if k.endswith("::ecc"):
                            view_state[k] = v.to(cfg.corr_dtype)
                        elif (k + "::ecc") in view_state:
                            view_state[k] = v.to(cfg.primary_dtype)
                if pecc is not None and p.dtype != pecc.primary_dtype:
                    before = utils._tensor_key(p)
                    p.data = p.data.to(pecc.primary_dtype)
                    if before in optimizer.mapping_inverse:
                        optimizer.mapping_inverse[utils._tensor_key(p)] = optimizer.mapping_inverse.pop(before)
            if pecc is not None:
                optimizer._init_param_ecc_group(group)

    # ------------------------------------------------------------------ transforms
    @property
    def fns(self):
        return self._fns

    @fns.setter
    def fns(self, value):
        self._fns = set_indices(value, retain=True)
        trs = list(_walk_fns(self._fns))
        self._needs_gather = any(getattr(tr, "needs_full_param", False) for tr in trs)
        self._transform_ids = frozenset(
            layer.index
            for tr in trs
            for layer in tr.layers
            if layer.index is not None and layer.needs_init and not layer.under_bucket
        )
        self._lowered = None

    def _set_indices(self, retain=True):
        self._fns = set_indices(self._fns, retain)

    def _find_val_name(self, name):
        for tr in _walk_fns(self._fns):
            names = tr._val_names
            if name in names:
                return names[name]
        raise KeyError(f"No transform stores '{name}'")

    # ------------------------------------------------------------------ stepping
    def _step(self, group):
        from .parallel import fsdp as _fsdp

        if "base_lr" not in group:
            group["base_lr"] = group["lr"]
        elif group["base_lr"] != group["lr"]:
            utils.warn_once(
                "Learning rate changed between steps. This is an experimental feature and "
                f"only supported with multi_tensor=True (currently multi_tensor={group['multi_tensor']})."
            )
            group["base_lr"] = group["lr"]
        if self._orig_shapes is None:
            self._orig_shapes = _fsdp.detect_orig_shapes([p for g in self.param_groups for p in g["params"]])
        views, gathers = _fsdp.reshape_params(group["params"], self._orig_shapes, self._needs_gather, cache_owner=self)
        group["_orig_shapes"] = self._orig_shapes
        try:
            self._step_inner(group)
        finally:
            _fsdp.restore_params(views, gathers)

    def _recover_step(self, group):
        step = group.get("_group_step")
        if step is not None:
            return utils.as_int(step)
        for param in group["params"]:
            per_view = self.state.get(param)
            if not isinstance(per_view, dict):
                continue
            for st in per_view.values():
                if isinstance(st, dict) and "step" in st and not isinstance(st["step"], float):
                    found = st["step"]
                    if isinstance(found, Tensor) and found.dtype.is_floating_point:
                        continue  # PSGD keeps an unrelated fp64 "step" under an indexed key only
                    return utils.as_int(found)
        return 0

    def _step_inner(self, group):
        pairs = list(self.split_p_and_g_in_group(group, should_promote=self.promote))
        if not pairs:
            return
        p, g = zip(*pairs)
        caution = group["caution"]
        step = self._recover_step(group) + 1
        group["_group_step"] = group["step"] = step
        self.state_(p[0])["step"] = torch.tensor(step, dtype=torch.int64)
        group["prev_lr"] = group["lr"] = group["base_lr"] * step / max(step, group["warmup_steps"] + 1)
        try:
            if not group["multi_tensor"] or len(p) == 1:
                for pi, gi in zip(p, g):
                    self._chain(group, [gi], [pi], caution)
            else:
                self._chain(group, g, p, caution)
        finally:
            group["caution"] = caution
            group["lr"] = group["base_lr"]
            group["step"] = None

    def _run_chain(self, state, group, g, p, caution):
        chain(state, group, g, p, *self.fns)

    def _needs_init(self, state):
        if not self._transform_ids:
            return False
        done = set()
        for st in state:
            done.update(st.get("is_initialized", ()))
        return not self._transform_ids.issubset(done)

    def _chain(self, group, g, p, caution):
        state = [self.state_(pi) for pi in p]
        pecc = ECCConfig.from_group(group, key="param_ecc")
        if pecc is not None:
            # a parameter gathered on its owner rank is larger than the local rows its residual was created for: the
            # owner keeps the residual of the whole tensor, like the rest of the state
            for st, pi in zip(state, p):
                held = st.get("param::ecc")
                if held is None or held.shape != pi.shape:
                    st["param::ecc"] = torch.zeros_like(pi, dtype=pecc.corr_dtype)
        from . import lowering

        if (p[0].is_cuda or lowering.cpu_programs) and lowering.try_run(self, state, group, list(g), list(p)):
            return
        self._run_chain(state, group, list(g), list(p), caution)


def _as_list(ps):
    return [ps] if isinstance(ps, Tensor) else list(ps)


def _is_dtensor(p):
    from .parallel import fsdp as _fsdp

    return _fsdp.is_dtensor(p)


str_or_fn = Union[str, callable, None, Literal[use_default]]


def default(a, b):
    return b if a is use_default else a


# scale_by_X <-> update_by_X: the fused form writes the parameter inside the transform
_FUSION_PAIRS = (
    (scale_by_delayed_psgd, update_by_delayed_psgd),
    (scale_by_psgd, update_by_psgd),
    (scale_by_psgd_lra, update_by_psgd_lra),
    (scale_by_delayed_psgd_lra, update_by_delayed_psgd_lra),
    (scale_by_adam, update_by_adam),
    (scale_by_nadam, update_by_nadam),
    (scale_by_laprop, update_by_laprop),
    (scale_by_adopt, update_by_adopt),
    (scale_by_ademamix, update_by_ademamix),
    (scale_by_psgd_pro, update_by_psgd_pro),
)
_scale_to_update_map = {s.get_fn(): u for s, u in _FUSION_PAIRS}
_scale_to_update_map_inv = {u.get_fn(): s for s, u in _FUSION_PAIRS}


class BaseOpt(ChainOpt):
    """Adds the cross-cutting constructor options to a chain.

    ``gradient_clipping`` — function (or name in ``utils``) applied to incoming gradients first;
    ``update_clipping`` — applied to the outgoing update, which disables fused ``update_by_*`` forms;
    ``palm`` — PaLM beta2 schedule; ``mars`` (from ``defaults``) — MARS gradient correction;
    ``promote`` — widen gradients to fp32 before the chain; ``compile_step`` — accepted for source
    compatibility (fused execution is selected automatically on CUDA).
    """

    gradient_clipping: str_or_fn = None
    update_clipping: str_or_fn = None
    palm: bool = False
    auto_fuse: bool = True

    def __init__(self, params, defaults, gradient_clipping: str_or_fn = None, update_clipping: str_or_fn = None,
                 palm: bool = use_default, fns: Iterable[callable] = (), compile_step: bool = use_default,
                 promote: bool = use_default):  # fmt: skip
        if not fns:
            raise ValueError("No functions provided. If that's on purpose (SGD-like), use `identity`")
        fns = tuple(fns)
        last, bound = fns[-1], None
        if isinstance(last, functools.partial):
            last, bound = last.func, (last.args, last.keywords)
        last_fn = last.get_fn() if isinstance(last, FunctionTransform) else last
        rebind = lambda f: f if bound is None else functools.partial(f, *bound[0], **bound[1])  # noqa: E731

        clip = default(update_clipping, self.update_clipping)
        if clip is None:
            if self.auto_fuse and last_fn in _scale_to_update_map:
                fns = fns[:-1] + (rebind(_scale_to_update_map[last_fn]),)
        elif last_fn in _scale_to_update_map_inv:
            if not self.auto_fuse:
                raise ValueError(
                    "update_clipping is currently not compatible with update_by_* functions. "
                    "Manually select scale_by_* functions or set auto_fuse=True."
                )
            fns = fns[:-1] + (rebind(_scale_to_update_map_inv[last_fn]),)

        self.compile_step = default(default(compile_step, defaults.pop("compile_step", use_default)), self.compile_step)
        self.promote = default(default(promote, defaults.pop("promote", use_default)), self.promote)
        defaults.pop("update_clipping", None)  # callables must not leak into the state_dict
        defaults.pop("gradient_clipping", None)
        if default(palm, self.palm):
            fns = (palm_beta2,) + fns
        gclip = default(gradient_clipping, self.gradient_clipping)
        if gclip is not None:
            fns = (apply_to_idx(gclip, 2),) + fns
        if defaults.get("mars", False):
            fns = (mars,) + fns
        if clip is not None:
            fns = fns + (apply_to_idx(clip, 2),)
        super().__init__(params, defaults, *fns)


class _ModeSwitching(BaseOpt):
    """Optimizers whose parameters differ between training and evaluation."""

    def eval(self):
        return self.train(False)

    def _switch(self, group, p, z, mode):
        raise NotImplementedError

    def train(self, mode: bool = True):
        z_key = self._find_val_name("z")
        for group in self.param_groups:
            if group.get("train_mode", True) == mode:
                continue
            group["train_mode"] = mode
            for p in group["params"]:
                st = self.state_(p)
                if z_key in st:
                    self._switch(group, p, st[z_key], mode)
        return self


class ScheduleFree(_ModeSwitching):
    """``eval()`` moves the parameters from the gradient-evaluation point ``y`` to the averaged
    iterate ``x``; ``train()`` moves them back."""

    def _switch(self, group, p, z, mode):
        beta1 = utils.get_beta1(group)
        if beta1 <= 0:
            return
        w = 1 - beta1 if mode else 1 - 1 / beta1
        p32 = utils.promote(p.data)
        utils.copy_stochastic_(p.data, p32.lerp(utils.promote(z), w))


class MSAM(_ModeSwitching):
    """``eval()`` swaps the perturbed parameters with the unperturbed copy ``z``."""

    def _switch(self, group, p, z, mode):
        held = p.data.clone()
        utils.copy_stochastic_(p.data, z)
        utils.copy_stochastic_(z, held)
