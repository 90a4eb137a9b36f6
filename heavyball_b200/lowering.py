"""Chain lowering: run a whole transform chain as a handful of sm_100a kernel launches.

``ChainOpt`` offers every step to :func:`try_run`.  The chain is matched against a small set of
*programs*; when one fits and the tensors are eligible, the step executes through
``heavyball_b200.ops`` and the PyTorch definitions in ``chainable`` / ``utils`` are bypassed.
Otherwise ``try_run`` returns ``False`` and the caller runs those definitions (same results up to
rounding-noise layout, which the tests bound).

Programs
--------
``elementwise``   ``[mars] [palm] <rule>``: one launch per group (two with ``caution``: the mask's
                  keep-ratio is a per-tensor reduction over the finished update, so the masked update is
                  parked in a scratch buffer, counted, then applied).
``orthogonal``    ``[mars] [palm] <momentum rule> orthogonalize_update``: momentum launch -> batched
                  Newton–Schulz per shape bucket (tcgen05 GEMM chain) -> parameter-update launch.

``soap``          ``[mars] [palm] scale_by_soap | scale_by_soap_laprop``: gradients -> bucket-major fp32 buffer (one
                  launch) -> per shape bucket the batched stage of ``matrix_stage.SoapBucket`` (projections with the
                  Adam step fused into a GEMM epilogue, statistics with the lerp fused, cached split eigenbases) ->
                  parameter-update launch.  Vectors (no eigenbasis) take one Adam launch.
``psgd``          ``[mars] [palm] [<element-wise rule>] scale_by_psgd | update_by_psgd [trust_region_clip_]``: rule launch
                  into the bucket-major buffer -> ``matrix_stage.PsgdBucket`` (cached ``Q^T Q`` applied with two
                  products, fitting on preconditioner steps) -> update launch with the clip folded in.

State is created by the PyTorch path on the first step of a parameter (``ZeroSlots`` hands out views
of one slab per slot, so buffers of a group are contiguous); lowering engages once all state exists,
and writes the same state keys, so checkpoints do not depend on which path ran.
"""

from __future__ import annotations

import functools
import os
from typing import List, Optional

import torch

from . import chainable as C
from . import matrix_stage, ops, utils
from .utils.tracing import stage as _stage

enabled = os.environ.get("HB200_DISABLE_LOWERING") != "1"

# transform name -> (algo, state slot names in kernel order, needs second beta)
_RULES = {
    "update_by_adam": (ops.ADAM, ("exp_avg", "exp_avg_sq")),
    "update_by_adamc": (ops.ADAM, ("exp_avg", "exp_avg_sq")),
    "scale_by_adam": (ops.ADAM, ("exp_avg", "exp_avg_sq")),
    "update_by_laprop": (ops.LAPROP, ("exp_avg", "exp_avg_sq")),
    "scale_by_laprop": (ops.LAPROP, ("exp_avg", "exp_avg_sq")),
    "update_by_adopt": (ops.ADOPT, ("exp_avg", "exp_avg_sq")),
    "scale_by_adopt": (ops.ADOPT, ("exp_avg", "exp_avg_sq")),
    "update_by_ademamix": (ops.ADEMAMIX, ("exp_avg_fast", "exp_avg_sq", "exp_avg_slow")),
    "scale_by_ademamix": (ops.ADEMAMIX, ("exp_avg_fast", "exp_avg_sq", "exp_avg_slow")),
    "scale_by_exp_avg_sq": (ops.RMSPROP, (None, "exp_avg_sq")),
    "scale_by_unscaled_adam": (ops.UNSCALED_ADAM, ("exp_avg", "exp_avg_sq")),
    "exp_avg": (ops.EXP_AVG, ("exp_avg",)),
    "nesterov_ema": (ops.NESTEROV_EMA, ("momentum",)),
    "heavyball_momentum": (ops.HEAVYBALL, ("momentum",)),
    "nesterov_momentum": (ops.NESTEROV_MOM, ("momentum",)),
    "update_by_nadam": (ops.NADAM, ("exp_avg", "exp_avg_sq")),
}
# gradient clips that become a segmented sum of squares plus a factor applied on load: (mode, over the whole group)
_GRAD_CLIPS = {
    "l2_clip_": (ops.CLIP_L2, False), "rmsnorm_clip_": (ops.CLIP_RMS, False),
    "global_l2norm_clip": (ops.CLIP_L2, True), "global_rmsnorm_clip": (ops.CLIP_RMS, True),
}  # fmt: skip


_SOAP_INNER = {"scale_by_soap": "adam", "scale_by_soap_laprop": "laprop"}
# name -> (writes the parameter itself, fits after applying)
_PSGD_STAGES = {
    "scale_by_psgd": (False, False), "update_by_psgd": (True, False),
    "scale_by_delayed_psgd": (False, True), "update_by_delayed_psgd": (True, True),
}  # fmt: skip


class _Program:
    __slots__ = ("kind", "mars", "palm", "rule", "ortho", "stage", "stage_kw", "u_op", "gclip", "post", "routes", "workspace",
                 "pre_project", "after", "stateless")

    def __init__(self, kind, mars, palm, rule, ortho=None, stage=None, stage_kw=None, u_op=0, gclip=None, post=None,
                 routes=None):  # fmt: skip
        self.kind, self.mars, self.palm, self.rule, self.ortho = kind, mars, palm, rule, ortho
        self.stage, self.stage_kw, self.u_op = stage, stage_kw or {}, u_op
        self.gclip = gclip  # (mode, global) of a leading gradient clip, or None
        self.post = post  # transform that consumes the rule's output inside the same launch (schedule-free)
        self.routes = routes  # kind "route": [(predicate or None for the default, sub-program)]
        self.workspace = {}
        self.pre_project = False  # OrthoGrad on the gradient before the rule (dot products, then folded into the load)
        self.after = None  # what happens to the rule's output in a second launch: ("sign", graft) or ("project",)
        self.stateless = ()  # transforms of the chain that keep no state but still mark themselves as run


def _unwrap(fn):
    """``(transform, bound keyword arguments)`` of a chain entry that may be a ``functools.partial``."""
    if isinstance(fn, functools.partial) and not fn.args:
        return fn.func, dict(fn.keywords)
    return fn, {}


def _match(fns) -> Optional[_Program]:
    fns = list(fns)
    mars = palm = None
    if fns and isinstance(fns[0], C.FunctionTransform) and fns[0].fn_name == "mars":
        mars = fns.pop(0)
    gclip = None
    clip_fn = getattr(fns[0], "wrapped_fn", None) if fns else None
    if clip_fn is not None and fns[0].__name__.endswith("_to_2") and getattr(utils, getattr(clip_fn, "__name__", ""), None) is clip_fn:
        if clip_fn.__name__ in _GRAD_CLIPS and mars is None:  # the norm is taken of the update the rule sees
            gclip = _GRAD_CLIPS[clip_fn.__name__]
            fns.pop(0)
    if fns and getattr(fns[0], "__name__", "") == "palm_beta2" and not isinstance(fns[0], C.FunctionTransform):
        palm = fns.pop(0)
    if not fns:
        return None
    if isinstance(fns[-1], C.Route) and mars is None and gclip is None and not any(isinstance(f, C.Route) for f in fns[:-1]):
        shared, router = fns[:-1], fns[-1]  # transforms in front of the router run in every branch
        routes = []
        for pred, sub in [*router.routes, (None, router.default)]:
            if sub is None:
                return None
            inner = _match([*shared, *sub])
            if inner is None or inner.kind == "route" or inner.palm is not None:
                return None
            routes.append((pred, inner))
        return _Program("route", None, palm, None, routes=routes)
    prog = _match_tail(fns, mars, palm)
    if prog is not None and gclip is not None:
        if prog.kind not in ("elementwise", "orthogonal") or prog.pre_project or prog.after is not None:
            return None
        prog.gclip = gclip
    return prog


def _match_tail(fns, mars, palm) -> Optional[_Program]:
    u_op = 0
    if getattr(fns[-1], "wrapped_fn", None) is utils.trust_region_clip_ and fns[-1].__name__.endswith("_to_2"):
        fns.pop()
        u_op = 1
    pairs = [_unwrap(f) for f in fns]
    if not pairs or not all(isinstance(f, C.FunctionTransform) for f, _ in pairs):
        return None
    last, last_kw = pairs[-1]
    if last.fn_name in _PSGD_STAGES and len(pairs) <= 2:
        rule = None
        if len(pairs) == 2:
            rule, rule_kw = pairs[0]
            if rule.fn_name not in _RULES or rule_kw or rule.fn_name.startswith("update_by"):
                return None
        if last_kw.get("cached", False):
            return None
        return _Program("psgd", mars, palm, rule, stage=last, stage_kw=last_kw, u_op=u_op)
    if len(pairs) >= 2 and pairs[-1][0].fn_name == "apply_update" and not pairs[-1][1]:
        pairs = pairs[:-1]  # the parameter update every lowered program ends with
    if u_op == 0 and len(pairs) == 2 and mars is None:
        (first, first_kw), (second, second_kw) = pairs
        if (second.fn_name in ("update_by_msam", "update_by_hyperball") and first.fn_name == "scale_by_exp_avg_sq"
                and not first_kw and not second_kw):  # fmt: skip
            prog = _Program("elementwise", mars, palm, first, None)
            prog.after = ("msam" if second.fn_name == "update_by_msam" else "hyperball", second)
            prog.stateless = ()
            return prog
        if second.fn_name == "sign" and not first_kw and first.fn_name in _RULES and not first.fn_name.startswith("update_by"):
            if set(second_kw) <= {"graft"}:
                prog = _Program("elementwise", mars, palm, first, None)
                prog.after = ("sign", bool(second_kw.get("graft", True)))
                prog.stateless = (second,)
                return prog
        if not first_kw and not second_kw:
            if second.fn_name == "orthogonalize_grad_to_param" and first.fn_name in _RULES and not first.fn_name.startswith("update_by"):
                prog = _Program("elementwise", mars, palm, first, None)
                prog.after = ("project",)
                prog.stateless = (second,)
                return prog
            if first.fn_name == "orthogonalize_grad_to_param" and second.fn_name in _RULES:
                prog = _Program("elementwise", mars, palm, second, None)
                prog.pre_project = True
                prog.stateless = (first,)
                return prog
    if u_op or any(kw for _, kw in pairs):
        return None
    fns = [f for f, _ in pairs]
    rule = fns[0]
    if len(fns) == 1 and rule.fn_name in _SOAP_INNER:
        return _Program("soap", mars, palm, None, stage=rule)
    if rule.fn_name not in _RULES:
        return None
    if len(fns) == 1:
        return _Program("elementwise", mars, palm, rule, None)
    if len(fns) == 2 and rule.fn_name == "scale_by_exp_avg_sq" and fns[1].fn_name == "update_by_schedule_free" and mars is None:
        return _Program("elementwise", mars, palm, rule, None, post=fns[1])
    if len(fns) == 2 and fns[1].fn_name == "orthogonalize_update":
        return _Program("orthogonal", mars, palm, rule, fns[1])
    return None


def _program(opt) -> Optional[_Program]:
    cached = opt._lowered
    if cached is None:
        cached = opt._lowered = _match(opt.fns) or False
    return cached or None


def describe(opt) -> str:
    """One line on what runs the chain of ``opt``: the lowered program (kernel launches) or the PyTorch definitions.

    ``"elementwise(update_by_adam)"``, ``"orthogonal(heavyball_momentum)"``, ``"soap(adam)"``, ``"psgd(update_by_psgd)"``,
    ``"route[orthogonal(nesterov_ema) | elementwise(update_by_adam)]"``, or ``"not lowered"``.
    """

    def one(prog):
        if prog.kind == "route":
            return "route[" + " | ".join(one(sub) for _, sub in prog.routes) + "]"
        if prog.kind == "soap":
            inner = _SOAP_INNER[prog.stage.fn_name]
        elif prog.kind == "psgd":
            inner = prog.stage.fn_name if prog.rule is None else f"{prog.rule.fn_name} -> {prog.stage.fn_name}"
        else:
            inner = prog.rule.fn_name
        extra = [name for name, on in (("mars", prog.mars), ("palm", prog.palm), ("grad_clip", prog.gclip),
                                       ("trust_region", prog.u_op), ("schedule_free", prog.post),
                                       ("orthograd", prog.pre_project), (prog.after[0] if prog.after else "", prog.after)) if on]  # fmt: skip
        return f"{prog.kind}({inner})" + ("".join(f" +{e}" for e in extra))

    prog = _program(opt)
    return "not lowered" if prog is None else one(prog)


_MARKED_LAYERS = (C.ZeroSlots, C.CopySlots, C.InitSlots, C.Tag, C.PerTensor, C.Warmup)


def _mark_initialized(tr: C.FunctionTransform, st: dict):
    """Records in the view's state that the transform's layers have run (what the layers do themselves on the PyTorch
    path).  Called for every state of every step, so the layer walk is done once per transform and a state that
    already carries the marks costs one set comparison."""
    indices = tr.__dict__.get("_mark_indices")
    if indices is None:
        indices = tr.__dict__["_mark_indices"] = frozenset(
            layer.index for layer in tr.layers if isinstance(layer, _MARKED_LAYERS)
        )
    done = st.get("is_initialized")
    if isinstance(done, set) and indices <= done:
        return
    for index in indices:
        C._mark(st, index)


def _state_ready(tr: C.FunctionTransform, states: List[dict], ecc: bool) -> bool:
    keys = [k for layer in tr.layers if not isinstance(layer, C.AccumSlots) for k in layer.keys.values()]
    warm = [(layer.counter, len(layer.warmup_fns)) for layer in tr.layers if isinstance(layer, C.Warmup)]
    for st in states:
        for k in keys:
            if k not in st or (ecc and k + "::ecc" not in st):
                return False
        for counter, need in warm:
            if st.get(counter, 0) < need:
                return False
    return True


def _state_keys_present(tr: C.FunctionTransform, states: List[dict], ecc: bool) -> bool:
    keys = [k for layer in tr.layers if not isinstance(layer, C.AccumSlots) for k in layer.keys.values()]
    return all(k in st and (not ecc or k + "::ecc" in st) for st in states for k in keys)


def _eligible(t: torch.Tensor) -> bool:
    return t.is_cuda and t.is_contiguous() and t.dtype in (torch.float32, torch.bfloat16, torch.float16)


def _group_index(opt, group) -> int:
    for i, g in enumerate(opt.param_groups):
        if g is group:
            return i
    return 0


def _seed(opt, group, launch: int) -> int:
    """Philox seed of one launch.  Built only from values that are equal on every rank and in every run that
    starts from the same ``torch.manual_seed``: the generator's seed at the optimizer's first step, the position of
    the group in ``param_groups``, the step count and the launch number within the step.  Replicated execution
    (every rank updating the same elements) therefore draws the same rounding noise everywhere."""
    base = getattr(opt, "_rng_base", None)
    if base is None:
        base = opt._rng_base = torch.initial_seed() & 0xFFFFFFFFFFFF
    return (
        base * 0x9E3779B1 + group["step"] * 1315423911 + launch * 2654435761 + _group_index(opt, group) * 40503
    ) & 0x7FFFFFFFFFFFFFFF


def _slots(tr, states, names, ecc: bool):
    """Kernel slot lists (s0, s0e, s1, s1e, s2, s2e) for a rule transform."""
    out = []
    for n in names + (None,) * (3 - len(names)):
        if n is None:
            out += [[], []]
            continue
        key = tr._val_names[n]
        out.append([st[key] for st in states])
        out.append([st[key + "::ecc"] for st in states] if ecc else [])
    return out


def _rule_scalars(rule_name, group):
    """Host-side coefficients, computed exactly as the PyTorch definitions do."""
    step = group["step"]
    cfg = {"eps": group["eps"]}
    algo = _RULES[rule_name][0]
    if algo in (ops.ADAM, ops.LAPROP, ops.UNSCALED_ADAM):
        cfg["b1"] = utils.beta_debias(utils.get_beta1(group), step)
        cfg["b2"] = utils.beta_debias(utils.get_beta2(group), step)
    elif algo == ops.ADOPT:
        cfg["b1"] = utils.beta_debias(utils.get_beta1(group), step - 1)
        cfg["b3"] = 1 - utils.beta_debias(utils.get_beta2(group), step)
    elif algo == ops.ADEMAMIX:
        b1, b2, b3, alpha = utils._compute_ademamix_hparams(
            group["betas"], step, group["alpha"], group.get("beta3_warmup"), group.get("alpha_warmup")
        )
        cfg.update(b1=utils.beta_debias(b1, step), b2=utils.beta_debias(b2, step), b3=b3, alpha=alpha)
    elif algo == ops.RMSPROP:
        cfg["b2"] = utils.beta_debias(utils.get_beta2(group), step)
    elif algo == ops.EXP_AVG:
        cfg["b1"] = utils.beta_debias(utils.get_beta1(group), step)
    else:  # momentum flavours use the raw coefficient
        cfg["b1"] = utils.get_beta1(group)
    return cfg


def _weight_decay(rule_name, group):
    if rule_name == "update_by_adamc":
        return group["lr"] * group["weight_decay"] / group["max_lr"]
    return group["weight_decay"]


def _nadam_scalars(prog, states, group):
    """NAdam's momentum schedule: the running product of ``mu`` is a 0-d state tensor per parameter (all equal).  It
    is advanced on the device with one multi-tensor multiply and mirrored on the host, which is read from the device
    only when the mirror is not from the previous step (first lowered step, or after a checkpoint was loaded)."""
    step = group["step"]
    beta1, beta2 = utils.get_beta1(group), utils.get_beta2(group)
    mu, mu_next = utils._nadam_moments(beta1, step, group["momentum_decay"])
    key = prog.rule._val_names["mu_product"]
    cache_key = ("mu_product", id(group))
    held = prog.workspace.get(cache_key)
    product = held[1] if held is not None and held[0] == step - 1 else float(states[0][key])
    product *= mu
    torch._foreach_mul_([st[key] for st in states], mu)
    prog.workspace[cache_key] = (step, product)
    return {
        "eps": group["eps"], "b1": beta1, "b2": utils.beta_debias(beta2, step),
        "b3": (1 - mu) / (1 - product), "alpha": mu_next / (1 - product * mu_next),
    }  # fmt: skip


def _materialize_zero_state(tr: C.FunctionTransform, states, group, params):
    """Allocates the (all-zero) state of a rule without running it; used when gradients must not be
    consumed by the PyTorch path (peer data parallelism reduces them inside the kernels)."""
    for depth, layer in enumerate(tr.layers):
        if isinstance(layer, C.ZeroSlots):
            if len(params) > 1:
                layer._slab_init(states, group, params)
            for st, p in zip(states, params):
                layer.init(st, group, None, None, p)
    for st in states:
        _mark_initialized(tr, st)


def _cut(t, seg):
    return t if seg is None else t.view(-1)[seg[0] : seg[1]]


_NS_WORKSPACE_BYTES = 2 << 30  # Newton–Schulz work copies per call; larger buckets are processed in chunks
cpu_programs = False  # tests: run the staged programs with PyTorch products on CPU to check their logic


def try_run(opt, states, group, grads, params) -> bool:
    if not enabled:
        return False
    on_gpu = params[0].is_cuda and ops.available()
    if not on_gpu and not (cpu_programs and not params[0].is_cuda):
        return False
    prog = _program(opt)
    if prog is None:
        return False
    if prog.kind == "route":
        return _run_route(opt, prog, states, group, grads, params, on_gpu)
    return _run(opt, prog, states, group, grads, params, on_gpu, False)


def _run_route(opt, prog, states, group, grads, params, on_gpu) -> bool:
    """Every parameter goes through the program of the first route whose predicate accepts it.  All routes are checked
    before any of them runs, so a step is either lowered as a whole or left to the PyTorch definitions as a whole."""
    if getattr(opt, "_peer", None) is not None and opt._peer.plan_for(group) is not None:
        return False
    taken, parts = set(), []
    for pred, sub in prog.routes:
        idx = [i for i, p in enumerate(params) if i not in taken and (pred is None or pred(p))]
        taken.update(idx)
        if idx:
            pick = lambda xs: [xs[i] for i in idx]  # noqa: E731
            parts.append((sub, pick(states), pick(grads), pick(params)))
    if not all(_run(opt, sub, st, group, g, p, on_gpu, True) for sub, st, g, p in parts):
        return False
    if prog.palm is not None:
        prog.palm(None, group, None, None, None)
    for sub, st, g, p in parts:
        if not _run(opt, sub, st, group, g, p, on_gpu, False):
            raise RuntimeError("a routed sub-chain refused to run after it had been accepted")
    return True


def _run(opt, prog, states, group, grads, params, on_gpu, check_only) -> bool:
    if prog.kind in ("soap", "psgd"):
        return _run_precond(opt, prog, states, group, grads, params, on_gpu, check_only)
    if not on_gpu:
        return False
    if not all(_eligible(p) for p in params):
        return False
    ecc_mode, pecc_mode = group.get("ecc"), group.get("param_ecc")
    if prog.kind == "orthogonal" and utils.zeroth_power_mode != "newtonschulz":
        return False
    peer = getattr(opt, "_peer", None)
    plan = peer.plan_for(group) if peer is not None else None
    warming = []
    if plan is not None and not check_only:  # state is created here: the PyTorch path would see unreduced gradients
        for tr in (prog.rule, prog.mars):
            if tr is not None and not _state_keys_present(tr, states, bool(ecc_mode)):
                _materialize_zero_state(tr, states, group, params)
        # a warm-up step (ADOPT seeds its second moment and makes no update) runs through the same kernel below
        warming = [layer for layer in prog.rule.layers if isinstance(layer, C.Warmup)
                   and any(st.get(layer.counter, 0) < len(layer.warmup_fns) for st in states)]  # fmt: skip
        for layer in warming:
            for st in states:
                st[layer.counter] = st.get(layer.counter, 0) + 1
    if not _state_ready(prog.rule, states, bool(ecc_mode)):
        return False
    if prog.mars is not None and not _state_ready(prog.mars, states, bool(ecc_mode)):
        return False
    if pecc_mode and any("param::ecc" not in st for st in states):
        return False
    grads = [g if g.is_contiguous() else g.contiguous() for g in grads]
    gdt = grads[0].dtype
    if any(g.dtype != gdt or not g.is_cuda for g in grads) or gdt not in (torch.float32, torch.bfloat16, torch.float16):
        return False
    pdt = params[0].dtype
    if any(p.dtype != pdt for p in params):
        return False
    rule_name = prog.rule.fn_name
    algo, names = _RULES[rule_name]
    key0 = prog.rule._val_names[next(n for n in names if n is not None)]
    sdt = states[0][key0].dtype
    if any(st[key0].dtype != sdt for st in states):
        return False
    post = prog.post
    if post is not None:  # schedule-free: point-wise, but its caution rescaling would need a second pass
        if group["caution"] or plan is not None or ecc_mode or pecc_mode or not _state_ready(post, states, False):
            return False
        if any(st[post._val_names["z"]].dtype != sdt for st in states):
            return False
    if algo == ops.NADAM and group["weight_decay"] != 0 and not group.get("decoupled_weight_decay", False):
        return False  # L2-style decay enters the moments: left to the PyTorch definition
    if prog.gclip is not None and plan is not None:
        return False  # the clip needs the norm of the reduced gradient, which peer kernels never materialise
    if prog.pre_project or prog.after is not None:
        # per-tensor dot products / norms of whole tensors: not under a partition plan; the projection reads the
        # parameter next to the gradient (one dtype for the dot-product kernel); caution would need a third pass
        if plan is not None or pecc_mode or pdt != torch.float32 or (prog.pre_project and gdt != pdt):
            return False
        if prog.after is not None and group["caution"]:
            return False
        if prog.after is not None and prog.after[0] in ("msam", "hyperball"):
            consumer = prog.after[1]
            if ecc_mode or sdt != torch.float32 or not _state_ready(consumer, states, False):
                return False
        if (prog.pre_project or (prog.after is not None and prog.after[0] == "project")) and any(p.numel() < 16 for p in params):
            # the norm of the projected vector is taken from the dot products (x.x - 2 c p.x + c^2 p.p), which cancels
            # completely when x is parallel to p - always the case for a one-element tensor
            return False
    if check_only:
        return True

    if prog.palm is not None:
        prog.palm(None, group, None, None, None)
    for st in states:
        _mark_initialized(prog.rule, st)
        if prog.mars is not None:
            _mark_initialized(prog.mars, st)
        if prog.ortho is not None:
            _mark_initialized(prog.ortho, st)
        if post is not None:
            _mark_initialized(post, st)
        for tr in prog.stateless:
            _mark_initialized(tr, st)
        if prog.after is not None and prog.after[0] in ("msam", "hyperball"):
            _mark_initialized(prog.after[1], st)

    # ---- selection: everything (single process / replicated) or this rank's share (peer data parallelism)
    peer_in, peer_out = {}, {}
    if plan is not None:
        by_id = {id(p): i for i, p in enumerate(params)}
        group_pos = {id(p): j for j, p in enumerate(group["params"])}
        pos_to_local = {group_pos[pid]: i for pid, i in by_id.items() if pid in group_pos}
        missing = [j for j, _ in plan["sel"] if j not in pos_to_local]
        if missing and all(group["params"][j].grad is not None for j in missing):
            raise RuntimeError("peer data parallelism: the step's parameters do not match the partition plan of their group")
        sel = [(pos_to_local[j], seg) for j, seg in plan["sel"] if j in pos_to_local]
        args = peer.peer_args(params[0].dtype)
        peer_in = {"g_delta": args["g_delta"], "g_scale": args["g_scale"], "g_mc_delta": args["g_mc_delta"]}
        peer_out = {"p_delta": args["p_delta"], "p_mc_delta": args["p_mc_delta"]}
    else:
        sel = [(i, None) for i in range(len(params))]
    pick = lambda xs: [_cut(xs[i], seg) for i, seg in sel] if len(xs) else []  # noqa: E731
    params_v, grads_v = pick(params), pick(grads)
    if plan is not None:  # the kernels add cross-GPU offsets to these addresses: never launch on anything but slab views
        for (i, seg), pv, gv in zip(sel, params_v, grads_v):
            peer.validate(params[i], seg, pv, gv)
    sub_states = [states[i] for i, _ in sel]
    s0, s0e, s1, s1e, s2, s2e = (
        [_cut(t, seg) for t, (_, seg) in zip(lst, sel)] for lst in _slots(prog.rule, sub_states, names, bool(ecc_mode))
    )
    base = dict(
        dt_g=ops.dtype_code(grads[0]), dt_s=ops.dtype_code(states[0][key0], ecc_mode),
        dt_p=ops.dtype_code(params[0], pecc_mode), n_state=len(names), algo=algo,
    )  # fmt: skip
    base.update(_nadam_scalars(prog, states, group) if algo == ops.NADAM else _rule_scalars(rule_name, group))
    if prog.gclip is not None:  # F2 pre-pass: per-tensor sums of squares, folded to one value for the global clips
        mode, whole_group = prog.gclip
        gsq = ops.sumsq(grads_v)
        if whole_group:
            gsq = gsq.double().sum().float().reshape(1)
            base["g_clip_numel"] = float(sum(g.numel() for g in grads_v))
        base.update(gsq=gsq, g_clip_mode=mode, g_clip_at=1.0)
    mars_kw = {}
    if prog.mars is not None:
        mkey = prog.mars._val_names["mars_old_grad"]
        gamma, beta1 = utils.get_beta1(group), group["mars_gamma"]  # argument order of the transform
        mars_kw = dict(
            mars=[_cut(st[mkey], seg) for st, (_, seg) in zip(sub_states, sel)],
            marse=[_cut(st[mkey + "::ecc"], seg) for st, (_, seg) in zip(sub_states, sel)] if ecc_mode else [],
            mars_a=-gamma * beta1 / (1 - beta1),
        )  # fmt: skip
    pe = [_cut(st["param::ecc"], seg) for st, (_, seg) in zip(sub_states, sel)] if pecc_mode else []
    epilogue = dict(
        lr=group["lr"], wd=_weight_decay(rule_name, group), cautious_wd=int(bool(group.get("cautious_weight_decay", False)))
    )
    caution = bool(group["caution"])
    if warming:  # seed the second moment from this gradient; moments' first slot and the parameters stay as they are
        base.update(b1=1.0, b3=1.0)
        epilogue.update(lr=0.0, wd=0.0)
        caution = False
    launch = ops.fused_chain
    if not params_v:
        return True  # this rank owns nothing in this group

    if prog.kind == "elementwise" and post is not None:
        step = group["step"]
        if group.get("_sf_step") != step:  # the running weight sum advances once per optimizer step
            group["weight_sum"] = group.get("weight_sum", 0) + C._sf_weight(group)
            group["_sf_step"] = step
        total = group["weight_sum"]
        ckp1 = C._sf_weight(group) / total if total != 0 else 0
        z = [_cut(st[post._val_names["z"]], seg) for st, (_, seg) in zip(sub_states, sel)]
        base.update(b3=ckp1, alpha=utils.get_beta1(group))
        launch(p=params_v, g=grads_v, s0=s0, s1=s1, s2=z, out_mode=ops.OUT_SCHEDULE_FREE, seed=_seed(opt, group, 0),
               **base, **epilogue)  # fmt: skip
        return True
    if prog.kind == "elementwise" and prog.pre_project:
        # OrthoGrad: g <- graft(g, g - (w.g / (w.w + eps)) w); the three dot products of every tensor come from one
        # segmented reduction, the projection itself happens on load inside the rule's launch
        n = len(params_v)
        dots = ops.dot(params_v + params_v + grads_v, grads_v + params_v + grads_v).view(3, n).t().contiguous()
        base.update(gsq=dots, gsq_stride=3, g_clip_mode=ops.CLIP_ORTHO, g_clip_at=group["eps"], g_clip_numel=1.0)
    if prog.kind == "elementwise" and prog.after is not None and prog.after[0] == "msam":
        # Momentum-SAM: z holds the unperturbed weights, the parameter sits at the ascent point z - rho m / |m|.
        # Launch one advances second moment, momentum and z and sums m^2 per tensor; then p <- z, p -= (rho / |m|) m.
        consumer = prog.after[1]
        m = [st[consumer._val_names["exp_avg"]] for st in sub_states]
        z = [st[consumer._val_names["z"]] for st in sub_states]
        sums = torch.zeros(len(params_v), dtype=torch.float32, device=params[0].device)
        launch(g=grads_v, s0=m, s1=s1, s2=z, out_mode=ops.OUT_UPDATE, dt_u=ops.NONE, scale=sums, accum_sumsq=1,
               post_state=ops.POST_MSAM, seed=_seed(opt, group, 0),
               **{**base, "n_state": 3, "b3": utils.beta_debias(utils.get_beta1(group), group["step"])}, **epilogue)  # fmt: skip
        coef = sums.sqrt_().clamp_(min=1e-8).reciprocal_().mul_(group["sam_step_size"])
        torch._foreach_copy_(params_v, z)
        launch(p=params_v, u=m, scale=coef, use_tensor_scale=1, algo=ops.IDENTITY, u_is_input=1, out_mode=ops.OUT_PARAM,
               dt_u=ops.dtype_code(m[0]), dt_p=base["dt_p"], dt_g=ops.NONE, dt_s=ops.NONE, lr=1.0, wd=0.0,
               seed=_seed(opt, group, 1))  # fmt: skip
        return True
    if prog.kind == "elementwise" and prog.after is not None and prog.after[0] == "hyperball":
        # u <- u + p d;  p <- p - lr n0 u / |u|;  p <- p n0 / |p|   (n0: the tensor's norm at initialisation)
        consumer = prog.after[1]
        n0 = torch.stack([st[consumer._val_names["init_norm"]].to(torch.float32).reshape(()) for st in sub_states])
        scratch = _scratch(prog, params_v)
        sums = torch.zeros(len(params_v), dtype=torch.float32, device=params[0].device)
        decay = dict(post_state=ops.POST_DECAY_IN, p=params_v, wd=epilogue["wd"], cautious_wd=epilogue["cautious_wd"]) \
            if epilogue["wd"] != 0 else {}  # fmt: skip
        launch(g=grads_v, u=scratch, s0=s0, s0e=s0e, s1=s1, s1e=s1e, s2=s2, s2e=s2e, out_mode=ops.OUT_UPDATE, dt_u=ops.F32,
               scale=sums, accum_sumsq=1, seed=_seed(opt, group, 0), **base, **decay)  # fmt: skip
        coef = n0 / sums.sqrt_().clamp_(min=1e-12)
        launch(p=params_v, u=scratch, scale=coef, use_tensor_scale=1, algo=ops.IDENTITY, u_is_input=1, out_mode=ops.OUT_PARAM,
               dt_u=ops.F32, dt_p=base["dt_p"], dt_g=ops.NONE, dt_s=ops.NONE, lr=group["lr"], wd=0.0,
               seed=_seed(opt, group, 1))  # fmt: skip
        # back onto the sphere: p <- p s with s = n0 / |p|, written as p - (1 - s) p so the same kernel does it
        shrink = 1.0 - n0 / ops.sumsq(params_v).sqrt_().clamp_(min=1e-12)
        launch(p=params_v, u=params_v, scale=shrink, use_tensor_scale=1, algo=ops.IDENTITY, u_is_input=1,
               out_mode=ops.OUT_PARAM, dt_u=base["dt_p"], dt_p=base["dt_p"], dt_g=ops.NONE, dt_s=ops.NONE, lr=1.0, wd=0.0,
               seed=_seed(opt, group, 2))  # fmt: skip
        return True
    if prog.kind == "elementwise" and prog.after is not None:
        n, dev = len(params_v), params[0].device
        scratch = _scratch(prog, params_v)
        second = dict(p=params_v, u=scratch, algo=ops.IDENTITY, u_is_input=1, out_mode=ops.OUT_PARAM, dt_u=ops.F32,
                      dt_p=base["dt_p"], dt_g=ops.NONE, dt_s=ops.NONE, seed=_seed(opt, group, 1), **epilogue)  # fmt: skip
        if prog.after[0] == "sign":
            sums = torch.zeros(n, 2, dtype=torch.float32, device=dev)  # per tensor: sum u^2, number of non-zero u
            launch(g=grads_v, u=scratch, s0=s0, s0e=s0e, s1=s1, s1e=s1e, s2=s2, s2e=s2e, out_mode=ops.OUT_UPDATE, dt_u=ops.F32,
                   scale=sums, scale_stride=2, accum_sumsq=2, seed=_seed(opt, group, 0), **base)  # fmt: skip
            launch(scale=sums, scale_stride=2, u_op=ops.UOP_SIGN_GRAFT if prog.after[1] else ops.UOP_SIGN, **second)
        else:
            launch(g=grads_v, u=scratch, s0=s0, s0e=s0e, s1=s1, s1e=s1e, s2=s2, s2e=s2e, out_mode=ops.OUT_UPDATE, dt_u=ops.F32,
                   seed=_seed(opt, group, 0), **base)  # fmt: skip
            dots = ops.dot(params_v + params_v + scratch, scratch + params_v + scratch).view(3, n).t().contiguous()
            launch(gsq=dots, gsq_stride=3, g_clip_mode=ops.CLIP_ORTHO, g_clip_at=group["eps"], g_clip_numel=1.0, **second)
        return True
    if prog.kind == "elementwise":
        if not caution:
            launch(p=params_v, pe=pe, g=grads_v, s0=s0, s0e=s0e, s1=s1, s1e=s1e, s2=s2, s2e=s2e, out_mode=ops.OUT_PARAM,
                   seed=_seed(opt, group, 0), **base, **epilogue, **mars_kw, **peer_in, **peer_out)  # fmt: skip
            return True
        scratch = _scratch(prog, params_v)
        masked = torch.zeros(len(params_v), dtype=torch.int32, device=params[0].device)
        launch(g=grads_v, u=scratch, s0=s0, s0e=s0e, s1=s1, s1e=s1e, s2=s2, s2e=s2e, masked=masked, count_caution=1,
               out_mode=ops.OUT_UPDATE, dt_u=ops.F32, seed=_seed(opt, group, 0), **base, **mars_kw, **peer_in,
               **({"p": params_v} if prog.pre_project else {}))  # fmt: skip
        ops.fused_chain(p=params_v, pe=pe, u=scratch, masked=masked, algo=ops.IDENTITY, u_is_input=1, caution_apply=1,
                        out_mode=ops.OUT_PARAM, dt_u=ops.F32, dt_p=base["dt_p"], dt_g=ops.NONE, dt_s=ops.NONE,
                        seed=_seed(opt, group, 1), **epilogue, **peer_out)  # fmt: skip
        return True

    # ---- orthogonal program: momentum -> Newton–Schulz per shape bucket -> parameter update
    # updates live bucket-major (same-shape matrices adjacent), so a bucket is one (B, R, C) tensor and the
    # iteration writes its result over its own input: no second buffer of the group's size
    layout, scratch, _ = _bucket_layout(prog, params_v)
    dev = params[0].device
    sq = torch.zeros(len(scratch), dtype=torch.float32, device=dev)  # squared norms, accumulated by the momentum kernel
    with _stage("momentum"):
        launch(g=grads_v, u=scratch, s0=s0, s0e=s0e, s1=s1, s1e=s1e, s2=s2, s2e=s2e, out_mode=ops.OUT_UPDATE, dt_u=ops.F32,
               scale=sq, accum_sumsq=1, seed=_seed(opt, group, 0), **base, **mars_kw, **peer_in)  # fmt: skip
    scale_mode = "scale"
    final = list(scratch)
    buckets = [(shape, idx, U) for shape, idx, U, _ in layout if len(shape) >= 2]
    # shape buckets are independent chains of small launches: run them on side streams so they share the GPU
    main = torch.cuda.current_stream(dev)
    streams = prog.workspace.get("streams")
    if streams is None:
        streams = prog.workspace["streams"] = [torch.cuda.Stream(device=dev) for _ in range(4)]
    ready = torch.cuda.Event()
    ready.record(main)
    used = []
    for k, (shape, idx, U) in enumerate(buckets):
        R, Cc = shape[0], U[0].numel() // shape[0]
        U3 = U.view(len(idx), R, Cc)
        if not ops.ns_supported(R, Cc):
            for b in range(len(idx)):
                utils.inplace_orthogonal_(U3[b], out=U3[b], scale_mode=scale_mode)
            continue
        sel_idx = prog.workspace.get(("idx", R, Cc, tuple(idx)))
        if sel_idx is None:
            sel_idx = prog.workspace[("idx", R, Cc, tuple(idx))] = torch.tensor(idx, dtype=torch.long, device=dev)
        side = streams[k % len(streams)] if len(buckets) > 1 else main
        if side is not main:
            side.wait_event(ready)
            used.append(side)
        chunk = max(1, _NS_WORKSPACE_BYTES // (R * Cc * 8))  # four bf16 work copies per matrix
        with torch.cuda.stream(side), _stage(f"ns/{R}x{Cc}"):
            norms = sq.index_select(0, sel_idx)
            for c0 in range(0, len(idx), chunk):
                c1 = min(len(idx), c0 + chunk)
                ops.newton_schulz_batched(
                    list(U3[c0:c1].unbind(0)), utils.NS5_COEFFS, out=U3[c0:c1], out_scale=max(1, R / Cc) ** 0.5,
                    seed=_seed(opt, group, 2 + len(final) + R + c0), sumsq=norms[c0:c1],
                )
    for side in used:
        main.wait_stream(side)
    with _stage("update"):
        _orthogonal_update(opt, group, caution, params_v, grads_v, final, pe, base, epilogue, peer_in, peer_out)
    return True


def _orthogonal_update(opt, group, caution, params_v, grads_v, final, pe, base, epilogue, peer_in, peer_out):
    if caution:
        masked = torch.zeros(len(params_v), dtype=torch.int32, device=params_v[0].device)
        ops.fused_chain(g=grads_v, u=final, masked=masked, algo=ops.IDENTITY, u_is_input=1, count_caution=1,
                        out_mode=ops.OUT_UPDATE, dt_u=ops.F32, dt_g=base["dt_g"], dt_s=ops.NONE, dt_p=ops.NONE,
                        seed=_seed(opt, group, 1), **peer_in)  # fmt: skip
        ops.fused_chain(p=params_v, pe=pe, u=final, masked=masked, algo=ops.IDENTITY, u_is_input=1, caution_apply=1,
                        out_mode=ops.OUT_PARAM, dt_u=ops.F32, dt_p=base["dt_p"], dt_g=ops.NONE, dt_s=ops.NONE,
                        seed=_seed(opt, group, 3), **epilogue, **peer_out)  # fmt: skip
    else:
        ops.fused_chain(p=params_v, pe=pe, u=final, algo=ops.IDENTITY, u_is_input=1, out_mode=ops.OUT_PARAM, dt_u=ops.F32,
                        dt_p=base["dt_p"], dt_g=ops.NONE, dt_s=ops.NONE, seed=_seed(opt, group, 3), **epilogue,
                        **peer_out)  # fmt: skip


def _scratch(prog: _Program, params) -> List[torch.Tensor]:
    """fp32 update buffers, one per parameter, carved from one slab and cached on the program."""
    key = ("u", tuple(p.data_ptr() for p in params))
    hit = prog.workspace.get(key)
    if hit is None:
        sizes = [(p.numel() + 15) // 16 * 16 for p in params]
        slab = torch.empty(sum(sizes), dtype=torch.float32, device=params[0].device)
        hit, off = [], 0
        for p, n in zip(params, sizes):
            hit.append(slab[off : off + p.numel()].view(p.shape))
            off += n
        prog.workspace = {k: v for k, v in prog.workspace.items() if k[0] != "u"}
        prog.workspace[key] = hit
    return hit


# ======================================================================================== SOAP / PSGD programs


def _bucket_layout(prog: _Program, params):
    """Bucket-major fp32 buffers: for every distinct parameter shape one ``(B, *shape)`` input and one output tensor;
    returns ``(buckets, u_views, out_views)`` with per-parameter views in parameter order.  Cached on the program."""
    key = ("layout", tuple(tuple(p.shape) for p in params), params[0].device)
    hit = prog.workspace.get(key)
    if hit is not None:
        return hit
    by_shape = {}
    for i, p in enumerate(params):
        by_shape.setdefault(tuple(p.shape), []).append(i)
    dev = params[0].device
    buckets, u_views, out_views = [], [None] * len(params), [None] * len(params)
    for shape, idx in by_shape.items():
        U = torch.empty((len(idx), *shape), dtype=torch.float32, device=dev)
        O = torch.empty_like(U)
        for b, i in enumerate(idx):
            u_views[i], out_views[i] = U[b], O[b]
        buckets.append((shape, idx, U, O))
    prog.workspace = {k: v for k, v in prog.workspace.items() if k[0] != "layout"}
    hit = prog.workspace[key] = (buckets, u_views, out_views)
    return hit


def _stage_bucket(prog: _Program, group, shape, n: int, make):
    key = ("bucket", _group_key(group), shape, n)
    hit = prog.workspace.get(key)
    if hit is None:
        hit = prog.workspace[key] = make()
    return hit


def _group_key(group):
    return id(group)


def _prime_owned_state(opt, peer, plan, states, group, grads, params):
    """First step of a group whose second-order state is partitioned over the ranks of a data-parallel job.  That state
    is initialised from the gradient (eigenbases of its outer products, the scale of the Kronecker factors), so this one
    step averages the group's gradients with a collective and runs the PyTorch definitions on every rank; afterwards
    the parameters are made identical again and every rank keeps only the state of the matrices it owns."""
    peer.average_gradients(group)
    C.chain(states, group, grads, params, *opt.fns)
    peer.broadcast_parameters(group)
    owned = {j for j, _ in plan["sel"]}
    for j, p in enumerate(group["params"]):
        if j not in owned:
            opt.state.pop(p, None)
    plan["primed"] = True


def _precond_unsupported(opt, prog, group, params) -> bool:
    """Options the staged programs do not cover (the PyTorch definitions handle them)."""
    if group.get("storage_dtype", "float32") != "float32" or group.get("precond_grad_accum", False):
        return True
    if getattr(opt, "hessian_approx", False) or group.get("sqrt", False) or group.get("param_ecc") or group.get("split", False):
        return True
    if prog.kind == "soap" and group.get("ecc"):
        return True
    if prog.kind == "psgd" and (not group.get("momentum_into_precond_update", True) or group.get("q_dtype", "float32") != "float32"):
        return True
    if any(p.dtype != torch.float32 or not p.is_contiguous() for p in params):
        return True
    return False


def _run_precond(opt, prog: _Program, states, group, grads, params, on_gpu: bool, check_only: bool = False) -> bool:
    if _precond_unsupported(opt, prog, group, params):
        return False
    peer = getattr(opt, "_peer", None)
    plan = peer.plan_for(group) if peer is not None else None
    peer_in, peer_out = {}, {}
    if plan is not None:
        if check_only or not on_gpu:
            return False
        if not plan["primed"]:
            _prime_owned_state(opt, peer, plan, states, group, grads, params)
            return True
        # this rank's matrices only: it reduces their gradients on load, runs their matrix stage, and stores the new
        # values into every rank's parameter slab
        pos_of = {p.data_ptr(): j for j, p in enumerate(group["params"])}
        owned = {j for j, _ in plan["sel"]}
        keep = [i for i, p in enumerate(params) if pos_of.get(p.data_ptr()) in owned]
        for i in keep:
            peer.validate(group["params"][pos_of[params[i].data_ptr()]], None, params[i], grads[i])
        states, grads, params = ([xs[i] for i in keep] for xs in (states, grads, params))
        if not params:
            return True
        args = peer.peer_args(params[0].dtype)
        peer_in = {"g_delta": args["g_delta"], "g_scale": args["g_scale"], "g_mc_delta": args["g_mc_delta"]}
        peer_out = {"p_delta": args["p_delta"], "p_mc_delta": args["p_mc_delta"]}
    stage = prog.stage
    ecc_mode = group.get("ecc")
    if not _state_ready(stage, states, False):
        return False  # first step of a parameter: the PyTorch path initialises (and, for SOAP, skips the update)
    for tr in (prog.rule, prog.mars):
        if tr is not None and not _state_ready(tr, states, bool(ecc_mode)):
            return False
    keys = stage._val_names
    if prog.kind == "soap":
        if any(len(st[keys["Q"]]) > 2 or st[keys["exp_avg"]].ndim > 3 for st in states):
            return False  # tensors of order > 2 after dimension merging
    elif any(len(st[keys["Q"]]) > 2 for st in states):
        return False
    grads = [g if g.is_contiguous() else g.contiguous() for g in grads]
    if on_gpu and any(g.dtype != grads[0].dtype or g.dtype not in (torch.float32, torch.bfloat16, torch.float16) for g in grads):
        return False
    if check_only:
        return True

    if prog.palm is not None:
        prog.palm(None, group, None, None, None)
    buckets, u_views, out_views = _bucket_layout(prog, params)
    step = group["step"]
    caution = bool(group["caution"])

    # ---- stage A: gradients -> [mars] -> [rule] -> bucket-major fp32 updates
    if on_gpu:
        kw = dict(dt_g=ops.dtype_code(grads[0]), dt_u=ops.F32, dt_p=ops.NONE, out_mode=ops.OUT_UPDATE, seed=_seed(opt, group, 0))
        if prog.rule is not None:
            algo, names = _RULES[prog.rule.fn_name]
            key0 = prog.rule._val_names[next(n for n in names if n is not None)]
            s0, s0e, s1, s1e, s2, s2e = _slots(prog.rule, states, names, bool(ecc_mode))
            kw.update(algo=algo, n_state=len(names), dt_s=ops.dtype_code(states[0][key0], ecc_mode), s0=s0, s0e=s0e, s1=s1,
                      s1e=s1e, s2=s2, s2e=s2e, **_rule_scalars(prog.rule.fn_name, group))  # fmt: skip
        else:
            kw.update(algo=ops.IDENTITY, n_state=0, dt_s=ops.dtype_code(None))
        if prog.mars is not None:
            mkey = prog.mars._val_names["mars_old_grad"]
            gamma, beta1 = utils.get_beta1(group), group["mars_gamma"]  # argument order of the transform
            if prog.rule is None:
                kw["dt_s"] = ops.dtype_code(states[0][mkey], ecc_mode)
            kw.update(mars=[st[mkey] for st in states], marse=[st[mkey + "::ecc"] for st in states] if ecc_mode else [],
                      mars_a=-gamma * beta1 / (1 - beta1))  # fmt: skip
        ops.fused_chain(g=grads, u=u_views, **kw, **peer_in)
    else:
        upd = [g.float().clone() for g in grads]
        for tr in (prog.mars, prog.rule):
            if tr is not None:
                upd = tr(states, group, upd, grads, params)
        for dst, src in zip(u_views, upd):
            dst.copy_(src.view(dst.shape))

    # ---- stage B: per shape bucket
    if prog.kind == "soap":
        b1 = utils.beta_debias(utils.get_beta1(group), step - 1)
        b2 = utils.beta_debias(utils.get_beta2(group), step - 1)
        stat_w = 1 - utils.beta_debias(group["shampoo_beta"], step)
        vec = []  # members without any eigenbasis: plain Adam / LaProp on the update
        for shape, idx, U, O in buckets:
            members = [states[i] for i in idx]
            if all(q is None for q in members[0][keys["Q"]]):
                vec += idx
                continue
            U3, O3 = (U, O) if U.ndim == 3 else (U.unsqueeze(1), O.unsqueeze(1))
            bucket = _stage_bucket(prog, group, shape, len(idx), lambda: matrix_stage.SoapBucket(keys, _SOAP_INNER[stage.fn_name]))
            with _stage("soap.refresh" if group["is_preconditioning"] else "soap.project"):
                bucket.run(members, U3, O3, group, b1=b1, b2=b2, eps=group["eps"], stat_w=stat_w,
                           refresh=bool(group["is_preconditioning"]))  # fmt: skip
        if vec:
            m = [states[i][keys["exp_avg"]] for i in vec]
            v = [states[i][keys["exp_avg_sq"]] for i in vec]
            if on_gpu:
                algo = ops.ADAM if _SOAP_INNER[stage.fn_name] == "adam" else ops.LAPROP
                ops.fused_chain(g=[u_views[i] for i in vec], u=[out_views[i] for i in vec], s0=m, s1=v, algo=algo, n_state=2,
                                out_mode=ops.OUT_UPDATE, dt_g=ops.F32, dt_u=ops.F32, dt_s=ops.F32, dt_p=ops.NONE, b1=b1, b2=b2,
                                eps=group["eps"], seed=_seed(opt, group, 1))  # fmt: skip
            else:
                fn = utils.adam_ if _SOAP_INNER[stage.fn_name] == "adam" else utils.laprop_
                res = fn(m, v, [u_views[i].clone().view(mm.shape) for i, mm in zip(vec, m)], utils.get_beta1(group),
                         utils.get_beta2(group), step - 1, group["eps"])  # fmt: skip
                for i, r in zip(vec, res):
                    out_views[i].copy_(r.view(out_views[i].shape))
        fused_caution_ref = None
    else:
        fused, delayed = _PSGD_STAGES[stage.fn_name]
        line = bool(group["store_triu_as_line"])
        fit = bool(group["is_preconditioning"])
        if fit:
            group["is_cached"] = False
        for shape, idx, U, O in buckets:
            members = [states[i] for i in idx]
            bucket = _stage_bucket(prog, group, shape, len(idx), lambda: matrix_stage.PsgdBucket(keys, line))
            inner = [len(idx), *(d for d in shape if d != 1)]  # the transform sees size-1 dims squeezed away
            with _stage("psgd.fit" if fit else "psgd.apply"):
                bucket.run(members, U.view(inner), O.view(inner), group, fit=fit, delayed=delayed)
        # the fused form masks against the incoming update, the unfused one against the gradient
        fused_caution_ref = u_views if fused else None

    # ---- stage C: [clip] -> [caution] -> weight decay -> parameter write
    lr, wd = group["lr"], group["weight_decay"]
    cwd = bool(group.get("cautious_weight_decay", False))
    if on_gpu:
        epilogue = dict(lr=lr, wd=wd, cautious_wd=int(cwd))
        common = dict(algo=ops.IDENTITY, u_is_input=1, dt_u=ops.F32, dt_s=ops.NONE)
        if caution:
            ref = fused_caution_ref if fused_caution_ref is not None else grads
            masked = torch.zeros(len(params), dtype=torch.int32, device=params[0].device)
            ref_in = peer_in if ref is grads else {}  # gradients are reduced over the ranks on load, local buffers are not
            ops.fused_chain(g=ref, u=out_views, masked=masked, count_caution=1, out_mode=ops.OUT_UPDATE, dt_g=ops.dtype_code(ref[0]),
                            dt_p=ops.NONE, u_op=prog.u_op, seed=_seed(opt, group, 2), **common, **ref_in)  # fmt: skip
            ops.fused_chain(p=params, u=out_views, masked=masked, caution_apply=1, out_mode=ops.OUT_PARAM, dt_g=ops.NONE,
                            dt_p=ops.dtype_code(params[0]), seed=_seed(opt, group, 3), **common, **epilogue, **peer_out)  # fmt: skip
        else:
            ops.fused_chain(p=params, u=out_views, out_mode=ops.OUT_PARAM, dt_g=ops.NONE, dt_p=ops.dtype_code(params[0]),
                            u_op=prog.u_op, seed=_seed(opt, group, 3), **common, **epilogue, **peer_out)  # fmt: skip
    else:
        final = [o.clone().view(p.shape) for o, p in zip(out_views, params)]
        if prog.u_op:
            utils.trust_region_clip_(final)
        ref = [u.view(p.shape) for u, p in zip(fused_caution_ref, params)] if fused_caution_ref is not None else grads
        utils.update_param_(params, final, lr, wd, caution=caution, cautious_decay=cwd, grad=ref)
    return True
