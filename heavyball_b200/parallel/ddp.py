"""Data-parallel training without a separate gradient all-reduce.

``wrap(model, optimizer)`` re-homes parameters and gradients into two slabs of *symmetric memory*
(every rank can address every other rank's copy over NVLink) and partitions the optimizer work:

* element-wise chains (AdamW, LaProp, ...): the flat element range of a param group is cut into
  ``world`` contiguous pieces; rank ``r`` updates piece ``r`` only.  Its kernel reads the matching
  gradient elements from **all** ranks' slabs (peer loads, summed and scaled by ``1/world`` in
  registers - the reduce-scatter), runs the transform chain on its state, and stores the new
  parameter elements into **all** ranks' slabs (peer stores - the all-gather).  One kernel does the
  collective and the optimizer math; no reduced gradient is ever materialised.
* orthogonalising chains (Muon, MuonLaProp): every matrix has one owner rank (balanced by estimated
  Newton–Schulz cost).  The owner's momentum kernel reduces the gradient from all ranks on load, the
  batched Newton–Schulz runs on the owned matrices only, and the parameter-update kernel stores the
  result into all ranks' slabs.
* anything else (SOAP, PSGD, user chains): gradients of those parameters are averaged with a
  ``torch.distributed`` all-reduce and the optimizer runs replicated, as the reference does under
  ``DistributedDataParallel`` (``examples/ddp_training.py:47-52`` there).

Synchronisation is two epoch-flag barriers per step in symmetric memory (``ops/csrc/peer_sync.cu``):
"my gradients are complete" before the first optimizer kernel and "I am done reading your gradients and
writing your parameters" after the last.  Waits are bounded; :meth:`PeerContext.check` raises if a peer
never arrived.  Every parameter element has exactly one writer, so replicas stay bit-identical.

Optimizer state is partitioned the same way (a rank only advances the state it owns).  Before saving a
checkpoint call ``wrapped.peer.consolidate_state()`` on every rank: it completes the state everywhere, so that
the ``state_dict`` of any one rank is the whole optimizer state.

``mode="nccl"`` (or a single process) falls back to ``DistributedDataParallel``.
"""

from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..utils.tracing import stage as _stage


def _world():
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _inner_optimizers(optimizer):
    return list(getattr(optimizer, "optimizers", None) or [optimizer])


def check_slab_view(what: str, ptr: int, nbytes: int, dtype, slab_ptr: int, slab_bytes: int, slab_dtype,
                    expected_offset_bytes: Optional[int] = None):  # fmt: skip
    """Raises unless ``[ptr, ptr + nbytes)`` lies inside ``[slab_ptr, slab_ptr + slab_bytes)``, has the slab's dtype
    and (when given) starts at the expected byte offset.  The peer kernels add cross-GPU byte offsets to these
    addresses, so a tensor outside its slab would be read or written at an arbitrary address on another GPU."""
    if dtype != slab_dtype:
        raise RuntimeError(
            f"peer data parallelism: {what} has dtype {dtype}, the symmetric slab holds {slab_dtype} "
            "(was the gradient promoted or re-created outside the slab?)"
        )
    if ptr < slab_ptr or ptr + nbytes > slab_ptr + slab_bytes:
        raise RuntimeError(
            f"peer data parallelism: {what} does not live in the symmetric slab (it was re-allocated, e.g. by "
            "`model.zero_grad(set_to_none=True)`, `.contiguous()` or a dtype cast); the step was not launched"
        )
    if expected_offset_bytes is not None and ptr - slab_ptr != expected_offset_bytes:
        raise RuntimeError(f"peer data parallelism: {what} sits at byte {ptr - slab_ptr} of the slab, expected {expected_offset_bytes}")


class PeerContext:
    """Owns the symmetric slabs, the work partition and the step barriers."""

    def __init__(self, model: torch.nn.Module, optimizer, group=None, timeout_s: float = 10.0):
        import torch.distributed._symmetric_memory as symm_mem

        from .. import lowering

        self.group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > ops.load().MAX_WORLD:
            raise ValueError(f"peer data parallelism supports at most {ops.load().MAX_WORLD} ranks per node")
        self.timeout_s = timeout_s
        self.epoch = 0
        self.optimizer = optimizer

        params = [p for p in model.parameters() if p.requires_grad]
        if not params:
            raise ValueError("model has no trainable parameters")
        self.device = params[0].device
        if any(p.device != self.device for p in params):
            raise ValueError("peer data parallelism needs all parameters on one device")
        self.params = params

        # ---- slab layout: one parameter slab and one gradient slab per dtype (error-corrected parameters are 16-bit next
        # to fp32 ones), 16-element aligned segments, identical on every rank
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            try:  # required by older releases, a deprecated no-op in newer ones
                symm_mem.enable_symm_mem_for_group(self.group.group_name)
            except Exception:  # noqa: BLE001
                pass
        self.offsets: Dict[int, int] = {}
        self.slabs: Dict[torch.dtype, dict] = {}
        totals: Dict[torch.dtype, int] = {}
        for p in params:
            self.offsets[id(p)] = totals.get(p.dtype, 0)
            totals[p.dtype] = self.offsets[id(p)] + (p.numel() + 15) // 16 * 16
        self.flags = symm_mem.empty(4 * ops.load().MAX_WORLD, dtype=torch.int32, device=self.device)
        self.flags.zero_()
        self._hdl = [symm_mem.rendezvous(self.flags, self.group)]
        self.f_ptrs = list(self._hdl[0].buffer_ptrs)
        for dtype in sorted(totals, key=str):  # same creation order on every rank
            P = symm_mem.empty(totals[dtype], dtype=dtype, device=self.device)
            G = symm_mem.empty(totals[dtype], dtype=dtype, device=self.device)
            P.zero_()
            G.zero_()
            hp, hg = symm_mem.rendezvous(P, self.group), symm_mem.rendezvous(G, self.group)
            self._hdl += [hp, hg]
            p_ptrs, g_ptrs = list(hp.buffer_ptrs), list(hg.buffer_ptrs)
            # NVSwitch multicast addresses of the two slabs (0 where the fabric has none): reductions and broadcasts then
            # happen inside the switch
            use_mc = os.environ.get("HB200_PEER_MULTIMEM", "1") != "0"
            mc_p = int(getattr(hp, "multicast_ptr", 0) or 0) if use_mc else 0
            mc_g = int(getattr(hg, "multicast_ptr", 0) or 0) if use_mc else 0
            self.slabs[dtype] = {
                "P": P, "G": G,
                "p_delta": [ptr - p_ptrs[self.rank] for ptr in p_ptrs],
                "g_delta": [ptr - g_ptrs[self.rank] for ptr in g_ptrs],
                "p_mc_delta": (mc_p - p_ptrs[self.rank]) if mc_p else 0,
                "g_mc_delta": (mc_g - g_ptrs[self.rank]) if mc_g else 0,
            }  # fmt: skip
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

        with torch.no_grad():
            for p in params:
                P = self.slabs[p.dtype]["P"]
                view = P[self.offsets[id(p)] : self.offsets[id(p)] + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
            for slab in self.slabs.values():
                dist.broadcast(slab["P"], src=dist.get_global_rank(self.group, 0), group=self.group)
        self._attach_grads()

        # ---- which parameters are handled by peer kernels, which by the all-reduce fallback
        self.plans: Dict[int, dict] = {}
        self.fallback_ranges: List[Tuple[torch.dtype, int, int]] = []
        self._optimizers = list(_inner_optimizers(optimizer))
        self.consolidations = 0
        self.stale_state = False  # True between an optimizer step and the next consolidate_state()
        for opt in self._optimizers:
            prog = lowering._program(opt) if hasattr(opt, "_lowered") else None
            kind = None if prog is None else prog.kind
            for g in getattr(opt, "param_groups", []):
                ok = kind in ("elementwise", "orthogonal", "soap", "psgd") and all(id(p) in self.offsets for p in g["params"])
                if ok and (prog.gclip is not None or prog.post is not None):
                    ok = False  # need the norm of the reduced gradient / a second parameter-sized state written everywhere
                if ok and kind in ("soap", "psgd") and lowering._precond_unsupported(opt, prog, g, g["params"]):
                    ok = False
                if ok:
                    # a caution mask is counted per tensor, and a matrix stage needs its whole matrix: whole-tensor
                    # ownership; everything else is cut by element
                    whole = kind != "elementwise" or bool(g.get("caution"))
                    self.plans[id(g)] = self._plan_group(g, kind, whole)
                else:
                    for p in g["params"]:
                        if id(p) in self.offsets:
                            self.fallback_ranges.append((p.dtype, self.offsets[id(p)], p.numel()))
            if hasattr(opt, "consume_grad"):
                opt.consume_grad = False  # gradients live in the slab for the whole run
            opt._peer = self
        self.fallback_ranges = self._coalesce(self.fallback_ranges)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    # ------------------------------------------------------------------ layout helpers
    def _attach_grads(self):
        for p in self.params:
            off = self.offsets[id(p)]
            p.grad = self.slabs[p.dtype]["G"][off : off + p.numel()].view(p.shape)

    def _check_grads_in_slab(self):
        """Backward must have accumulated into the slab views.  A gradient that was set to ``None`` and re-created by
        autograd lives elsewhere; publishing the (zero) slab for it would silently drop that gradient."""
        for p in self.params:
            g = p.grad
            if g is None:
                continue  # parameter unused in this step: its slab range is zero
            G = self.slabs[p.dtype]["G"]
            if g.dtype != p.dtype or g.data_ptr() != G.data_ptr() + self.offsets[id(p)] * G.element_size():
                raise RuntimeError(
                    "peer data parallelism: a parameter's .grad is no longer the symmetric-slab view (it was set to "
                    "None and re-created, cast or replaced).  Use `optimizer.zero_grad()` / `model.zero_grad()` of the "
                    "wrapped objects, which keep the views, and do not replace `.grad`."
                )

    @staticmethod
    def _coalesce(ranges):
        """Merges ``(dtype, offset, length)`` ranges of one slab that touch (up to the alignment padding between them)."""
        out = []
        for dtype, off, n in sorted(ranges, key=lambda r: (str(r[0]), r[1])):
            if out and out[-1][0] == dtype and out[-1][1] + out[-1][2] + 15 >= off:
                out[-1] = (dtype, out[-1][1], off + n - out[-1][1])
            else:
                out.append((dtype, off, n))
        return out

    def _plan_group(self, group, kind, whole):
        ps = group["params"]
        if whole:  # whole tensors, balanced by matrix-stage cost (element count for element-wise chains)
            loads, owned = [0.0] * self.world, []
            order = sorted(range(len(ps)), key=lambda i: -ps[i].numel())
            owner_of = {}
            for i in order:
                p = ps[i]
                side = min(p.shape[0], p[0].numel()) if (p.ndim >= 2 and kind != "elementwise") else 1
                cost = p.numel() * side
                r = min(range(self.world), key=loads.__getitem__)
                loads[r] += cost
                owner_of[i] = r
            owned = [(i, None) for i in range(len(ps)) if owner_of[i] == self.rank]
            return {"kind": kind, "sel": owned, "owner_of": owner_of, "primed": False}
        # flat element partition
        starts, total = [], 0
        for p in ps:
            starts.append(total)
            total += p.numel()
        lo = total * self.rank // self.world
        hi = total * (self.rank + 1) // self.world
        sel = []
        for i, p in enumerate(ps):
            a = max(lo, starts[i]) - starts[i]
            b = min(hi, starts[i] + p.numel()) - starts[i]
            # keep segment starts 16-byte aligned relative to the tensor for every buffer down to the one-byte residuals
            # of error-corrected state: boundaries move down to a multiple of 16 elements
            a = a // 16 * 16 if a > 0 else 0
            b = b // 16 * 16 if b < p.numel() else p.numel()
            if b > a:
                sel.append((i, (a, b)))
        return {"kind": kind, "sel": sel}

    # ------------------------------------------------------------------ step protocol
    def _barrier(self, slot):
        ext = ops.load()
        ext.peer_signal(self.f_ptrs, slot, self.rank, self.epoch)
        ext.peer_wait(self.flags, slot, self.world, self.epoch, self.timeout_s, self.status)
        ops.launch_counter.count += 2

    def begin_step(self):
        """After backward: publish "my gradients are complete" and wait for every peer's."""
        self.epoch += 1
        self.stale_state = True
        self._check_grads_in_slab()
        with _stage("peer.begin"):
            self._barrier(0)
        self._mark(0)
        for dtype, off, n in self.fallback_ranges:
            dist.all_reduce(self.slabs[dtype]["G"][off : off + n], op=dist.ReduceOp.AVG, group=self.group)

    def _mark(self, which: int):
        """Two events per step bracket the work between the barriers (the time a rank spends waiting for the slowest
        peer at the first barrier is arrival skew of the backward passes, not optimizer work)."""
        events = self.__dict__.setdefault("_step_events", [torch.cuda.Event(enable_timing=True) for _ in range(2)])
        events[which].record(torch.cuda.current_stream(self.device))

    def work_ms(self) -> Optional[float]:
        """Device time of the last step between its two barriers (synchronises); ``None`` before the first step."""
        events = self.__dict__.get("_step_events")
        if events is None:
            return None
        events[1].synchronize()
        return events[0].elapsed_time(events[1])

    def end_step(self):
        """After the last optimizer kernel: wait until every peer has finished reading this rank's
        gradients and writing this rank's parameters, then clear the gradient slab."""
        self._mark(1)
        with _stage("peer.end"):
            self._barrier(1)
        for slab in self.slabs.values():
            slab["G"].zero_()  # gradients stay the slab views they were (checked again at the next begin_step)

    def consolidate_state(self):
        """Makes the optimizer state complete on every rank.  Collective: call it on all ranks, e.g. before rank 0
        saves ``optimizer.state_dict()``.

        Under the peer scheme a rank only advances the state (moments, momentum buffers) of the elements or matrices
        it owns; the rest of each state tensor stays as it was.  Here every rank keeps its owned pieces, zeroes the
        others in a scratch copy and the copies are summed across ranks, so afterwards all ranks hold the same,
        complete state (and a checkpoint written by one rank resumes correctly under any world size)."""
        self.consolidations += 1
        self.stale_state = False
        pieces = []  # (tensor, owned ranges): everything this rank must contribute / receive
        for opt in self._optimizers:
            for group in getattr(opt, "param_groups", []):
                plan = self.plans.get(id(group))
                if plan is None:
                    continue  # fallback groups are updated on every rank already
                if plan["kind"] in ("soap", "psgd"):
                    continue  # preconditioner state exists on the owner only (as under sharded training)
                owned = {}
                for i, rng in plan["sel"]:
                    owned.setdefault(i, []).append(rng)
                for i, p in enumerate(group["params"]):
                    for t in self._state_tensors(opt, p):
                        pieces.append((t, owned.get(i, [])))
        by_dtype = {}
        for t, ranges in pieces:
            by_dtype.setdefault(t.dtype, []).append((t, ranges))
        for dtype, items in by_dtype.items():  # one collective per dtype instead of one per state tensor
            flat = torch.zeros(sum(t.numel() for t, _ in items), dtype=dtype, device=self.device)
            off = 0
            for t, ranges in items:
                src = t.reshape(-1)
                for rng in ranges:
                    a, b = (0, src.numel()) if rng is None else rng
                    flat[off + a : off + b] = src[a:b]
                off += t.numel()
            wire = flat if dtype != torch.bfloat16 else flat.float()  # exact: every element has one non-zero contributor
            dist.all_reduce(wire, group=self.group)
            if wire is not flat:
                flat.copy_(wire)
            off = 0
            for t, _ in items:
                t.reshape(-1).copy_(flat[off : off + t.numel()])
                off += t.numel()

    @staticmethod
    def _state_tensors(opt, p):
        """Per-element state of ``p`` (tensors shaped like the parameter), whatever the nesting of the state dict."""
        found, stack = [], [opt.state.get(p, {})]
        while stack:
            node = stack.pop()
            if isinstance(node, dict):
                stack.extend(node.values())
            elif isinstance(node, (list, tuple)):
                stack.extend(node)
            elif isinstance(node, torch.Tensor) and node.numel() == p.numel() and node.numel() > 1 and (
                node.is_floating_point() or node.dtype in (torch.int8, torch.int16)
            ):  # moments, momentum buffers, and the integer residuals of error-corrected state
                found.append(node)
        return found

    def check(self):
        """Host-synchronising health check: raises if a bounded wait expired."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"peer barrier timed out waiting for rank {code - 2} (epoch {self.epoch})")

    def plan_for(self, group) -> Optional[dict]:
        return self.plans.get(id(group))

    def group_ranges(self, group):
        return self._coalesce([(p.dtype, self.offsets[id(p)], p.numel()) for p in group["params"] if id(p) in self.offsets])

    def average_gradients(self, group):
        """Plain collective average of one group's gradient ranges (used for the one step that creates second-order
        state from the reduced gradient with the PyTorch definitions)."""
        for dtype, off, n in self.group_ranges(group):
            dist.all_reduce(self.slabs[dtype]["G"][off : off + n], op=dist.ReduceOp.AVG, group=self.group)

    def broadcast_parameters(self, group, src: int = 0):
        for dtype, off, n in self.group_ranges(group):
            dist.broadcast(self.slabs[dtype]["P"][off : off + n], src=dist.get_global_rank(self.group, src), group=self.group)

    def validate(self, param, seg, p_view, g_view):
        """Checks, on the host and before any launch, that the slices handed to a peer kernel are the slab views
        this context created (same dtype, inside the slab, at the parameter's slab offset plus the slice start)."""
        off = self.offsets.get(id(param))
        if off is None:
            raise RuntimeError("peer data parallelism: parameter is not part of the wrapped model")
        slabs = self.slabs.get(param.dtype)
        if slabs is None:
            raise RuntimeError(f"peer data parallelism: no symmetric slab holds {param.dtype} parameters (dtype changed after wrapping?)")
        start = 0 if seg is None else seg[0]
        for what, view, slab in (("parameter", p_view, slabs["P"]), ("gradient", g_view, slabs["G"])):
            es = slab.element_size()
            check_slab_view(
                what, view.data_ptr(), view.numel() * view.element_size(), view.dtype, slab.data_ptr(),
                slab.numel() * es, slab.dtype, (off + start) * es,
            )  # fmt: skip

    def peer_args(self, dtype):
        slab = self.slabs[dtype]
        return {"g_delta": slab["g_delta"], "g_scale": 1.0 / self.world, "p_delta": slab["p_delta"],
                "g_mc_delta": slab["g_mc_delta"], "p_mc_delta": slab["p_mc_delta"]}  # fmt: skip

    @property
    def multicast(self) -> bool:
        """True when gradient reduction and parameter broadcast go through NVSwitch multicast addresses."""
        return any(slab["g_mc_delta"] or slab["p_mc_delta"] for slab in self.slabs.values())


class _PeerModule(torch.nn.Module):
    """Thin module wrapper; all the work happens in the optimizer step."""

    def __init__(self, module, ctx: PeerContext):
        super().__init__()
        self.module = module
        self.peer = ctx

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)


def wrap(model: torch.nn.Module, optimizer=None, mode: str = "peer", **kwargs):
    """Prepare ``model`` (and ``optimizer``) for data-parallel training on the ranks of the default
    process group.  ``mode="peer"`` (default on CUDA with an optimizer from this package) uses the
    symmetric-memory scheme described in the module docstring; ``mode="nccl"`` uses
    ``DistributedDataParallel``."""
    if _world() == 1:
        return model
    cuda = next(model.parameters()).is_cuda
    if mode == "peer" and cuda and optimizer is not None and ops.available():
        ctx = PeerContext(model, optimizer, **kwargs)
        real_step = optimizer.step

        def step(closure=None):
            ctx.begin_step()
            try:
                return real_step(closure)
            finally:
                ctx.end_step()

        optimizer.step = step
        optimizer.zero_grad = lambda set_to_none=True: None  # the slab is cleared by end_step
        model.zero_grad = lambda set_to_none=True: None  # likewise: dropping .grad would detach it from the slab
        real_state_dict = optimizer.state_dict

        def state_dict(*a, **kw):
            if ctx.stale_state:
                import warnings

                warnings.warn(
                    "optimizer state is partitioned across ranks under peer data parallelism: call "
                    "`model.peer.consolidate_state()` on every rank before `state_dict()`, or this checkpoint holds only "
                    "the part this rank owns", stacklevel=2)
            return real_state_dict(*a, **kw)

        optimizer.state_dict = state_dict
        return _PeerModule(model, ctx)
    from torch.nn.parallel import DistributedDataParallel

    kwargs.pop("timeout_s", None)
    kwargs.setdefault("gradient_as_bucket_view", True)
    return DistributedDataParallel(model, device_ids=[torch.cuda.current_device()] if cuda else None, **kwargs)
