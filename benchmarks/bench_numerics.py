"""Numerics studies of the second-order building blocks, as sub-commands of one script (text tables, optional CSV).

    python benchmarks/bench_numerics.py singular-values      # max/min singular value estimators vs exact SVD
    python benchmarks/bench_numerics.py sv-methods           # cholesky sketch vs power iteration: error and time
    python benchmarks/bench_numerics.py klsoap-pinv          # KL-Shampoo eigenvalue inversion: clamp vs pseudo-inverse
    python benchmarks/bench_numerics.py variance-rotation    # second-moment transport under an eigenbasis rotation
    python benchmarks/bench_numerics.py precond-fitting      # how well PSGD's Kronecker factors fit a known Hessian

Studies of the same questions in the reference: ``benchmarks/bench_singular_values.py``,
``test/benchmark_psgd_lb.py``, ``benchmarks/bench_klsoap_pinv.py``, ``benchmarks/bench_soap_variance_rotation.py``,
``test/benchmark_precond_fitting.py``.  Runs on the GPU when there is one, else on the CPU.
"""

import argparse
import csv
import itertools
import math
import os
import statistics
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from heavyball_b200 import utils  # noqa: E402

DEVICE = "cuda" if torch.cuda.is_available() else "cpu"
DTYPE_NAMES = {torch.bfloat16: "bf16", torch.float32: "fp32", torch.float64: "fp64"}


def _sync():
    if DEVICE == "cuda":
        torch.cuda.synchronize()


def _table(title, header, rows):
    widths = [max(len(str(h)), *(len(str(r[i])) for r in rows)) for i, h in enumerate(header)] if rows else [len(h) for h in header]
    print(f"\n{title}")
    print("  ".join(str(h).ljust(w) for h, w in zip(header, widths)))
    print("-" * (sum(widths) + 2 * (len(widths) - 1)))
    for r in rows:
        print("  ".join(str(c).ljust(w) for c, w in zip(r, widths)))


def _maybe_csv(path, header, rows):
    if not path:
        return
    with open(path, "w", newline="") as fh:
        w = csv.writer(fh)
        w.writerow(header)
        w.writerows(rows)
    print(f"\nwrote {len(rows)} rows to {path}")


def _orthonormal(rows, cols, gen):
    return torch.linalg.qr(torch.randn(rows, cols, generator=gen, dtype=torch.float64)).Q


def _with_spectrum(shape, cond, dtype, symmetric, seed):
    """Matrix with singular values ``cond ** linspace(0, -1)`` and Haar-random singular vectors."""
    gen = torch.Generator().manual_seed(seed)
    m, n = shape
    r = min(m, n)
    left = _orthonormal(m, r, gen)
    right = left if symmetric else _orthonormal(n, r, gen)
    spectrum = torch.tensor(float(cond), dtype=torch.float64) ** torch.linspace(0, -1, r, dtype=torch.float64)
    return ((left * spectrum) @ right.mT).to(dtype).to(DEVICE)


# ------------------------------------------------------------------------------------------ singular values


def cmd_singular_values(args):
    shapes = [(4, 4), (32, 32), (128, 128), (10, 5), (5, 10)]
    conds = [1, 10, 1e4, 1e10, 1e18, 1e30]
    raw = []
    for dtype, iters in itertools.product(DTYPE_NAMES, (0, 5, 20)):
        for name, fn, sym_only in (("max_sv", utils.max_singular_value, False), ("min_sv", utils.min_singular_value, True)):
            for shape, cond in itertools.product(shapes, conds):
                if sym_only and shape[0] != shape[1]:
                    continue
                A = _with_spectrum(shape, cond, dtype, sym_only, seed=0)
                sv = torch.linalg.svdvals(A.double())
                exact = sv.min() if sym_only else sv.max()
                try:
                    got = fn(A, power_iter=iters).double()
                    err = abs(got - exact).item() if exact.abs() < 1e-8 else abs((got - exact) / exact).item()
                    status = "ok"
                except Exception as exc:  # noqa: BLE001 - the failure type is the datum
                    err, status = float("nan"), type(exc).__name__
                raw.append((name, DTYPE_NAMES[dtype], iters, f"{shape[0]}x{shape[1]}", cond, err, status))
    rows = []
    for key, group in itertools.groupby(sorted(raw, key=lambda r: r[:3]), key=lambda r: r[:3]):
        group = list(group)
        good = [r[5] for r in group if r[6] == "ok" and math.isfinite(r[5])]
        rows.append((*key, f"{min(good):.2e}" if good else "-", f"{statistics.median(good):.2e}" if good else "-",
                     f"{max(good):.2e}" if good else "-", len(group) - len(good), len(group)))  # fmt: skip
    _table("relative error of the estimators against exact SVD (fp64)",
           ("function", "dtype", "power_iter", "best", "median", "worst", "failed", "cases"), rows)  # fmt: skip
    _maybe_csv(args.csv, ("function", "dtype", "power_iter", "shape", "cond", "rel_error", "status"), raw)


def cmd_sv_methods(args):
    kinds = {
        "normal": lambda n: torch.randn(n, n),
        "uniform": lambda n: torch.rand(n, n),
        "normal*arange": lambda n: torch.randn(n, n) * torch.arange(n).view(1, -1),
        "exp(normal)": lambda n: torch.randn(n, n).exp(),
        "normal**16": lambda n: torch.randn(n, n) ** 16,
    }
    methods = {
        "exact": lambda x: torch.linalg.matrix_norm(x, ord=2),
        "cholesky": utils.max_singular_value_cholesky,
        "power_iter(0)": lambda x: utils.max_singular_value_power_iter(x, iterations=0),
        "power_iter(2)": lambda x: utils.max_singular_value_power_iter(x, iterations=2),
        "power_iter(6)": lambda x: utils.max_singular_value_power_iter(x, iterations=6),
    }
    torch.manual_seed(0x12378)
    rows = []
    with torch.inference_mode():
        for size in [2**k for k in range(1, int(math.log2(args.max_size)) + 1)]:
            for kind, make in kinds.items():
                mats = [make(size).float().to(DEVICE) for _ in range(args.attempts)]
                exact = None
                for name, fn in methods.items():
                    for x in mats:
                        fn(x)
                    _sync()
                    t0 = time.perf_counter()
                    vals = torch.stack([torch.as_tensor(fn(x)).double().reshape(()).cpu() for x in mats])
                    _sync()
                    dt = (time.perf_counter() - t0) / len(mats)
                    exact = vals if name == "exact" else exact
                    rel = ((vals - exact).abs() / exact.clamp(min=1e-8)).mean().item()
                    rows.append((size, kind, name, f"{rel:.3e}", f"{dt * 1e6:.0f}"))
    _table("largest singular value: estimator error and time", ("n", "matrix", "method", "mean rel err", "us / matrix"), rows)
    _maybe_csv(args.csv, ("n", "matrix", "method", "rel_error", "us"), rows)


# ------------------------------------------------------------------------------------------ KL-Shampoo inverse


def cmd_klsoap_pinv(args):
    """With few accumulated gradients the statistic ``L = mean(G G^T)`` is rank deficient.  ``clamp`` inverts
    ``max(eig, eps)`` (huge weights on the null space), ``pinv`` drops eigenvalues below ``eps * max(eig)``."""

    def invert(method, eig, eps):
        if method == "clamp":
            return eig.clamp_min(eps).reciprocal()
        return torch.where(eig > eps * eig.amax(-1, keepdim=True), eig.reciprocal(), torch.zeros_like(eig))

    apply = lambda Q, w, X: Q @ (w.unsqueeze(-1) * (Q.mT @ X))  # noqa: E731
    raw = []
    for shape, k, eps, dtype, seed in itertools.product(
        [(64, 64), (128, 32), (32, 128), (256, 16), (16, 256)], [0, 1, 2, 4, 8, 16], [1e-12, 1e-8, 1e-4],
        [torch.float32, torch.float64], range(args.seeds),
    ):  # fmt: skip
        gen = torch.Generator().manual_seed(seed)
        grads = [torch.randn(*shape, generator=gen, dtype=dtype) for _ in range(k + 1)]
        L = sum(g @ g.mT for g in grads) / (shape[1] * (k + 1))
        eig64, Q64 = torch.linalg.eigh(L.double())
        eig64 = eig64.clamp_min(0)
        truth = apply(Q64, invert("pinv", eig64, shape[0] * torch.finfo(torch.float64).eps), grads[-1].double()).to(dtype)
        rank = int((eig64 > eig64.max() * 1e-12).sum())
        eig, Q = eig64.to(dtype), Q64.to(dtype)
        rec = [f"{shape[0]}x{shape[1]}", DTYPE_NAMES[dtype], k, eps, seed, f"{rank}/{shape[0]}"]
        for method in ("clamp", "pinv"):
            w = invert(method, eig, eps)
            rec += [w.max().item(), ((apply(Q, w, grads[-1]) - truth).norm() / truth.norm()).item()]
        raw.append(tuple(rec))
    rows = []
    for key, group in itertools.groupby(sorted(raw, key=lambda r: (r[0], r[1], r[2], r[3])), key=lambda r: (r[0], r[1], r[2], r[3])):
        group = list(group)
        rows.append((*key, group[0][5], *(f"{max(g[i] for g in group):.3e}" for i in (6, 7, 8, 9))))
    header = ("shape", "dtype", "k", "eps", "rank/d", "max 1/eig clamp", "err clamp", "max 1/eig pinv", "err pinv")
    _table("inverse of a rank-deficient statistic applied to the last gradient (worst over seeds)", header, rows)
    _maybe_csv(args.csv, ("shape", "dtype", "k", "eps", "seed", "rank", "maxinv_clamp", "err_clamp", "maxinv_pinv", "err_pinv"), raw)


# ------------------------------------------------------------------------------------------ variance transport


def cmd_variance_rotation(args):
    """When the eigenbasis moves from ``Q_old`` to ``Q_new`` the diagonal second moment ``v`` must follow.
    ``none`` keeps it, ``linear`` applies the first moment's rotation, ``hadamard`` applies ``(R * R)^T`` per
    side with ``R = Q_old^T Q_new`` - the diagonal of the rotated covariance, which is what
    ``utils.get_orthogonal_matrix_QR(..., heavy=True)`` does."""
    letters_in, letters_out, letters_mid = "abcd", "efgh", "ABCD"

    def transport(method, v, old, new):
        n = len(old)
        i, o, m = letters_in[:n], letters_out[:n], letters_mid[:n]
        if method == "none":
            return v
        if method == "linear":
            ops = ",".join(a + b for a, b in zip(m, i)) + "," + ",".join(a + b for a, b in zip(m, o))
            return torch.einsum(f"{i},{ops}->{o}", v, *old, *new)
        sq = [(a.mT @ b).square() for a, b in zip(old, new)]
        return torch.einsum(f"{i}," + ",".join(a + b for a, b in zip(i, o)) + f"->{o}", v, *sq)

    def second_moment(shape, kind, gen, dtype):
        if kind == "uniform":
            return torch.rand(shape, generator=gen, dtype=dtype) + 0.1
        if kind == "exponential":
            return -(torch.rand(shape, generator=gen, dtype=dtype) + 1e-6).log()
        v = torch.full(shape, 1e-3, dtype=dtype)
        v.view(-1)[0] = 1.0
        return v

    raw = []
    for shape, theta, kind, dtype, seed in itertools.product(
        [(16,), (256,), (16, 16), (32, 8), (8, 32), (64, 64)], [0.0, 1e-3, 1e-2, 0.1, 0.5, 1.0, math.pi / 2],
        ["uniform", "exponential", "spike"], [torch.float32, torch.float64], range(args.seeds),
    ):  # fmt: skip
        gen = torch.Generator().manual_seed(seed)
        old, new = [], []
        for d in shape:
            q = torch.linalg.qr(torch.randn(d, d, generator=gen, dtype=dtype)).Q
            skew = torch.randn(d, d, generator=gen, dtype=dtype)
            skew = (skew - skew.mT) / 2
            skew = skew / skew.norm() * math.sqrt(d)
            old.append(q)
            new.append(q @ torch.linalg.matrix_exp(theta * skew))
        v = second_moment(shape, kind, gen, dtype)
        truth = transport("hadamard", v, old, new)
        rec = [len(shape), DTYPE_NAMES[dtype], theta]
        for method in ("none", "linear", "hadamard"):
            out = transport(method, v, old, new)
            rec += [(out - truth).abs().max().item(), out.min().item(), (out.sum() - v.sum()).item() / v.sum().item()]
        raw.append(tuple(rec))
    rows = []
    for key, group in itertools.groupby(sorted(raw, key=lambda r: r[:3]), key=lambda r: r[:3]):
        group = list(group)
        cells = []
        for base in (3, 6, 9):
            cells += [f"{max(g[base] for g in group):.2e}", f"{min(g[base + 1] for g in group):.2e}",
                      f"{max(abs(g[base + 2]) for g in group):.2e}"]  # fmt: skip
        rows.append((f"{key[0]}d", key[1], f"{key[2]:.4f}", *cells))
    header = ("modes", "dtype", "theta") + tuple(f"{s} {m}" for m in ("none", "linear", "hadamard") for s in ("err", "min", "|dsum|"))
    _table("second moment after a rotation by angle theta (worst over shapes, kinds, seeds)", header, rows)
    _maybe_csv(args.csv, ("modes", "dtype", "theta") + tuple(f"{s}_{m}" for m in ("none", "linear", "hadamard") for s in ("err", "min", "dsum")), raw)


# ------------------------------------------------------------------------------------------ PSGD fitting


def cmd_precond_fitting(args):
    """Feeds ``psgd_update_precond`` pairs ``(v, H v)`` with ``H = kron(H_1, H_2)`` known and reports
    ``prod_i cond(Q_i^T Q_i H_i)`` after ``--steps`` updates: 1 means the factors whiten the Hessian exactly."""
    draws = {
        "normal": lambda s: torch.randn(*s, device=DEVICE),
        "laplace": lambda s: torch.distributions.Laplace(0.0, 1.0).sample(s).to(DEVICE),
        "rademacher": lambda s: torch.randint(0, 2, s, device=DEVICE, dtype=torch.float32) * 2 - 1,
        "uniform": lambda s: torch.rand(*s, device=DEVICE) * 2 - 1,
        "sparse normal (80% zeros)": lambda s: torch.randn(*s, device=DEVICE) * (torch.rand(*s, device=DEVICE) > 0.8),
    }

    def spd(n, cond):
        q = torch.linalg.qr(torch.randn(n, n, device=DEVICE)).Q
        return (q * torch.logspace(0, math.log10(cond), n, device=DEVICE)) @ q.mT

    rows = []
    for (name, draw), cond, lr, iters in itertools.product(draws.items(), args.cond, args.precond_lr, args.power_iter):
        torch.manual_seed(args.seed)
        shape = tuple(args.shape)
        factors = [spd(d, cond) for d in shape]
        Q = utils.init_Q_exprs(torch.zeros(1, *shape, device=DEVICE), 1.0, 1.0, 0.0, max(shape), 1, None, None, None)
        lower = [torch.zeros((1,), device=DEVICE, dtype=torch.float64) for _ in shape]
        for step in range(args.steps):
            torch.manual_seed(args.seed + 1 + step)
            v = draw(shape)
            hv = v
            for mode, h in enumerate(factors):
                hv = torch.movedim(torch.tensordot(h, hv, dims=([1], [mode])), 0, mode)
            utils.psgd_update_precond(hv.unsqueeze(0).contiguous(), lr, Q, False, args.beta2, v.unsqueeze(0), lower, args.lower_bound_beta, iters)
        misfit = 1.0
        for q, h in zip(Q, factors):
            q = q[0] if q.ndim == 3 else torch.diag(q[0])
            misfit *= torch.linalg.cond((q.mT @ q).double() @ h.double()).item()
        rows.append((name, f"{cond:g}", lr, iters, f"{misfit:.3f}"))
    _table(f"PSGD Kronecker fit after {args.steps} steps on a {'x'.join(map(str, args.shape))} problem (1 = exact)",
           ("probe distribution", "cond(H_i)", "precond_lr", "power_iter", "prod cond(Q^T Q H)"), rows)  # fmt: skip
    _maybe_csv(args.csv, ("dist", "cond", "precond_lr", "power_iter", "misfit"), rows)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--csv", default=None, help="also write the raw rows to this file")
    sub = ap.add_subparsers(dest="command", required=True)
    sub.add_parser("singular-values").set_defaults(fn=cmd_singular_values)
    p = sub.add_parser("sv-methods")
    p.add_argument("--max-size", type=int, default=64)
    p.add_argument("--attempts", type=int, default=4)
    p.set_defaults(fn=cmd_sv_methods)
    p = sub.add_parser("klsoap-pinv")
    p.add_argument("--seeds", type=int, default=3)
    p.set_defaults(fn=cmd_klsoap_pinv)
    p = sub.add_parser("variance-rotation")
    p.add_argument("--seeds", type=int, default=3)
    p.set_defaults(fn=cmd_variance_rotation)
    p = sub.add_parser("precond-fitting")
    p.add_argument("--shape", type=int, nargs="+", default=[16, 16])
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--cond", type=float, nargs="+", default=[10.0, 1e3])
    p.add_argument("--precond-lr", type=float, nargs="+", default=[0.1, 0.3])
    p.add_argument("--power-iter", type=int, nargs="+", default=[0, 2])
    p.add_argument("--beta2", type=float, default=0.9)
    p.add_argument("--lower-bound-beta", type=float, default=0.9)
    p.set_defaults(fn=cmd_precond_fitting)
    args = ap.parse_args()
    args.fn(args)


if __name__ == "__main__":
    main()
