"""Small, self-terminating workloads for kernel profiling (launch lists and single-kernel captures).

    python benchmarks/profile_targets.py opt_step_gpt2   # 3 optimizer steps, GPT-2-small parameter shapes
    python benchmarks/profile_targets.py ns_small        # Newton-Schulz on 8 x (1024 x 4096) bf16-sized work
    python benchmarks/profile_targets.py adam_small      # fused AdamW over 64M fp32 parameters (768 MB state+params)
    python benchmarks/profile_targets.py ce_small        # cross-entropy fwd+bwd kernel, 4096 x 50304 bf16 logits (412 MB)
    python benchmarks/profile_targets.py ln_small        # LayerNorm fwd + bwd kernels, 16384 x 768 fp32 (50 MB) x 4 tensors
    python benchmarks/profile_targets.py gelu_small      # GELU fwd, and bwd + bias gradient, 16384 x 3072 bf16 (100 MB per tensor)
    python benchmarks/profile_targets.py tf32_small      # split-tf32 GEMM, 4 x (2048 x 2048 x 2048)
    python benchmarks/profile_targets.py qr_small        # panel-wise Cholesky QR of 8 x (1024 x 1024), eager launches
    python benchmarks/profile_targets.py ns_big          # Newton-Schulz on 4 x (4096 x 4096): the 256 x 256-tile kernel
    python benchmarks/profile_targets.py soap_small      # one plain SOAP step on 8 x 1024^2 (tf32 GEMMs with fused epilogues)
    python benchmarks/profile_targets.py psgd_small      # one plain PSGDKron step on 8 x 1024^2 (cached P = Q^T Q operands)
    python benchmarks/profile_targets.py psgd_fit        # one PSGDKron step with a preconditioner fit, 8 x (1024 x 4096)
    python benchmarks/profile_targets.py soap_refresh    # one SOAP step with an eigenbasis refresh, 8 x (2048 x 2048)

Each case holds well under a few GB on the device and launches only a handful of kernels.
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import heavyball_b200 as hb  # noqa: E402
from heavyball_b200 import ops, utils  # noqa: E402


def opt_step_gpt2(steps=3):
    from heavyball_b200.models import GPT, GPTConfig, split_param_groups

    m = GPT(GPTConfig(12, 12, 768, 0, 50257, 1024)).cuda()
    mats, rest = split_param_groups(m)
    opt = hb.SplitOpt([
        {"params": mats, "optimizer": hb.Muon, "lr": 0.02},
        {"params": rest, "optimizer": hb.AdamW, "lr": 3e-4},
    ])
    grads = [torch.randn_like(p) * 0.01 for p in m.parameters()]

    def one_step():
        for p, g in zip(m.parameters(), grads):
            p.grad = g
        opt.step()

    one_step()  # the first step initialises state through the PyTorch path
    one_step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()  # with `ncu --profile-from-start off` only the steady-state steps are captured
    for _ in range(steps):
        one_step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()


def ns_small():
    mats = [torch.randn(1024, 4096, device="cuda") for _ in range(8)]
    out = ops.newton_schulz_batched(mats, utils.NS5_COEFFS)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    out = ops.newton_schulz_batched(mats, utils.NS5_COEFFS)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()
    print(float(out.abs().mean()))


def adam_small():
    params = [torch.nn.Parameter(torch.randn(4096, 4096, device="cuda")) for _ in range(4)]
    opt = hb.AdamW(params, lr=1e-3, consume_grad=False)
    for p in params:
        p.grad = torch.randn_like(p)
    for _ in range(3):
        opt.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    opt.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


def _timed(fn, reps=5):
    """Median CUDA-event time of ``fn`` in microseconds, with a 256 MB L2 flush before each repetition."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    times = []
    for _ in range(reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    return sorted(times)[len(times) // 2]


def ce_small():
    rows, vocab, padded = 4096, 50257, 50304
    logits = (torch.randn(rows, padded, device="cuda") * 2).to(torch.bfloat16)
    targets = torch.randint(0, vocab, (rows,), device="cuda")
    scale = torch.full((1,), 1.0 / rows, device="cuda")
    ext = ops.load()
    work = logits.clone()
    us = _timed(lambda: ext.cross_entropy_(work, targets, scale, vocab, -100))
    gb = 2 * rows * padded * 2 / 1e9
    print(f"cross_entropy {rows}x{padded}: {us:.1f} us, {gb / us * 1e6:.0f} GB/s of algorithmic traffic (1 read + 1 write)")
    work.copy_(logits)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    ext.cross_entropy_(work, targets, scale, vocab, -100)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


def ln_small():
    rows, d = 16384, 768
    x = torch.randn(rows, d, device="cuda")
    w, b = torch.rand(d, device="cuda") + 0.5, torch.randn(d, device="cuda")
    dy = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
    dres = torch.randn(rows, d, device="cuda")  # gradient arriving on the residual stream
    ext = ops.load()
    y, mean, rstd = ext.layer_norm_fwd(x, None, w, b, 1e-5, True)
    us_f = _timed(lambda: ext.layer_norm_fwd(x, None, w, b, 1e-5, True))
    us_b = _timed(lambda: ext.layer_norm_bwd(dy, x, w, mean, rstd, dres, True))
    print(f"layer_norm fwd {rows}x{d}: {us_f:.1f} us, {(rows * d * 6) / us_f / 1e3:.0f} GB/s (fp32 in, bf16 out)")
    print(f"layer_norm bwd {rows}x{d}: {us_b:.1f} us, {(rows * d * 16) / us_b / 1e3:.0f} GB/s (bf16 dy + fp32 x + fp32 residual-stream gradient in, fp32 + bf16 dx out)")
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    ext.layer_norm_fwd(x, None, w, b, 1e-5, True)
    ext.layer_norm_bwd(dy, x, w, mean, rstd, dres, True)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


def gelu_small():
    rows, cols = 16384, 3072
    u = (torch.randn(rows, cols, device="cuda") * 2).to(torch.bfloat16)
    dy = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    ext = ops.load()
    uf = u.clone().requires_grad_()
    yf = torch.nn.functional.gelu(uf, approximate="tanh")
    n = rows * cols
    us_f = _timed(lambda: ext.gelu_fwd(u))
    us_b = _timed(lambda: ext.gelu_bwd(dy, u))
    us_ff = _timed(lambda: torch.nn.functional.gelu(u, approximate="tanh"))
    us_fb = _timed(lambda: torch.autograd.grad(yf, uf, dy, retain_graph=True)) + _timed(lambda: ext.colsum_bf16(dy))
    print(f"gelu fwd {rows}x{cols} bf16: {us_f:.1f} us, {n * 4 / us_f / 1e3:.0f} GB/s; framework kernel {us_ff:.1f} us")
    print(f"gelu bwd + bias gradient: {us_b:.1f} us, {n * 6 / us_b / 1e3:.0f} GB/s; framework backward + column-sum kernel {us_fb:.1f} us")
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    ext.gelu_fwd(u)
    ext.gelu_bwd(dy, u)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


def tf32_small():
    a = torch.randn(4, 2048, 2048, device="cuda")
    b = torch.randn(4, 2048, 2048, device="cuda")
    out = ops.matmul3(a, b)
    us = _timed(lambda: ops.matmul3(a, b))
    us_ref = _timed(lambda: torch.matmul(a, b))
    flops = 2 * 4 * 2048**3
    print(f"matmul3 4x2048^3: {us:.1f} us incl. both split passes = {flops / us / 1e6:.1f} useful TFLOP/s "
          f"({3 * flops / us / 1e6:.1f} tf32 TFLOP/s issued); torch fp32 matmul {us_ref:.1f} us = {flops / us_ref / 1e6:.1f} TFLOP/s")
    err = (out.double() - a.double() @ b.double()).abs().max().item()
    ref_err = (torch.matmul(a, b).double() - a.double() @ b.double()).abs().max().item()
    print(f"max abs error vs fp64: ours {err:.3e}, torch fp32 {ref_err:.3e}")
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    ops.matmul3(a, b)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()


def qr_small():
    from heavyball_b200.utils.orthogonal import _panel_cholesky_qr

    torch.manual_seed(0)
    basis = torch.linalg.qr(torch.randn(8, 1024, 1024, device="cuda")).Q
    gg = (basis * torch.logspace(0, -6, 1024, device="cuda")) @ basis.mT
    power = gg @ torch.linalg.qr(basis + 1e-3 * torch.randn_like(basis)).Q
    q = _panel_cholesky_qr(power)
    us = _timed(lambda: _panel_cholesky_qr(power), reps=3)
    err = (q.mT @ q - torch.eye(1024, device="cuda")).abs().max().item()
    us_ref = _timed(lambda: torch.linalg.qr(power), reps=3)
    print(f"panel QR 8x1024x1024: {us:.0f} us eager launches (library Householder QR {us_ref:.0f} us), |Q^T Q - I| = {err:.1e}")
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    _panel_cholesky_qr(power)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


def ns_big():
    mats = [torch.randn(4096, 4096, device="cuda") for _ in range(4)]
    out = ops.newton_schulz_batched(mats, utils.NS5_COEFFS)
    us = _timed(lambda: ops.newton_schulz_batched(mats, utils.NS5_COEFFS), reps=3)
    # per iteration: Gram (upper tiles count half), polynomial (same), apply; 5 iterations
    dense = 5 * 3 * 2 * 4 * 4096**3
    print(f"newton_schulz 4x4096^2: {us:.0f} us, {dense / us / 1e6:.0f} dense-equivalent TFLOP/s, "
          f"{dense * (2 / 3) / us / 1e6:.0f} TFLOP/s counting symmetric products once")
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    out = ops.newton_schulz_batched(mats, utils.NS5_COEFFS)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()
    print(float(out.abs().mean()))


def _second_order(cls, shape=(1024, 1024), count=8, fresh_grads=False, **kw):
    params = [torch.nn.Parameter(torch.randn(*shape, device="cuda")) for _ in range(count)]
    opt = cls(params, lr=1e-3, **kw)
    grads = [torch.randn_like(p) for p in params]

    def one_step():
        for p, g in zip(params, grads):
            if fresh_grads:  # statistics accumulated over different gradients are full rank, as in training
                g.normal_()
            p.grad = g
        opt.step()

    return opt, one_step


def soap_small():
    opt, one_step = _second_order(hb.SOAP, precondition_frequency=100)
    for _ in range(4):
        one_step()
    us = _timed(one_step)
    print(f"SOAP plain step 8x1024^2: {us:.0f} us")
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    one_step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()


def psgd_small():
    opt, one_step = _second_order(hb.PSGDKron, preconditioner_update_probability=1e-9)
    for _ in range(4):
        one_step()
    us = _timed(one_step)
    print(f"PSGDKron plain step 8x1024^2: {us:.0f} us")
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    one_step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()


def _periodic(cls, shape, count, label, **kw):
    """Times and exposes one step that includes the periodic stage (fit / refresh): the schedule is set so that every
    step does it; the first two run eagerly / are captured, the profiled one is the steady state."""
    opt, one_step = _second_order(cls, shape, count, fresh_grads=True, **kw)
    for _ in range(6):
        one_step()
    us = _timed(one_step, reps=3)
    print(f"{label} {count}x{shape[0]}x{shape[1]}: {us:.0f} us")
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    one_step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()


def psgd_fit():
    _periodic(hb.PSGDKron, (1024, 4096), 8, "PSGDKron step with fit", preconditioner_update_probability=1.0,
              max_size_triangular=8192)


def soap_refresh():
    from heavyball_b200.utils import orthogonal

    _periodic(hb.SOAP, (2048, 2048), 8, "SOAP step with refresh", precondition_frequency=1)
    print("QR paths taken:", orthogonal.qr_stats)


if __name__ == "__main__":
    {"psgd_fit": psgd_fit, "soap_refresh": soap_refresh, "ns_big": ns_big, "soap_small": soap_small, "psgd_small": psgd_small, "qr_small": qr_small, "opt_step_gpt2": opt_step_gpt2, "ns_small": ns_small, "adam_small": adam_small, "ce_small": ce_small,
     "ln_small": ln_small, "tf32_small": tf32_small, "gelu_small": gelu_small}[sys.argv[1]]()
