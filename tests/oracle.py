"""Runs a small training job under either library in a fresh interpreter and returns what it produced.

The job is described by plain data (class name, kwargs, model recipe) so the *same* description drives
the reference (imported as ``heavyball`` from a path given on the command line, compile disabled) and
this package.  Used by the parity tests as an independent oracle: trajectories, state-dict structure
and cross-loading of checkpoints.
"""

import io
import json
import os
import pickle
import subprocess
import sys

WORKER = r'''
import os, sys, json, pickle, warnings, io
os.environ["TORCH_COMPILE_DISABLE"] = "1"
warnings.filterwarnings("ignore")
job = json.loads(sys.argv[1])
if job["lib"] == "reference":
    sys.path.insert(0, job["ref_path"])
    import heavyball as hb
    hb.utils.compile_mode = None
else:
    sys.path.insert(0, job["root"])
    import heavyball_b200 as hb
import torch, torch.nn as nn, torch.nn.functional as F
torch.set_num_threads(2)

def make(job):
    torch.manual_seed(job.get("seed", 0))
    dims = job.get("dims", [16, 32, 32, 10])
    layers = []
    for a, b in zip(dims[:-1], dims[1:]):
        layers += [nn.Linear(a, b), nn.GELU()]
    m = nn.Sequential(*layers[:-1])
    for p in m.parameters():
        if p.ndim >= 2: nn.init.normal_(p, 0, job.get("std", 0.02))
        else: nn.init.zeros_(p)
    if job.get("dtype") == "float64":
        m = m.double()
    x = torch.randn(job.get("batch", 32), dims[0], dtype=next(m.parameters()).dtype)
    y = torch.randint(0, dims[-1], (job.get("batch", 32),))
    return m, x, y

def build(job, m):
    kw = dict(job.get("kwargs", {}))
    if "betas" in kw: kw["betas"] = tuple(kw["betas"])
    if job["cls"] == "SplitOpt":
        mats = [p for p in m.parameters() if p.ndim >= 2]; vecs = [p for p in m.parameters() if p.ndim < 2]
        return hb.SplitOpt([{"params": mats, "optimizer": hb.Muon, "lr": 0.02}, {"params": vecs, "optimizer": hb.AdamW, "lr": 1e-3}])
    return getattr(hb, job["cls"])(m.parameters(), **kw)

def run_one(job):
  m, x, y = make(job)
  o = build(job, m)
  if job.get("load"):
      sd = torch.load(job["load"], weights_only=False)
      m.load_state_dict(sd["model"]); o.load_state_dict(sd["opt"])
  losses = []
  for i in range(job["steps"]):
      torch.manual_seed(1000 + i)
      loss = F.cross_entropy(m(x), y); loss.backward(); o.step(); o.zero_grad(); losses.append(loss.item())
  out = {"losses": losses}
  sd = o.state_dict()
  def describe(v):
      if isinstance(v, torch.Tensor): return ["T", str(v.dtype), list(v.shape)]
      if isinstance(v, (list, tuple)): return [type(v).__name__, [describe(i) for i in v]]
      if isinstance(v, dict): return {str(k): describe(i) for k, i in v.items()}
      if isinstance(v, set): return ["set", sorted(v)]
      if isinstance(v, bytes): return ["bytes"]
      return [type(v).__name__]
  out["structure"] = describe(sd)
  if job.get("save"):
      torch.save({"model": m.state_dict(), "opt": sd}, job["save"])
  out["params"] = [p.detach().double().flatten()[:8].tolist() for p in m.parameters()]
  return out

results = []
for sub in job["jobs"]:
    sub = dict(job, **sub)
    try:
        results.append(run_one(sub))
    except Exception as e:
        import traceback
        results.append({"error": traceback.format_exc()[-1500:]})
print("@@RESULT@@" + json.dumps(results))
'''


def run_many(lib, jobs, ref_path=None, timeout=1800):
    """Runs every job description in ``jobs`` inside one fresh interpreter using library ``lib``
    (``"reference"`` or ``"ours"``); returns one result dict per job (``{"error": ...}`` on failure)."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    job = dict(lib=lib, jobs=list(jobs), root=root, ref_path=ref_path, cls="<batch>")
    proc = subprocess.run([sys.executable, "-c", WORKER, json.dumps(job)], capture_output=True, text=True, timeout=timeout)
    if proc.returncode != 0:
        raise RuntimeError(f"worker failed ({job['lib']} {job['cls']}):\n{proc.stderr[-3000:]}")
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("@@RESULT@@")][-1]
    return json.loads(line[len("@@RESULT@@"):])


def run(job, ref_path=None, timeout=600):
    out = run_many(job["lib"], [job], ref_path, timeout)[0]
    if "error" in out:
        raise RuntimeError(out["error"])
    return out
