"""Helpers shared by the tests."""
import glob
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = ("out", "dq", "dk1", "dk2", "dv1", "dv2")


def golden_files(prefix=""):
    """Operator goldens (naive_*, outer_*); stack_* holds a whole decoder stack and has its own test."""
    return sorted(f for f in glob.glob(os.path.join(GOLDEN, prefix + "*.npz"))
                  if not os.path.basename(f).startswith("stack_"))


def load_golden(path):
    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in z.files if z[k].ndim > 0}
    return t, int(z["w1"]), int(z["w2"])


def rel_err(x, ref, floor=1e-3):
    """max-norm relative error  ||x - ref||_inf / max(||ref||_inf, floor).  The floor keeps
    tensors that are analytically zero (dq when every window holds one key) from dividing
    by zero; callers pass a fraction of the largest sibling tensor's norm."""
    x, ref = x.detach().double().cpu(), ref.detach().double().cpu()
    return ((x - ref).abs().max() / ref.abs().max().clamp_min(floor)).item()


def max_abs(x, ref):
    return (x.detach().double().cpu() - ref.detach().double().cpu()).abs().max().item()
