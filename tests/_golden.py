"""Loader of the golden fixtures (outputs of the reference's own kernels)."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    d = {k: torch.from_numpy(z[k]) for k in z.files if k not in ("causal", "sm_scale")}
    d["causal"] = bool(z["causal"])
    s = float(z["sm_scale"])
    d["sm_scale"] = None if np.isnan(s) else s
    d["packed"] = "qkv" in d
    if d["packed"]:
        d["q"], d["k"], d["v"] = d["qkv"][:, :, 0], d["qkv"][:, :, 1], d["qkv"][:, :, 2]
    return d
