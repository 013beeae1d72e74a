"""Loading of the golden fixtures recorded from the reference (tests/golden/*.npz)."""
import glob
import json
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    cfg = json.loads(bytes(z["cfg"]).decode())
    return cfg, {k: z[k] for k in z.files if k != "cfg"}


def names(kind_prefix):
    out = []
    for p in sorted(glob.glob(os.path.join(GOLDEN_DIR, kind_prefix + "*.npz"))):
        out.append(os.path.basename(p)[:-4])
    return out


def assert_close(a, b, rel=1e-5, what=""):
    """fp32 parity metric: max|a-b| <= rel * max|b| (and elementwise allclose with that atol)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    scale = max(np.abs(b).max(initial=0.0), 1e-30)
    err = np.abs(a - b).max(initial=0.0)
    assert err <= rel * scale, f"{what}: max abs err {err:.3e} > {rel:g} * {scale:.3e}"
