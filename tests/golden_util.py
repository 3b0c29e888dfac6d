"""Loading of the committed fixtures (tests/golden/*.npz, written by make_golden.py)."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    manifest = json.loads(bytes(z["manifest"]).decode())
    return z, manifest


def f64(bits):
    return np.ascontiguousarray(bits, dtype=np.uint64).view(np.float64)


def u64(x):
    return np.ascontiguousarray(x, dtype=np.float64).view(np.uint64)


def same_bits(a, b):
    """Bit equality, any NaN equal to any NaN (payloads are not part of the contract)."""
    a = np.ascontiguousarray(a, np.float64)
    b = np.ascontiguousarray(b, np.float64)
    if a.shape != b.shape:
        return False
    nan = np.isnan(a) & np.isnan(b)
    return bool(np.all(nan | (a.view(np.uint64) == b.view(np.uint64))))


def scalar(bits):
    return float(np.array([bits], np.uint64).view(np.float64)[0])
