"""Shared helpers of the parity tests: golden-file access and the two float criteria.

Float tolerance: per tensor, cosine similarity >= 0.9999 and
max|a-b| / max|b| <= 1e-2 against the fp32 reference.  Integer / int8-path results must be
bit-exact.
"""
import glob
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
COS_MIN = 0.9999
REL_MAX = 1e-2


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def golden_names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


def cosine(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na == 0 and nb == 0:
        return 1.0
    return float(a @ b / (na * nb + 1e-300))


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    m = np.abs(b).max()
    return float(np.abs(a - b).max() / (m if m > 0 else 1.0))


def assert_close(got, ref, what=""):
    got = np.asarray(got)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    c, r = cosine(got, ref), rel_err(got, ref)
    assert c >= COS_MIN and r <= REL_MAX, f"{what}: cosine {c:.7f} (min {COS_MIN}), max rel err {r:.3e} (max {REL_MAX})"
