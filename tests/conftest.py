import os
import sys

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

GOLDEN = os.path.join(REPO, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name)))


def gc_from_golden(g):
    """Rebuild the reference's per-layer compressed dict from a fixture."""
    gc = {k: g[k] for k in ["k_coeffs", "k_coeff_scale", "k_basis_q", "k_basis_scale", "k_basis_f16",
                            "k_mean", "k_mean_f16", "v_indices_u8", "v_centroids_f16", "v_ch_f16"]}
    for k in ["sink_k", "sink_v", "win_k", "win_v"]:
        gc[k] = g[k][0]                       # drop the batch axis -> (nkv, n, hd)
    n_total, rank, n_comp, batch, start = (int(x) for x in g["meta"])
    gc.update(k_coeffs_shape=(n_total, rank), n_compress=n_comp, batch=batch, compress_start=start)
    return gc


@pytest.fixture(scope="session")
def golden_cfg0():
    return load_golden("cfg0.npz")


@pytest.fixture(scope="session")
def golden_chain512():
    return load_golden("chain512.npz")


def tol_ok(x, ref, atol=2e-3, rtol=1e-2):
    """|x - ref| <= atol + rtol * |ref| elementwise (the decode-attention bar)."""
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return bool(np.all(np.abs(x - ref) <= atol + rtol * np.abs(ref)))
