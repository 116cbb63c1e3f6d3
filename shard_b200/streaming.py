"""Host side of the 8-bit Lloyd-Max stream quantizer.

The codebook is a property of N(0, 1/d) only, so it is computed once on the
host in double precision (same recurrence as the reference's
src/shard/streaming.py:35-51, so the fp32 table is bit-identical) and cached
per device.  Quantisation and dequantisation of tokens run in CUDA
(csrc/stream.cu).  The optional 1-bit QJL residual of the reference is not
part of this path (it is off by default there) and is rejected.
"""
from __future__ import annotations

import math

import torch

# P. J. Acklam's rational approximation of the inverse normal CDF: central
# region numerator/denominator, tail numerator/denominator.
_CENTRAL_NUM = (-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02,
                1.383577518672690e+02, -3.066479806614716e+01, 2.506628277459239e+00)
_CENTRAL_DEN = (-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02,
                6.680131188771972e+01, -1.328068155288572e+01)
_TAIL_NUM = (-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00,
             -2.549732539343734e+00, 4.374664141464968e+00, 2.938163982698783e+00)
_TAIL_DEN = (7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00,
             3.754408661907416e+00)
_SPLIT = 0.02425


def _poly(coeffs, x):
    acc = coeffs[0]
    for c in coeffs[1:]:
        acc = acc * x + c
    return acc


def _inv_cdf(p):
    if p < _SPLIT:
        q = math.sqrt(-2 * math.log(p))
        return _poly(_TAIL_NUM, q) / (_poly(_TAIL_DEN, q) * q + 1)
    if p <= 1 - _SPLIT:
        q = p - 0.5
        r = q * q
        return _poly(_CENTRAL_NUM, r) * q / (_poly(_CENTRAL_DEN, r) * r + 1)
    q = math.sqrt(-2 * math.log(1 - p))
    return -_poly(_TAIL_NUM, q) / (_poly(_TAIL_DEN, q) * q + 1)


def lloyd_max_codebook(d, bits, n_iter=100):
    """2**bits Lloyd-Max centroids for N(0, 1/d), ascending, fp32."""
    levels = 1 << bits
    sigma = 1.0 / math.sqrt(d)
    cent = [_inv_cdf((i + 0.5) / levels) * sigma for i in range(levels)]
    root2, root2pi = math.sqrt(2), math.sqrt(2 * math.pi)
    for _ in range(n_iter):
        edges = [-1e9] + [(cent[k - 1] + cent[k]) / 2 for k in range(1, levels)] + [1e9]
        nxt = []
        for k in range(levels):
            za, zb = edges[k] / sigma, edges[k + 1] / sigma
            mass = 0.5 * (1 + math.erf(zb / root2)) - 0.5 * (1 + math.erf(za / root2))
            if mass < 1e-12:
                nxt.append(cent[k])
            else:
                dens = math.exp(-0.5 * za * za) / root2pi - math.exp(-0.5 * zb * zb) / root2pi
                nxt.append(dens * sigma / mass)
        moved = max(abs(a - b) for a, b in zip(nxt, cent))
        if moved < 1e-9:
            break
        cent = nxt
    return torch.tensor(cent, dtype=torch.float32)


_cache = {}


def get_codebook(d, bits, device):
    """Cached device copy of the (d, bits) codebook."""
    if bits != 8 or d != 128:
        raise NotImplementedError("the CUDA stream quantizer supports 8-bit codes of 128-dim heads")
    key = (d, bits, str(device))
    if key not in _cache:
        host = _cache.get((d, bits))
        if host is None:
            host = _cache[(d, bits)] = lloyd_max_codebook(d, bits)
        _cache[key] = host.to(device)
    return _cache[key]


def stream_signs(layer_idx, hd, device):
    """Per-layer +-1 vector from torch's CPU generator seeded 42 + 7919 * layer
    (reference: src/shard/cache.py:201-204)."""
    g = torch.Generator(device="cpu").manual_seed(42 + layer_idx * 7919)
    return (torch.randint(0, 2, (hd,), generator=g) * 2 - 1).to(device, torch.float32)
