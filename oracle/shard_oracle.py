"""CPU oracle for the compressed-KV attention path of bhengubv/shard.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain numpy, the algorithm
of the reference's CPU (PyTorch-fallback) path.  It is the checker the CUDA
kernels are compared against; the product never imports it and never falls
back to it.  Only the test-suite, the smoke check and the benchmark's
CPU-baseline / reference arm may call into it.

Parity status: PINNED.  Every function below is checked against outputs of
the reference's own Python implementation (imported from its source tree when
the fixtures were generated; see tests/golden/make_golden.py) that are stored
under tests/golden/*.npz.

Conventions
-----------
* "reference" paths are relative to the reference project root
  (src/shard/cache.py etc.).
* fp16 arithmetic of the reference is emulated with numpy float16 arrays:
  numpy, like PyTorch on CPU, evaluates each half-precision elementwise op in
  fp32 and rounds the result once to fp16.
* Reductions whose association order is an implementation detail of PyTorch
  (vector norm, mean, GEMM) are evaluated here in a wider type and rounded
  once; downstream integer stages are therefore exact *given identical fp32
  inputs*, which is how the parity tests drive them.
"""
from __future__ import annotations

import math
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

HOST_THREADS = os.cpu_count() or 1

F16 = np.float16
F32 = np.float32

# ---------------------------------------------------------------------------
# Hadamard  (reference: src/shard/cache.py:10-19)
# ---------------------------------------------------------------------------


def hadamard(x: np.ndarray) -> np.ndarray:
    """Normalised fast Walsh-Hadamard transform along the last axis.

    Follows src/shard/cache.py:10-19: stages h = 1, 2, 4, ... d/2; every block
    of 2h entries [a | b] becomes [a+b | a-b]; the result is divided by
    sqrt(d) at the end.  The dtype of ``x`` is preserved, so an fp16 input is
    rounded to fp16 after every stage exactly as the reference does in
    src/shard/attention.py:112.
    """
    d = x.shape[-1]
    lead = x.shape[:-1]
    dt = x.dtype
    y = np.array(x, copy=True)
    h = 1
    while h < d:
        y = y.reshape(lead + (d // (2 * h), 2 * h))
        a, b = y[..., :h], y[..., h:]
        y = np.concatenate([a + b, a - b], axis=-1).reshape(lead + (d,))
        h *= 2
    if dt == F16:
        return (y.astype(F32) / F32(math.sqrt(d))).astype(F16)
    return (y / np.asarray(math.sqrt(d), dtype=dt)).astype(dt)


# ---------------------------------------------------------------------------
# Lloyd-Max stream quantizer  (reference: src/shard/streaming.py)
# ---------------------------------------------------------------------------

# Coefficients of P. J. Acklam's rational approximation to the inverse normal
# CDF (published algorithm; the reference seeds Lloyd-Max with it,
# src/shard/streaming.py:11-33).
_ACK_A = (-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02,
          1.383577518672690e+02, -3.066479806614716e+01, 2.506628277459239e+00)
_ACK_B = (-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02,
          6.680131188771972e+01, -1.328068155288572e+01)
_ACK_C = (-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00,
          -2.549732539343734e+00, 4.374664141464968e+00, 2.938163982698783e+00)
_ACK_D = (7.784695709041462e-03, 3.224671290700398e-01,
          2.445134137142996e+00, 3.754408661907416e+00)


def _horner(coeffs, x):
    acc = coeffs[0]
    for c in coeffs[1:]:
        acc = acc * x + c
    return acc


def inv_normal_cdf(p: float) -> float:
    """Acklam inverse normal CDF, src/shard/streaming.py:21-33."""
    p_low = 0.02425
    if p < p_low:
        q = math.sqrt(-2 * math.log(p))
        return _horner(_ACK_C, q) / (_horner(_ACK_D, q) * q + 1)
    if p <= 1 - p_low:
        q = p - 0.5
        r = q * q
        return _horner(_ACK_A, r) * q / (_horner(_ACK_B, r) * r + 1)
    q = math.sqrt(-2 * math.log(1 - p))
    return -_horner(_ACK_C, q) / (_horner(_ACK_D, q) * q + 1)


def lloyd_max_codebook(d: int, bits: int, n_iter: int = 100) -> np.ndarray:
    """2**bits Lloyd-Max centroids of N(0, 1/d); src/shard/streaming.py:35-51.

    Python-double arithmetic in the same order as the reference so that the
    fp32 table is bit-identical.
    """
    n = 1 << bits
    sigma = 1.0 / math.sqrt(d)
    c = [inv_normal_cdf((i + 0.5) / n) * sigma for i in range(n)]

    def pdf(z):
        return math.exp(-0.5 * z * z) / math.sqrt(2 * math.pi)

    def cdf(z):
        return 0.5 * (1 + math.erf(z / math.sqrt(2)))

    for _ in range(n_iter):
        edges = [-1e9] + [(c[k - 1] + c[k]) / 2 for k in range(1, n)] + [1e9]
        nc = []
        for k in range(n):
            a, b = edges[k], edges[k + 1]
            mass = cdf(b / sigma) - cdf(a / sigma)
            nc.append(c[k] if mass < 1e-12 else (pdf(a / sigma) - pdf(b / sigma)) * sigma / mass)
        if max(abs(x - y) for x, y in zip(nc, c)) < 1e-9:
            break
        c = nc
    return np.asarray(c, dtype=np.float64).astype(F32)


def stream_signs(layer_idx: int, hd: int = 128) -> np.ndarray:
    """Per-layer random sign vector, src/shard/cache.py:201-204.

    The reference draws it with torch's CPU generator seeded 42 + 7919*layer;
    that stream is third-party (PyTorch's Philox/mt19937 front end), so the
    host code and this oracle both take the vector from torch.  Imported
    lazily to keep the numeric core numpy-only.
    """
    import torch
    g = torch.Generator(device="cpu").manual_seed(42 + layer_idx * 7919)
    return (torch.randint(0, 2, (hd,), generator=g) * 2 - 1).to(torch.float32).numpy()


def quantize_per_token(u: np.ndarray, signs: np.ndarray, codebook: np.ndarray) -> np.ndarray:
    """8-bit Lloyd-Max codes of unit vectors; src/shard/streaming.py:59-72.

    rot = hadamard(u * signs); idx = lower_bound(codebook, rot) clamped to the
    last entry; the left neighbour wins only if it is strictly closer.
    """
    rot = hadamard((u.astype(F32) * signs.astype(F32)).astype(F32))
    idx = np.searchsorted(codebook, rot, side="left")
    idx = np.minimum(idx, codebook.shape[0] - 1)
    left = np.maximum(idx - 1, 0)
    take_left = np.abs(codebook[left] - rot) < np.abs(codebook[idx] - rot)
    return np.where(take_left, left, idx).astype(np.uint8)


def dequantize_per_token(idx: np.ndarray, signs: np.ndarray, codebook: np.ndarray) -> np.ndarray:
    """fp16 unit vectors from codes; src/shard/streaming.py:74-79 (QJL off)."""
    rot = codebook[idx.astype(np.int64)]
    return (hadamard(rot.astype(F32)) * signs.astype(F32)).astype(F16)


def unit_norm(x_f16: np.ndarray):
    """Split fp16 vectors into (unit fp32 vector, fp32 norm); cache.py:207-210.

    The L2 norm is the correctly rounded one (exact sum of squares in double,
    square root, one rounding to fp32); PyTorch's own reduction order is an
    implementation detail and differs from it by at most one ulp.
    """
    x = x_f16.astype(F32)
    ss = (x.astype(np.float64) ** 2).sum(axis=-1)
    n = np.maximum(np.sqrt(ss).astype(F32), F32(1e-8))
    return (x / n[..., None]).astype(F32), n


def stream_quantize(k_f16, v_f16, signs, codebook):
    """One streamed token: codes and fp16 norms for K and V; cache.py:193-241.

    k_f16, v_f16: (..., hd) fp16.  Returns (k_idx u8, k_norm f16, v_idx u8,
    v_norm f16).
    """
    ku, kn = unit_norm(k_f16)
    vu, vn = unit_norm(v_f16)
    return (quantize_per_token(ku, signs, codebook), kn.astype(F16),
            quantize_per_token(vu, signs, codebook), vn.astype(F16))


def dequant_stream(idx, norm_f16, signs, codebook):
    """fp16 K or V of the streamed tokens; src/shard/cache.py:243-279.

    idx: (s, nkv, hd) u8, norm_f16: (s, nkv) -> (nkv, s, hd) fp16.
    """
    unit = dequantize_per_token(idx, signs, codebook).astype(F32)
    full = (unit * norm_f16.astype(F32)[..., None]).astype(F16)
    return np.ascontiguousarray(np.transpose(full, (1, 0, 2)))


# ---------------------------------------------------------------------------
# RoPE helpers  (reference: src/shard/rope.py:8-30)
# ---------------------------------------------------------------------------


def default_inv_freq(hd: int = 128, theta: float = 500000.0) -> np.ndarray:
    """1 / theta**(2i/hd) in fp32, src/shard/rope.py:47 (torch fp32 pow).

    Evaluated in torch so that the table is bit-identical to what the
    reference derives from a model config.
    """
    import torch
    return (1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))).numpy()


def rotate_half(x):
    h = x.shape[-1] // 2
    return np.concatenate([-x[..., h:], x[..., :h]], axis=-1)


def rope_cos_sin(positions, inv_freq):
    """cos/sin of fp32(pos) * fp32(inv_freq), duplicated over both halves."""
    ph = positions.astype(F32)[:, None] * inv_freq.astype(F32)[None, :]
    emb = np.concatenate([ph, ph], axis=-1).astype(F32)
    return np.cos(emb).astype(F32), np.sin(emb).astype(F32)


def undo_rope(keys, positions, inv_freq):
    """keys (..., T, hd) fp32 -> un-rotated; src/shard/rope.py:20-24."""
    cos, sin = rope_cos_sin(positions, inv_freq)
    return (keys * cos - rotate_half(keys) * sin).astype(F32)


def reapply_rope(keys, positions, inv_freq):
    """src/shard/rope.py:26-30."""
    cos, sin = rope_cos_sin(positions, inv_freq)
    return (keys * cos + rotate_half(keys) * sin).astype(F32)


# ---------------------------------------------------------------------------
# K compressor  (reference: src/shard/cache.py:368-396, 406-420; rope.py:49-161)
# ---------------------------------------------------------------------------


def dp_bit_allocation(variances, total_budget: int):
    """Bits per PCA component, src/shard/rope.py:49-84.

    Dynamic programme over groups of 64 components; each group gets 0, 2, 4, 6
    or 8 bits; cost is counted in units of 16 bits; dropping a group is
    charged 4x its variance, keeping it with b bits var / (3 * 4**b).
    """
    group, options, drop, unit = 64, (0, 2, 4, 6, 8), 4.0, 16
    v = np.asarray(variances, dtype=F32)
    d = v.shape[0]
    ng = (d + group - 1) // group
    sizes = [min(group, d - g * group) for g in range(ng)]
    # torch's fp32 .sum() over <=64 values: evaluate in double and round once.
    gvar = [float(F32(v[g * group: g * group + sizes[g]].astype(np.float64).sum())) for g in range(ng)]
    mu = total_budget // unit + 1
    inf = float("inf")
    best = [[inf] * (mu + 1) for _ in range(ng + 1)]
    choice = [[0] * (mu + 1) for _ in range(ng + 1)]
    best[0] = [0.0] * (mu + 1)
    for g in range(ng):
        for b in range(mu + 1):
            for bits in options:
                cost = 0 if bits == 0 else (sizes[g] * bits + unit - 1) // unit
                if b - cost < 0:
                    continue
                err = gvar[g] * drop if bits == 0 else gvar[g] / (3.0 * (1 << (2 * bits)))
                cand = best[g][b - cost] + err
                if cand < best[g + 1][b]:
                    best[g + 1][b] = cand
                    choice[g + 1][b] = bits
    b = min(range(mu + 1), key=lambda i: best[ng][i])
    alloc = [0] * d
    for g in range(ng - 1, -1, -1):
        bits = choice[g + 1][b]
        for i in range(g * group, g * group + sizes[g]):
            alloc[i] = bits
        if bits > 0:
            b -= (sizes[g] * bits + unit - 1) // unit
    return alloc


def quantize_basis(basis: np.ndarray):
    """int8 basis + per-column fp32 scale; src/shard/cache.py:389-391."""
    col_max = np.maximum(np.abs(basis).max(axis=0), F32(1e-6)).astype(F32)
    scale = (col_max / F32(127.0)).astype(F32)
    q = np.clip(np.rint((basis / scale).astype(F32)), -127, 127).astype(np.int8)
    return q, scale


def project(flat, mean, basis_q, scale):
    """proj = (flat - mean) @ (basis_q * scale), src/shard/cache.py:392.

    fp32 operands; the contraction is evaluated in double and rounded once
    (PyTorch's SGEMM order is not part of the algorithm).
    """
    w = (basis_q.astype(F32) * scale.astype(F32)[None, :]).astype(F32)
    centred = (flat.astype(F32) - mean.astype(F32)[None, :]).astype(F32)
    return (centred.astype(np.float64) @ w.astype(np.float64)).astype(F32)


def k_int4_codes(proj: np.ndarray, alloc):
    """int4 codes of the projected keys: the reference's double quantisation.

    Stage 1 (src/shard/rope.py:95-125, quantize_group): per column
    lo = min, rng = max - min clamped to 1e-6, levels = 2**bits - 1,
    code = round_half_even(clamp((x - lo) / rng, 0, 1) * levels).
    Stage 2 (src/shard/rope.py:127-161, dequantize_group):
    xhat = code / levels * rng + lo  (0 for a 0-bit column).
    Stage 3 (src/shard/cache.py:416-419): coeff_scale = colmax|xhat| / 7
    clamped below at 1e-6; q = clamp(round_half_even(xhat / coeff_scale), -7, 7).
    The zlib/bit-packed byte stream between stages 1 and 2 is pure transport.

    Returns (q int8 (n, keep), coeff_scale fp32 (keep,), xhat fp32).
    """
    proj = proj.astype(F32)
    n, keep = proj.shape
    xhat = np.zeros((n, keep), dtype=F32)
    for j in range(keep):
        bits = int(alloc[j])
        if bits == 0:
            continue
        col = proj[:, j]
        lo = col.min()
        rng = np.maximum(col.max() - lo, F32(1e-6)).astype(F32)
        levels = F32((1 << bits) - 1)
        unit = np.clip(((col - lo) / rng).astype(F32), F32(0), F32(1))
        code = np.clip(np.rint((unit * levels).astype(F32)), 0, levels).astype(F32)
        xhat[:, j] = ((code / levels).astype(F32) * rng).astype(F32) + lo
    col_max = np.maximum(np.abs(xhat).max(axis=0), F32(1e-6)).astype(F32)
    coeff_scale = (col_max / F32(7.0)).astype(F32)
    q = np.clip(np.rint((xhat / coeff_scale[None, :]).astype(F32)), -7, 7).astype(np.int8)
    return q, coeff_scale, xhat


def int4_pack(q: np.ndarray) -> np.ndarray:
    """Two signed nibbles per byte over the flat stream; triton_kernels.py:665-682.

    byte = ((x[2i] + 8) & 15) | (((x[2i+1] + 8) & 15) << 4); odd length is
    padded with one zero value.
    """
    flat = q.reshape(-1).astype(np.int16)
    if flat.shape[0] & 1:
        flat = np.concatenate([flat, np.zeros(1, np.int16)])
    s = ((flat + 8) & 0x0F).astype(np.uint8)
    return (s[0::2] | (s[1::2] << 4)).astype(np.uint8)


def int4_unpack(packed: np.ndarray, n_total: int, rank: int) -> np.ndarray:
    """Inverse of int4_pack as fp16 values; src/shard/attention.py:13-16."""
    lo = (packed & 0x0F).astype(F16) - F16(8.0)
    hi = ((packed >> 4) & 0x0F).astype(F16) - F16(8.0)
    return np.stack([lo, hi], axis=1).reshape(-1)[: n_total * rank].reshape(n_total, rank)


# ---------------------------------------------------------------------------
# V compressor  (reference: src/shard/cache.py:21-61, 398-404)
# ---------------------------------------------------------------------------


def vq_assign(x: np.ndarray, centroids: np.ndarray) -> np.ndarray:
    """Nearest centroid, first minimum wins; triton_kernels.py:689-746.

    dist = (((x0-c0)^2 + (x1-c1)^2) + (x2-c2)^2) + ... in fp32 with one
    rounding per multiply and per add (no fused multiply-add), centroids
    scanned in increasing index with a strict '<'.
    """
    x = x.astype(F32)
    c = centroids.astype(F32)
    n, d = x.shape
    out = np.empty(n, dtype=np.int64)
    step = 1 << 15
    for s in range(0, n, step):
        xb = x[s:s + step]
        dist = np.zeros((xb.shape[0], c.shape[0]), dtype=F32)
        for j in range(d):
            diff = (xb[:, j:j + 1] - c[None, :, j]).astype(F32)
            dist = (dist + (diff * diff).astype(F32)).astype(F32)
        out[s:s + step] = dist.argmin(axis=1)
    return out


def kmeans(data: np.ndarray, init_centroids: np.ndarray, n_iter: int = 30):
    """Lloyd iterations of src/shard/cache.py:21-39 from given initial centroids.

    The reference seeds them with data[randperm(n, seed 42)[:k]] (a
    device-specific PyTorch stream, so the caller supplies them).  Returns the
    updated centroids together with the assignment made against the
    *previous* centroids, as the reference does (cache.py:28, 39); empty
    clusters keep their old centroid (cache.py:35); stops once the largest
    change is below 1e-4 after at least six iterations (cache.py:36-37).
    Cluster means are accumulated in double and rounded once.
    """
    data = data.astype(F32)
    cent = init_centroids.astype(F32).copy()
    k = cent.shape[0]
    idx = None
    for it in range(n_iter):
        idx = vq_assign(data, cent)
        sums = np.zeros((k, data.shape[1]), dtype=np.float64)
        np.add.at(sums, idx, data.astype(np.float64))
        counts = np.bincount(idx, minlength=k).astype(np.float64)
        new = cent.copy()
        nz = counts > 0
        new[nz] = (sums[nz].astype(F32) / counts[nz].astype(F32)[:, None]).astype(F32)
        done = float(np.abs(new - cent).max()) < 1e-4 and it >= 5
        cent = new
        if done:
            break
    return cent, idx


def v_rotate_normalise(v_f16: np.ndarray):
    """Hadamard + per-channel max-abs normalisation; cache.py:398-404, 41-46.

    v_f16: (nkv, n, hd) fp16.  Returns (x fp32 (nkv*n*hd/gs... flattened by
    the caller), rot fp32 (nkv, n, hd), ch_max fp32 (nkv, hd)).
    """
    rot = hadamard(v_f16.astype(F32))
    ch_max = np.maximum(np.abs(rot).max(axis=1), F32(1e-8)).astype(F32)
    x = (rot / ch_max[:, None, :]).astype(F32)
    return x, rot, ch_max


# ---------------------------------------------------------------------------
# Decode attention  (reference: src/shard/attention.py)
# ---------------------------------------------------------------------------


def _h(x):
    return np.asarray(x).astype(F16)


def unrope_query(q_rope_f16, pos_q, inv_freq):
    """fp16 un-rotation of the query at pos_q; src/shard/attention.py:27-32."""
    fr = (F32(pos_q) * inv_freq.astype(F32)).astype(F32)
    emb = np.concatenate([fr, fr])
    cos_q = np.cos(emb).astype(F32).astype(F16)
    sin_q = np.sin(emb).astype(F32).astype(F16)
    q = _h(q_rope_f16)
    return ((q * cos_q).astype(F16) - (rotate_half(q) * sin_q).astype(F16)).astype(F16)


def delta_cos_sin(compress_start, n_comp, pos_q, inv_freq):
    """fp16 cos/sin of fp32(pos_t - pos_q) * fp32(inv_freq); attention.py:76-79."""
    delta = (np.arange(compress_start, compress_start + n_comp, dtype=np.int64) - int(pos_q)).astype(F32)
    phase = (delta[:, None] * inv_freq.astype(F32)[None, :]).astype(F32)
    return np.cos(phase).astype(F32).astype(F16), np.sin(phase).astype(F32).astype(F16)


def compressed_scores(q_rope_f16, gc, pos_q, inv_freq, nkv=8):
    """Scaled scores of the compressed middle; src/shard/attention.py:18-81.

    CPU (non-Triton) branch, lines 69-73, including its fp16 rounding points.
    q_rope_f16: (n_q, hd).  Returns (n_q, n_comp) fp16-valued fp32.
    """
    n_q, hd = q_rope_f16.shape
    hd2 = hd // 2
    gqa = n_q // nkv
    n_total, rank = gc["k_coeffs_shape"]
    n_comp = gc["n_compress"]

    q_n = unrope_query(q_rope_f16, pos_q, inv_freq)
    a, b = q_n[:, :hd2], q_n[:, hd2:]                                   # (n_q, 64) fp16
    basis = _h(gc["k_basis_f16"]).reshape(nkv, hd, rank)
    mean = _h(gc["k_mean_f16"]).reshape(nkv, hd)
    kv = np.arange(n_q) // gqa
    bc, bd = basis[kv, :hd2, :], basis[kv, hd2:, :]                     # (n_q, 64, R)
    mc, md = mean[kv, :hd2], mean[kv, hd2:]
    cs = _h(gc["k_coeff_scale"])

    a_mean = ((a * mc).astype(F16) + (b * md).astype(F16)).astype(F16)  # (n_q, 64)
    b_mean = ((b * mc).astype(F16) - (a * md).astype(F16)).astype(F16)
    A = (((a[..., None] * bc).astype(F16) + (b[..., None] * bd).astype(F16)).astype(F16) * cs).astype(F16)
    Bm = (((b[..., None] * bc).astype(F16) - (a[..., None] * bd).astype(F16)).astype(F16) * cs).astype(F16)

    coefs = int4_unpack(gc["k_coeffs"], n_total, rank)[:n_comp].astype(F32)  # (n_comp, R)
    cos_d, sin_d = delta_cos_sin(gc["compress_start"], n_comp, pos_q, inv_freq)
    cos_t = np.ascontiguousarray(cos_d.T).astype(F32)                   # (64, n_comp)
    sin_t = np.ascontiguousarray(sin_d.T).astype(F32)

    out = np.empty((n_q, n_comp), dtype=F32)
    coefs_t = np.ascontiguousarray(coefs.T)

    def one_head(h):
        U = ((A[h].astype(F32) @ coefs_t).astype(F16) + a_mean[h][:, None]).astype(F16)  # (64, n_comp)
        V = ((Bm[h].astype(F32) @ coefs_t).astype(F16) + b_mean[h][:, None]).astype(F16)
        s1 = (U.astype(F32) * cos_t).sum(axis=0).astype(F16)
        s2 = (V.astype(F32) * sin_t).sum(axis=0).astype(F16)
        s = (s1 + s2).astype(F16)
        out[h] = (s.astype(F32) / F32(math.sqrt(hd))).astype(F16).astype(F32)

    # heads are independent: spread them over the host cores (numpy releases the GIL)
    with ThreadPoolExecutor(max_workers=HOST_THREADS) as pool:
        list(pool.map(one_head, range(n_q)))
    return out


def vq_decode_rot(gc, nkv=8):
    """Rotated-space V of the middle: centroids[idx] * ch_max; cache.py:54-61."""
    cb = _h(gc["v_centroids_f16"]).astype(F32)
    ch = _h(gc["v_ch_f16"]).astype(F32)                                 # (nkv, hd)
    idx = gc["v_indices_u8"].astype(np.int64)                           # (nkv, n, ng)
    n = idx.shape[1]
    return (cb[idx].reshape(nkv, n, -1) * ch[:, None, :]).astype(F32)


def fused_attention_compressed(q_rope_f16, gc, pos_q, inv_freq, nkv=8, stream=None, attn_mask=None,
                               decode=None):
    """Decode attention over [sink | middle | window | fp16 decode buffer | stream];
    attention.py:270-343.

    q_rope_f16: (n_q, hd) fp16 (batch 1, one query token).  ``stream`` is an
    optional dict with k_idx, v_idx (s, nkv, hd) u8, k_norm, v_norm (s, nkv)
    fp16, signs, codebook.  ``decode`` is an optional pair (k, v) of fp16 arrays
    (nkv, s, hd): the tokens a non-streaming cache appends as they are
    (gc["decode_k"], gc["decode_v"], attention.py:307-308, 335-338).
    Returns (n_q, hd) fp16.
    """
    n_q, hd = q_rope_f16.shape
    gqa = n_q // nkv
    n_comp = gc["n_compress"]
    kv = np.arange(n_q) // gqa
    q32 = _h(q_rope_f16).astype(F32)
    inv_sqrt = F32(1.0 / math.sqrt(hd))

    def fp16_scores(k_f16, divide=False):                               # k (nkv, n, hd)
        k = k_f16.astype(F32)[kv]                                       # (n_q, n, hd)
        s = np.einsum("hd,hnd->hn", q32.astype(np.float64), k.astype(np.float64)).astype(F32)
        return (s / F32(math.sqrt(hd))).astype(F32) if divide else (s * inv_sqrt).astype(F32)

    parts = [fp16_scores(_h(gc["sink_k"])),
             compressed_scores(q_rope_f16, gc, pos_q, inv_freq, nkv),
             fp16_scores(_h(gc["win_k"]))]
    n_dec = 0
    if decode is not None and decode[0].shape[1] > 0:
        n_dec = decode[0].shape[1]
        parts.append(fp16_scores(_h(decode[0]), divide=True))
    sk = sv = None
    if stream is not None and stream["k_idx"].shape[0] > 0:
        sk = dequant_stream(stream["k_idx"], stream["k_norm"], stream["signs"], stream["codebook"])
        sv = dequant_stream(stream["v_idx"], stream["v_norm"], stream["signs"], stream["codebook"])
        parts.append(fp16_scores(sk, divide=True))
    scores = np.concatenate(parts, axis=-1).astype(F32)
    if attn_mask is not None:
        scores = (scores + attn_mask.astype(F32)).astype(F32)
    m = scores.max(axis=-1, keepdims=True)
    e = np.exp((scores - m).astype(F32)).astype(F32)
    w = (e / e.astype(np.float64).sum(axis=-1, keepdims=True).astype(F32)).astype(F32)

    n_sink = gc["sink_k"].shape[1]
    n_win = gc["win_k"].shape[1]
    w_sink = w[:, :n_sink]
    w_mid = w[:, n_sink:n_sink + n_comp]
    w_win = w[:, n_sink + n_comp:n_sink + n_comp + n_win]
    off = n_sink + n_comp + n_win

    v_rot = vq_decode_rot(gc, nkv)[kv]                                  # (n_q, n, hd)
    out_rot = np.einsum("hn,hnd->hd", w_mid.astype(np.float64), v_rot.astype(np.float64)).astype(F32)
    out = hadamard(out_rot.astype(F16)).astype(F32)                     # attention.py:112

    def pv(wseg, v_f16):
        v = v_f16.astype(F32)[kv]
        return np.einsum("hn,hnd->hd", wseg.astype(np.float64), v.astype(np.float64)).astype(F32)

    out = (out + pv(w_sink, _h(gc["sink_v"]))).astype(F32)
    out = (out + pv(w_win, _h(gc["win_v"]))).astype(F32)
    if n_dec:
        out = (out + pv(w[:, off:off + n_dec], _h(decode[1]))).astype(F32)
        off += n_dec
    if sv is not None:
        out = (out + pv(w[:, off:off + sv.shape[1]], sv)).astype(F32)
    return out.astype(F16)


def attention_exact(q_rope_f16, gc, pos_q, inv_freq, nkv=8, stream=None, tok_range=None,
                    with_fp16_segments=True, decode=None):
    """Float64 evaluation of the same compressed cache (no fp16 intermediates).

    Dequantises K as src/shard/cache.py:92-113 does (but in double), V as
    line 114, and runs plain softmax attention.  Returns (out (n_q, hd) f64,
    m (n_q,), l (n_q,), acc (n_q, hd)) where acc is the unnormalised
    sum(exp(s - m) * v) -- the (max, sum-exp, partial V) triple exchanged by
    the sequence-split mode.  ``tok_range`` restricts the middle segment.
    """
    n_q, hd = q_rope_f16.shape
    gqa = n_q // nkv
    kv = np.arange(n_q) // gqa
    n_total, rank = gc["k_coeffs_shape"]
    n_comp = gc["n_compress"]
    lo, hi = (0, n_comp) if tok_range is None else tok_range
    coef = int4_unpack(gc["k_coeffs"], n_total, rank)[:n_comp].astype(np.float64)[lo:hi]
    coef = coef * _h(gc["k_coeff_scale"]).astype(np.float64)
    basis = _h(gc["k_basis_f16"]).astype(np.float64)
    k_n = coef @ basis.T + _h(gc["k_mean_f16"]).astype(np.float64)      # (n, nkv*hd)
    k_n = k_n.reshape(hi - lo, nkv, hd).transpose(1, 0, 2)
    pos = np.arange(gc["compress_start"] + lo, gc["compress_start"] + hi)
    ph = pos.astype(F32)[:, None] * inv_freq.astype(F32)[None, :]
    emb = np.concatenate([ph, ph], -1).astype(np.float64)
    k_mid = k_n * np.cos(emb) + rotate_half(k_n) * np.sin(emb)
    v_rot = vq_decode_rot(gc, nkv).astype(np.float64)[:, lo:hi]
    v_mid = hadamard(v_rot)
    ks, vs = [k_mid], [v_mid]
    if with_fp16_segments:
        ks = [_h(gc["sink_k"]).astype(np.float64), k_mid, _h(gc["win_k"]).astype(np.float64)]
        vs = [_h(gc["sink_v"]).astype(np.float64), v_mid, _h(gc["win_v"]).astype(np.float64)]
        if decode is not None and decode[0].shape[1] > 0:
            ks.append(_h(decode[0]).astype(np.float64))
            vs.append(_h(decode[1]).astype(np.float64))
        if stream is not None and stream["k_idx"].shape[0] > 0:
            ks.append(dequant_stream(stream["k_idx"], stream["k_norm"], stream["signs"],
                                     stream["codebook"]).astype(np.float64))
            vs.append(dequant_stream(stream["v_idx"], stream["v_norm"], stream["signs"],
                                     stream["codebook"]).astype(np.float64))
    k = np.concatenate(ks, axis=1)[kv]
    v = np.concatenate(vs, axis=1)[kv]
    s = np.einsum("hd,hnd->hn", _h(q_rope_f16).astype(np.float64), k) / math.sqrt(hd)
    if s.shape[1] == 0:
        m = np.full(n_q, -np.inf)
        return np.zeros((n_q, hd)), m, np.zeros(n_q), np.zeros((n_q, hd))
    m = s.max(axis=-1)
    e = np.exp(s - m[:, None])
    l = e.sum(axis=-1)
    acc = np.einsum("hn,hnd->hd", e, v)
    return acc / l[:, None], m, l, acc


def lse_merge(ms, ls, accs):
    """Log-sum-exp combine of per-part (m, l, acc); src/shard/attention.py:262-266.

    ms, ls: (parts, n_q); accs: (parts, n_q, hd).  Parts are combined in index
    order: M = max m; out = sum e^{m-M} acc / sum e^{m-M} l.
    """
    ms = np.asarray(ms, dtype=np.float64)
    big = ms.max(axis=0)
    w = np.exp(ms - big[None, :])
    w = np.where(np.isfinite(ms), w, 0.0)
    z = (w * np.asarray(ls, dtype=np.float64)).sum(axis=0)
    num = (w[..., None] * np.asarray(accs, dtype=np.float64)).sum(axis=0)
    return num / z[:, None]


# ---------------------------------------------------------------------------
# Accounting  (reference: src/shard/cache.py:462-539)
# ---------------------------------------------------------------------------


def fp16_equivalent_bytes(seq, nkv, hd, layers):
    """K and V in fp16 for every layer; src/shard/cache.py:528."""
    return seq * nkv * hd * 4 * layers
