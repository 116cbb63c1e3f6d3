"""Pins the numpy oracle against outputs of the reference's own implementation.

The fixtures were produced by tests/golden/make_golden.py from the reference's
CPU path.  Integer stages must match bit for bit; floating stages within the
stated tolerance.
"""
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN, gc_from_golden, load_golden, tol_ok
from oracle import shard_oracle as O


def test_codebook_bit_exact():
    g = load_golden("codebook.npz")
    cb = O.lloyd_max_codebook(128, 8)
    assert cb.dtype == np.float32 and np.array_equal(cb, g["codebook"])
    for li in range(4):
        assert np.array_equal(O.stream_signs(li), g["signs"][li])
    assert np.array_equal(O.default_inv_freq(), g["inv_freq"])


def test_stream_codes_given_unit_vectors():
    g = load_golden("stream.npz")
    cb = O.lloyd_max_codebook(128, 8)
    assert np.array_equal(O.quantize_per_token(g["k_unit"], g["signs"], cb), g["k_idx"])
    assert np.array_equal(O.quantize_per_token(g["v_unit"], g["signs"], cb), g["v_idx"])
    assert np.array_equal(O.dequantize_per_token(g["k_idx"], g["signs"], cb), g["k_dequnit"])


def test_stream_from_fp16_tokens():
    """Norms within one fp32 ulp of PyTorch's; codes equal except at bucket edges."""
    g = load_golden("stream.npz")
    cb = O.lloyd_max_codebook(128, 8)
    ki, kn, vi, vn = O.stream_quantize(g["k"], g["v"], g["signs"], cb)
    for mine, ref in ((kn, g["k_norm"]), (vn, g["v_norm"])):
        ref16 = ref.astype(np.float16)
        assert np.mean(mine != ref16) < 1e-2
        assert np.allclose(mine.astype(np.float32), ref, rtol=1e-3)
    for mine, ref in ((ki, g["k_idx"]), (vi, g["v_idx"])):
        diff = mine.astype(int) - ref.astype(int)
        assert np.abs(diff).max() <= 1
        assert np.mean(diff != 0) < 1e-3


def test_rope_and_hadamard():
    g = load_golden("rope_hadamard.npz")
    inv_freq = O.default_inv_freq()
    un = O.undo_rope(g["k"].astype(np.float32), g["pos"], inv_freq)
    assert np.allclose(un, g["undo"], atol=2e-6, rtol=0)
    re = O.reapply_rope(g["undo"], g["pos"], inv_freq)
    assert np.allclose(re, g["reapply"], atol=2e-6, rtol=0)
    x, rot, ch = O.v_rotate_normalise(g["v"])
    assert np.array_equal(rot, g["rot"])
    assert np.array_equal(ch, g["ch_max"])
    assert np.array_equal(x, g["x"])
    assert np.array_equal(O.hadamard(g["v"]), g["rot16"])


def test_dp_bit_allocation():
    with open(os.path.join(GOLDEN, "dp_alloc.json")) as f:
        cases = json.load(f)
    for c in cases:
        assert O.dp_bit_allocation(np.array(c["eig"], np.float32), c["budget"]) == c["alloc"]


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_k_int4_codes_bit_exact(tag):
    g = load_golden("kquant.npz")
    q, cs, xhat = O.k_int4_codes(g[f"{tag}_proj"], g[f"{tag}_alloc"])
    assert np.array_equal(xhat, g[f"{tag}_xhat"])
    assert np.array_equal(cs, g[f"{tag}_scale"])
    assert np.array_equal(q, g[f"{tag}_q"])
    assert np.array_equal(O.int4_pack(q), g[f"{tag}_packed"])


def test_basis_quant_and_projection():
    g = load_golden("kquant.npz")
    bq, scale = O.quantize_basis(g["p_basis"])
    assert np.array_equal(bq, g["p_basis_q"]) and np.array_equal(scale, g["p_scale"])
    proj = O.project(g["p_flat"], g["p_mean"], bq, scale)
    assert np.allclose(proj, g["p_proj"], atol=2e-5, rtol=1e-5)


def test_chain512_int4_codes_from_captured_projection(golden_chain512):
    g = golden_chain512
    q, cs, _ = O.k_int4_codes(g["proj"], g["alloc"])
    assert np.array_equal(O.int4_pack(q), g["k_coeffs"])
    assert np.array_equal(cs.astype(np.float16), g["k_coeff_scale"])


def test_vq_assign_matches_reference():
    g = load_golden("vq.npz")
    idx = O.vq_assign(g["x"], g["c"])
    # the reference's CPU branch is cdist().argmin(); kernel_test.py demands
    # zero mismatches on exactly this shape
    assert np.array_equal(idx, g["idx"])


def test_kmeans_matches_reference():
    g = load_golden("vq.npz")
    cent, idx = O.kmeans(g["km_data"], g["km_init"], n_iter=30)
    assert np.array_equal(O.vq_assign(g["km_data"], g["km_prev"]), g["km_idx"])
    assert np.mean(idx != g["km_idx"]) < 2e-3
    assert np.allclose(cent, g["km_centroids"], atol=5e-3)


def test_compressed_scores_cfg0(golden_cfg0):
    g = golden_cfg0
    gc = gc_from_golden(g)
    s = O.compressed_scores(g["q"][0, :, 0, :], gc, int(g["pos_q"]), O.default_inv_freq())
    ref = g["scores"][0, :, 0, :].astype(np.float32)
    # fp16-valued scores; GEMM association may flip the last fp16 bit
    assert np.abs(s - ref).max() <= 4e-3
    assert np.mean(s != ref) < 0.05


def test_fused_attention_cfg0(golden_cfg0):
    g = golden_cfg0
    gc = gc_from_golden(g)
    inv_freq = O.default_inv_freq()
    out = O.fused_attention_compressed(g["q"][0, :, 0, :], gc, int(g["pos_q"]), inv_freq)
    ref = g["out"][0, :, 0, :]
    assert np.abs(out.astype(np.float32) - ref.astype(np.float32)).max() <= 1e-3
    # the exact evaluation of the same cache sits inside the decode tolerance
    exact, m, l, acc = O.attention_exact(g["q"][0, :, 0, :], gc, int(g["pos_q"]), inv_freq)
    assert tol_ok(exact, ref)
    assert tol_ok(exact, g["out_full"][0, :, 0, :], atol=4e-3)


def test_fused_attention_cfg0_with_stream(golden_cfg0):
    g = golden_cfg0
    gc = gc_from_golden(g)
    inv_freq = O.default_inv_freq()
    cb = O.lloyd_max_codebook(128, 8)
    assert np.array_equal(O.stream_signs(0), g["st_signs"])
    for j in range(5):
        stream = dict(k_idx=g["st_k_idx"][:j + 1, 0], v_idx=g["st_v_idx"][:j + 1, 0],
                      k_norm=g["st_k_norm"][:j + 1, 0], v_norm=g["st_v_norm"][:j + 1, 0],
                      signs=g["st_signs"], codebook=cb)
        out = O.fused_attention_compressed(g["st_q"][0, :, j, :], gc, 2048 + j, inv_freq, stream=stream)
        ref = g["st_out"][0, :, j, :]
        assert np.abs(out.astype(np.float32) - ref.astype(np.float32)).max() <= 1e-3
    ki, kn, vi, vn = O.stream_quantize(g["st_k"][0].transpose(1, 0, 2), g["st_v"][0].transpose(1, 0, 2),
                                       g["st_signs"], cb)
    assert np.array_equal(ki, g["st_k_idx"][:, 0]) and np.array_equal(vi, g["st_v_idx"][:, 0])
    assert np.array_equal(kn, g["st_k_norm"][:, 0]) and np.array_equal(vn, g["st_v_norm"][:, 0])


def test_fused_attention_cfg0_with_fp16_decode_buffer(golden_cfg0):
    """The reference's default (non-streaming) mode: decoded tokens appended as fp16 rows."""
    g, d = golden_cfg0, load_golden("cfg0_decbuf.npz")
    gc = gc_from_golden(g)
    inv_freq = O.default_inv_freq()
    for j in range(3):
        dec = (d["dec_k"][0][:, :j + 1], d["dec_v"][0][:, :j + 1])
        out = O.fused_attention_compressed(d["dec_q"][0, :, j, :], gc, 2048 + j, inv_freq, decode=dec)
        ref = d["dec_out"][0, :, j, :]
        assert np.abs(out.astype(np.float32) - ref.astype(np.float32)).max() <= 1e-3
        # the float64 evaluation of the same cache (the GPU tests' second yardstick) stays within
        # the reference's own fp16 noise of it
        exact, *_ = O.attention_exact(d["dec_q"][0, :, j, :], gc, 2048 + j, inv_freq, decode=dec)
        assert np.abs(ref.astype(np.float64) - exact).max() <= 5e-3


def test_fused_attention_chain512(golden_chain512):
    g = golden_chain512
    gc = gc_from_golden(g)
    out = O.fused_attention_compressed(g["q"][0, :, 0, :], gc, int(g["pos_q"]), O.default_inv_freq())
    assert np.abs(out.astype(np.float32) - g["out"][0, :, 0, :].astype(np.float32)).max() <= 1e-3


def test_lse_merge_of_token_ranges_equals_whole(golden_chain512):
    g = golden_chain512
    gc = gc_from_golden(g)
    inv_freq = O.default_inv_freq()
    q = g["q"][0, :, 0, :]
    whole, *_ = O.attention_exact(q, gc, 512, inv_freq, with_fp16_segments=False)
    n = gc["n_compress"]
    cuts = [0, 100, 101, 300, n]
    parts = [O.attention_exact(q, gc, 512, inv_freq, tok_range=(a, b), with_fp16_segments=False)
             for a, b in zip(cuts[:-1], cuts[1:])]
    merged = O.lse_merge([p[1] for p in parts], [p[2] for p in parts], [p[3] for p in parts])
    assert np.allclose(merged, whole, atol=1e-12)
