"""Generate the golden fixtures under tests/golden/ from the reference itself.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own Python package (CPU / PyTorch-fallback path),
drives it on small seeded inputs and stores inputs + outputs as .npz files.
The fixtures travel with the repository; the reference checkout does not, so
nothing else in the tests or the benchmark reads it.

The only modification applied to the reference is a two-token device shim:
`Cache._build_gpu_format` hard-codes the device string "cuda" and calls
`torch.cuda.empty_cache()`; both are rewritten to their CPU equivalents in a
copy of the function's source that is then executed inside the reference
module's namespace.
"""
from __future__ import annotations

import inspect
import json
import math
import os
import sys
import textwrap

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import synth  # noqa: E402  (tests/synth.py)


def load_reference(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import shard  # noqa: F401
    import shard.cache as rc
    src = textwrap.dedent(inspect.getsource(rc.Cache._build_gpu_format))
    src = src.replace('dev = "cuda"', 'dev = "cpu"').replace("torch.cuda.empty_cache()", "pass")
    ns = {}
    exec(src, rc.__dict__, ns)
    rc.Cache._build_gpu_format = ns["_build_gpu_format"]
    return rc


def t2n(t):
    return t.detach().cpu().numpy()


def save(name, **arrays):
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrays)
    print(f"  wrote {name}: {os.path.getsize(path) / 1024:.0f} KiB")


def gc_arrays(gc, prefix=""):
    keys = ["k_coeffs", "k_coeff_scale", "k_basis_q", "k_basis_scale", "k_basis_f16", "k_mean",
            "k_mean_f16", "v_indices_u8", "v_centroids_f16", "v_ch_f16", "sink_k", "sink_v",
            "win_k", "win_v"]
    out = {prefix + k: t2n(gc[k]) for k in keys}
    out[prefix + "meta"] = np.array([gc["k_coeffs_shape"][0], gc["k_coeffs_shape"][1],
                                     gc["n_compress"], gc["batch"], gc["compress_start"]], np.int64)
    return out


def build_cache(rc, k, v, inv_freq, streaming=False, k_target_cr=20.0):
    cache = rc.Cache(head_dim=128, num_layers=1, n_kv_heads=8, device="cpu",
                     k_target_cr=k_target_cr, rope_inv_freq=inv_freq)
    cache._streaming = streaming
    cache.layers[0].update(k, v)
    return cache


def decode_buffer_fixture(rc, ra, inv_freq):
    """configs[0] cache in the reference's DEFAULT mode (no stream: decoded tokens are appended to
    the fp16 buffers decode_k / decode_v, cache.py:168-181): three decode steps, each one update
    followed by fused_attention_compressed.  Only the tokens, queries and outputs are stored; the
    compressed tensors are those of cfg0.npz (compression is seeded), which is asserted here."""
    k, v, q = synth.make_kvq(2048, 0)
    cache = build_cache(rc, k, v, inv_freq, streaming=False)
    cache.compress()
    layer = cache.layers[0]
    gc = layer._gpu_compressed
    ref = np.load(os.path.join(HERE, "cfg0.npz"))
    for key in ("k_coeffs", "v_indices_u8", "k_basis_q", "v_centroids_f16"):
        assert np.array_equal(t2n(gc[key]), ref[key]), key
    cache._fused_decode_update = True
    toks_k, toks_v, qs, outs = [], [], [], []
    for j in range(3):
        kt, vt, qt = synth.make_token(700 + j)
        layer.update(kt, vt)
        toks_k.append(kt)
        toks_v.append(vt)
        qs.append(qt)
        outs.append(ra.fused_attention_compressed(qt, layer, 2048 + j, inv_freq, None))
    assert gc["decode_k"].shape[2] == 3
    save("cfg0_decbuf.npz", dec_k=t2n(torch.cat(toks_k, 2)), dec_v=t2n(torch.cat(toks_v, 2)),
         dec_q=t2n(torch.cat(qs, 2)), dec_out=t2n(torch.cat(outs, 2)))


def multi_token_fixture(rc, inv_freq):
    """configs[0] cache, then an 8-token continuation in ONE forward, the way the reference serves
    it (hidden_states.shape[1] > 1 after compression, src/shard/attention.py:357-362): `update`
    appends the tokens and returns the fully dequantised K / V (`_ensure_dequant`,
    src/shard/cache.py:87-124), and the stock attention runs over them with a causal mask.  Both
    append modes: the 8-bit stream and the default fp16 decode buffer."""
    import math
    out = {}
    g = torch.Generator().manual_seed(909)
    k_new = torch.randn(1, 8, 8, 128, generator=g).half()
    v_new = torch.randn(1, 8, 8, 128, generator=g).half()
    q_new = torch.randn(1, 32, 8, 128, generator=g).half()
    for tag, streaming in (("st", True), ("dec", False)):
        k, v, q = synth.make_kvq(2048, 0)
        cache = build_cache(rc, k, v, inv_freq, streaming=streaming)
        cache.compress()
        layer = cache.layers[0]
        keys, values = layer.update(k_new, v_new)                  # non-fused update: full dequantised K / V
        assert keys.shape == (1, 8, 2048 + 8, 128)
        kk = keys.float().repeat_interleave(4, dim=1)
        vv = values.float().repeat_interleave(4, dim=1)
        sc = torch.einsum("bhsd,bhkd->bhsk", q_new.float(), kk) / math.sqrt(128)
        mask = torch.full((8, 2048 + 8), float("-inf"))
        for j in range(8):
            mask[j, : 2048 + j + 1] = 0.0
        w = torch.softmax(sc + mask, dim=-1)
        out[tag + "_out"] = t2n(torch.einsum("bhsk,bhkd->bhsd", w, vv).half())
    save("cfg0_multi.npz", k_new=t2n(k_new), v_new=t2n(v_new), q_new=t2n(q_new), **out)


def main(ref_root, only=None):
    rc = load_reference(ref_root)
    import shard.attention as ra
    import shard.rope as rr
    import shard.streaming as rs
    import shard.triton_kernels as rk

    torch.manual_seed(0)
    inv_freq = synth.rope_inv_freq()
    if only == "decbuf":
        decode_buffer_fixture(rc, ra, inv_freq)
        return
    if only == "multi":
        multi_token_fixture(rc, inv_freq)
        return

    # ---- Lloyd-Max codebook, signs, inv_freq --------------------------------
    cb = rs.lloyd_max_codebook(128, 8)
    signs = []
    for li in range(4):
        g = torch.Generator(device="cpu").manual_seed(42 + li * 7919)
        signs.append((torch.randint(0, 2, (128,), generator=g) * 2 - 1).float())
    save("codebook.npz", codebook=t2n(cb), signs=t2n(torch.stack(signs)), inv_freq=t2n(inv_freq))

    # ---- stream quantizer ----------------------------------------------------
    g = torch.Generator().manual_seed(11)
    ks = (torch.randn(24, 8, 128, generator=g) * torch.rand(24, 8, 1, generator=g) * 3).half()
    vs = torch.randn(24, 8, 128, generator=g).half()
    vs[:, :, 5] *= 20
    sg = signs[1]

    def unit(t):
        t = t.float()
        n = t.norm(dim=-1).clamp(min=1e-8)
        return t / n.unsqueeze(-1), n

    ku, kn = unit(ks)
    vu, vn = unit(vs)
    kidx, _, _ = rs.quantize_per_token(ku, 8, sg)
    vidx, _, _ = rs.quantize_per_token(vu, 8, sg)
    kdq = rs.dequantize_per_token(kidx, 8, sg)
    save("stream.npz", k=t2n(ks), v=t2n(vs), signs=t2n(sg), k_unit=t2n(ku), v_unit=t2n(vu),
         k_norm=t2n(kn), v_norm=t2n(vn), k_idx=t2n(kidx), v_idx=t2n(vidx), k_dequnit=t2n(kdq))

    # ---- undo RoPE + Hadamard ------------------------------------------------
    g = torch.Generator().manual_seed(12)
    kmid = torch.randn(1, 8, 40, 128, generator=g).half()
    pos = torch.cat([torch.arange(4, 24), torch.arange(100000, 100010), torch.arange(131000, 131010)])
    un = rr.undo_rope(kmid.float(), pos, inv_freq)
    re = rr.reapply_rope(un, pos, inv_freq)
    vmid = torch.randn(8, 40, 128, generator=g).half()
    vmid[:, :, 17] *= 20
    rot = rc.hadamard(vmid.float())
    ch_max = rot.abs().amax(dim=1).clamp(min=1e-8)
    xn = rot / ch_max.unsqueeze(1)
    rot16 = rc.hadamard(vmid)
    save("rope_hadamard.npz", k=t2n(kmid), pos=t2n(pos), undo=t2n(un), reapply=t2n(re),
         v=t2n(vmid), rot=t2n(rot), ch_max=t2n(ch_max), x=t2n(xn), rot16=t2n(rot16))

    # ---- DP bit allocation ---------------------------------------------------
    cases = []
    g = torch.Generator().manual_seed(13)
    for d, budget, decay in [(192, 819, 0.02), (192, 1024, 0.05), (192, 409, 0.01), (187, 819, 0.03),
                             (128, 512, 0.1), (64, 64, 0.5), (192, 64, 0.02), (192, 2048, 0.001)]:
        ev = (torch.rand(d, generator=g) + 0.1) * torch.exp(-decay * torch.arange(d).float())
        ev = ev.sort(descending=True).values
        cases.append({"eig": [float(x) for x in ev], "budget": budget,
                      "alloc": rr.dp_bit_allocation(ev, budget)})
    with open(os.path.join(HERE, "dp_alloc.json"), "w") as f:
        json.dump(cases, f)
    print("  wrote dp_alloc.json")

    # ---- K quantiser (double quantisation + int4 pack) ----------------------
    g = torch.Generator().manual_seed(14)
    kq = {}
    for tag, n, alloc in [("a", 301, [4] * 192), ("b", 128, [8] * 64 + [4] * 64 + [2] * 64),
                          ("c", 77, [6] * 64 + [2] * 62), ("d", 50, [4] * 64 + [0] * 64)]:
        keep = len(alloc)
        proj = torch.randn(n, keep, generator=g) * torch.exp(-0.01 * torch.arange(keep).float()) * 3
        coeffs = rr.dequantize_group(rr.quantize_group(proj, alloc), alloc, n, "cpu")
        col_max = coeffs.abs().amax(dim=0).clamp(min=1e-6)
        cs = col_max / 7.0
        q = (coeffs / cs).round().clamp(-7, 7).to(torch.int8)
        kq.update({f"{tag}_proj": t2n(proj), f"{tag}_alloc": np.array(alloc, np.int32),
                   f"{tag}_xhat": t2n(coeffs), f"{tag}_scale": t2n(cs), f"{tag}_q": t2n(q),
                   f"{tag}_packed": t2n(rk.int4_pack(q))})
    # basis quantisation + projection on a small problem
    flat = torch.randn(96, 1024, generator=g)
    mean = flat.mean(dim=0)
    basis = torch.linalg.qr(torch.randn(1024, 64, generator=g)).Q
    col_max = basis.abs().max(dim=0).values.clamp(min=1e-6)
    scale = col_max / 127.0
    basis_q = (basis / scale).round().clamp(-127, 127).to(torch.int8)
    proj = (flat - mean.float()) @ (basis_q.float() * scale.float())
    kq.update(p_flat=t2n(flat), p_mean=t2n(mean), p_basis=t2n(basis), p_basis_q=t2n(basis_q),
              p_scale=t2n(scale), p_proj=t2n(proj))
    save("kquant.npz", **kq)

    # ---- VQ assign + k-means -------------------------------------------------
    g = torch.Generator().manual_seed(15)
    x = torch.randn(10000, 4, generator=g)
    c = torch.randn(256, 4, generator=g)
    idx = rk.vq_assign(x, c)
    data = torch.rand(6000, 4, generator=g) * 2 - 1
    calls = []
    orig = rk.vq_assign

    def spy(d, cent):
        out = orig(d, cent)
        calls.append((cent.clone(), out.clone()))
        return out

    rk.vq_assign = spy
    cent, kidx2 = rc.kmeans(data, 256, n_iter=30)
    rk.vq_assign = orig
    gg = torch.Generator(device="cpu").manual_seed(42)
    init = data[torch.randperm(6000, generator=gg)[:256]].clone()
    assert torch.equal(init, calls[0][0])
    save("vq.npz", x=t2n(x), c=t2n(c), idx=t2n(idx), km_data=t2n(data), km_init=t2n(init),
         km_centroids=t2n(cent), km_idx=t2n(kidx2), km_prev=t2n(calls[-1][0]),
         km_iters=np.array(len(calls)))

    # ---- full chain, 512 tokens (n_comp = 444): stage captures ---------------
    k, v, q = synth.make_kvq(512, 7)
    cap = {}
    orig_qg = rr.quantize_group

    def spy_qg(proj, alloc):
        cap["proj"] = proj.clone()
        cap["alloc"] = list(alloc)
        return orig_qg(proj, alloc)

    rc.quantize_group = spy_qg
    cache = build_cache(rc, k, v, inv_freq)
    cache.compress()
    rc.quantize_group = orig_qg
    gc = cache.layers[0]._gpu_compressed
    pos_q = 512
    out = ra.fused_attention_compressed(q, cache.layers[0], pos_q, inv_freq, None)
    sc = ra.compressed_scores(q, gc, pos_q, 32, 8, 128, inv_freq)
    save("chain512.npz", **gc_arrays(gc), q=t2n(q), pos_q=np.array(pos_q), out=t2n(out),
         scores=t2n(sc).astype(np.float16), proj=t2n(cap["proj"]),
         alloc=np.array(cap["alloc"], np.int32),
         mem=np.array([cache.memory_bytes(), cache.clean_memory_bytes(),
                       cache.fp16_equivalent_bytes()], np.int64))

    # ---- configs[0]: 2048 tokens, seed 0, with and without a stream ---------
    k, v, q = synth.make_kvq(2048, 0)
    cache = build_cache(rc, k, v, inv_freq, streaming=True)
    cache.compress()
    layer = cache.layers[0]
    gc = layer._gpu_compressed
    pos_q = 2048
    out0 = ra.fused_attention_compressed(q, layer, pos_q, inv_freq, None)
    out0_full = ra.fused_attention_compressed_full(q, layer, pos_q, inv_freq, None)
    sc0 = ra.compressed_scores(q, gc, pos_q, 32, 8, 128, inv_freq)
    mem0 = [cache.memory_bytes(), cache.clean_memory_bytes(), cache.fp16_equivalent_bytes()]
    # five streamed tokens, each followed by one decode step
    toks_k, toks_v, qs, outs = [], [], [], []
    for j in range(5):
        kt, vt, qt = synth.make_token(500 + j)
        layer._stream_append(kt, vt, 2048 + j)
        toks_k.append(kt)
        toks_v.append(vt)
        qs.append(qt)
        outs.append(ra.fused_attention_compressed(qt, layer, 2048 + j, inv_freq, None))
    s = gc["stream_n"]
    save("cfg0.npz", **gc_arrays(gc), q=t2n(q), pos_q=np.array(pos_q), out=t2n(out0),
         out_full=t2n(out0_full), scores=t2n(sc0).astype(np.float16),
         mem=np.array(mem0, np.int64),
         st_k=t2n(torch.cat(toks_k, 2)), st_v=t2n(torch.cat(toks_v, 2)), st_q=t2n(torch.cat(qs, 2)),
         st_out=t2n(torch.cat(outs, 2)), st_signs=t2n(gc["signs"]),
         st_k_idx=t2n(gc["k_idx_buf"][:s]), st_v_idx=t2n(gc["v_idx_buf"][:s]),
         st_k_norm=t2n(gc["k_norm_buf"][:s]), st_v_norm=t2n(gc["v_norm_buf"][:s]),
         mem_stream=np.array([cache.memory_bytes(), cache.clean_memory_bytes(),
                              cache.fp16_equivalent_bytes()], np.int64))
    decode_buffer_fixture(rc, ra, inv_freq)
    multi_token_fixture(rc, inv_freq)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit("usage: make_golden.py <reference checkout> [decbuf|multi]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else None)
