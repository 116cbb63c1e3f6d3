"""The decode entry point that carries its own scratch, for callers that cannot allocate.

Collected last on purpose (file name): a run that stops at the first failure has then
already exercised every other test.  The check: through the C ABI, the self-contained
entry point must give what the regular entry point (caller-provided workspace) gives, on
two calls in a row that share the library's built-in scratch area -- the second call sees
the first call's leftovers and must not be disturbed by them.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import load_golden, tol_ok

pytestmark = pytest.mark.gpu


def _run_both(layer, q_np, pos_q):
    """Returns (regular, self-contained) fp16 outputs for one query."""
    from shard_b200 import _lib, ops
    from shard_b200.attention import _phase_for, _seq_record, decode_layer
    from shard_b200.streaming import get_codebook
    lib = _lib.load()
    dev = "cuda"
    q = torch.from_numpy(q_np).to(dev).view(1, q_np.shape[0], 1, 128)
    ref = decode_layer(q, layer, pos_q).clone()                  # caller-owned workspace

    gc, cache = layer._gpu_compressed, layer._cache_ref
    n_q, nkv, n_comp = q_np.shape[0], cache._n_kv_heads, gc["n_compress"]
    out = torch.full((n_q, 128), float("nan"), dtype=torch.float16, device=dev)
    seq = _seq_record(gc, dev)
    seq.q, seq.out = q.view(n_q, 128).data_ptr(), out.data_ptr()
    seq.phase = _phase_for(cache, gc, pos_q, 0, n_comp, dev).data_ptr()
    n_stream = gc.get("stream_n", 0)
    shape = ops.make_shape(n_q, nkv, gc["k_rank_kernel"], n_comp, 0, n_comp, gc["sink_k"].shape[2],
                           gc["win_k"].shape[2], n_stream, pos_q)
    cb = get_codebook(128, 8, dev) if n_stream else None
    rc = lib.shard_b200_decode_attn_noalloc(C.addressof(seq), C.byref(shape), cache._inv_freq(dev).data_ptr(),
                                            None if cb is None else cb.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.shard_b200_status_string(rc)
    torch.cuda.synchronize()
    return ref.cpu().numpy(), out.cpu().numpy()


def test_self_contained_decode_matches_regular_entry_point_twice():
    from gpu_helpers import FakeCache, FakeLayer, gc_to_device, layer_from_golden, random_gc, random_query
    from oracle import shard_oracle as O
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    g = load_golden("chain512.npz")
    small, _ = layer_from_golden(g)
    big = FakeLayer(gc_to_device(random_gc(6000, seed=77)), FakeCache(torch.from_numpy(O.default_inv_freq())))
    # first call: many chunks; second call: a smaller problem that reuses (part of) the same scratch
    for layer, q_np, pos_q in ((big, random_query(seed=5), 6100), (small, g["q"][0, :, 0, :], int(g["pos_q"])),
                               (big, random_query(seed=6), 6101)):
        ref, got = _run_both(layer, q_np, pos_q)
        assert np.isfinite(got).all()
        # same launch plan, same records, same combine order: the two entry points agree bit for bit
        assert np.array_equal(got, ref), np.abs(got.astype(np.float32) - ref.astype(np.float32)).max()
    assert tol_ok(got, O.attention_exact(random_query(seed=6), random_gc(6000, seed=77), 6101,
                                         O.default_inv_freq())[0], atol=1.5e-3, rtol=5e-3)
    # no launch gave up on a wait: the status word kept inside the built-in scratch reads 0
    from shard_b200 import ops
    assert ops.decode_status(None) == 0


def test_self_contained_decode_refuses_oversized_requests():
    from shard_b200 import _lib, ops
    lib = _lib.load()
    seq = _lib.ShardSeq()
    shape = ops.make_shape(4 * 512, 512, 192, 200000, 0, 200000, 4, 64, 0, 200100)   # 2048 heads: > 2 MiB of records
    rc = lib.shard_b200_decode_attn_noalloc(C.addressof(seq), C.byref(shape), 1, None, None)
    assert rc == -4
    assert b"built-in" in lib.shard_b200_status_string(rc)
