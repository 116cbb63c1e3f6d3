"""Helpers shared by the GPU parity tests: fixtures -> device dictionaries, random caches."""
import numpy as np
import torch

from conftest import gc_from_golden


class FakeCache:
    """The few attributes of shard_b200.Cache that decode_layer touches."""

    def __init__(self, inv_freq, nkv=8, hd=128):
        self._n_kv_heads = nkv
        self.head_dim = hd
        self._rope_inv_freq = inv_freq
        self._decode_ws = None
        self._phase = None
        self._phase_key = None
        self._inv_freq_dev = None

    def _inv_freq(self, dev):
        if self._inv_freq_dev is None:
            self._inv_freq_dev = self._rope_inv_freq.to(dev, torch.float32).contiguous()
        return self._inv_freq_dev


class FakeLayer:
    def __init__(self, gc, cache, layer_idx=0):
        self._gpu_compressed = gc
        self._cache_ref = cache
        self.layer_idx = layer_idx


def gc_to_device(gc_np, dev="cuda", nkv=8):
    """numpy dictionary (oracle form: fp16 segments (nkv, n, hd)) -> torch dictionary of the
    product (segments (1, nkv, n, hd)) with the kernel-side format attached."""
    from shard_b200.cache import attach_kernel_format
    gc = {}
    for k, v in gc_np.items():
        if isinstance(v, np.ndarray):
            t = torch.from_numpy(np.ascontiguousarray(v)).to(dev)
            if k in ("sink_k", "sink_v", "win_k", "win_v"):
                t = t.unsqueeze(0)
            gc[k] = t
        else:
            gc[k] = v
    attach_kernel_format(gc, nkv)
    return gc


def layer_from_golden(g, dev="cuda"):
    gc_np = gc_from_golden(g)
    inv_freq = torch.from_numpy(np.load(__import__("os").path.join(
        __import__("conftest").GOLDEN, "codebook.npz"))["inv_freq"])
    cache = FakeCache(inv_freq)
    return FakeLayer(gc_to_device(gc_np, dev), cache), gc_np


def random_gc(n_comp, rank=192, nkv=8, n_sink=4, n_win=64, compress_start=None, seed=0):
    """A synthetic compressed layer in oracle (numpy) form with plausible magnitudes."""
    rng = np.random.default_rng(seed)
    hd = 128
    p = nkv * hd
    if compress_start is None:
        compress_start = n_sink
    q = rng.integers(-7, 8, size=(n_comp, rank)).astype(np.int8)
    from oracle import shard_oracle as O
    decay = np.exp(-0.01 * np.arange(rank))
    basis_q = rng.integers(-127, 128, size=(p, rank)).astype(np.int8)
    basis_scale = (0.08 / 127 * (0.5 + rng.random(rank))).astype(np.float16)
    coeff_scale = (decay * (0.3 + 0.2 * rng.random(rank))).astype(np.float16)
    mean = (rng.standard_normal(p) * 0.1).astype(np.float16)
    gc = {
        "k_coeffs": O.int4_pack(q),
        "k_coeff_scale": coeff_scale,
        "k_coeffs_shape": (n_comp, rank),
        "k_basis_q": basis_q,
        "k_basis_scale": basis_scale,
        "k_basis_f16": (basis_q.astype(np.float16) * basis_scale).astype(np.float16),
        "k_mean": mean, "k_mean_f16": mean,
        "v_indices_u8": rng.integers(0, 256, size=(nkv, n_comp, 32)).astype(np.uint8),
        "v_centroids_f16": (rng.standard_normal((256, 4)) * 0.4).astype(np.float16),
        "v_ch_f16": (0.5 + rng.random((nkv, hd)) * 3).astype(np.float16),
        "sink_k": rng.standard_normal((nkv, n_sink, hd)).astype(np.float16),
        "sink_v": rng.standard_normal((nkv, n_sink, hd)).astype(np.float16),
        "win_k": rng.standard_normal((nkv, n_win, hd)).astype(np.float16),
        "win_v": rng.standard_normal((nkv, n_win, hd)).astype(np.float16),
        "n_compress": n_comp, "batch": 1, "compress_start": compress_start,
    }
    return gc


def random_query(n_q=32, seed=1, scale=1.0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((n_q, 128)) * scale).astype(np.float16)
