"""Seeded synthetic K/V/query generator used by the tests and the benchmark.

The reference evaluates on real text with Llama-3.1-8B weights; neither is
available offline, so every measurement here runs on synthetic tensors with
the same shapes and value distributions: keys that are rank-192 (plus a little
noise) before RoPE, values with a few outlier channels per head.
"""
from __future__ import annotations

import math

import torch

N_KV = 8
N_Q = 32
HEAD_DIM = 128
ROPE_THETA = 500000.0


def rope_inv_freq(hd: int = HEAD_DIM, theta: float = ROPE_THETA) -> torch.Tensor:
    """inv_freq[i] = theta ** (-2i / hd), fp32, as HF Llama derives it."""
    return 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def make_kvq(T: int, seed: int, device="cpu", nkv: int = N_KV, n_q: int = N_Q,
             hd: int = HEAD_DIM, rank: int = 192, theta: float = ROPE_THETA):
    """Draw one layer of prefill K, V (1, nkv, T, hd) and a query (1, n_q, 1, hd), fp16.

    Draw order (fp32, generator seeded ``seed`` on ``device``): Z ~ N(0,1)
    [T, rank]; W ~ N(0,1) [rank, nkv*hd] / sqrt(rank); E ~ N(0,1) [T, nkv*hd];
    K_noRoPE = Z W + 0.01 E, then RoPE (rotate_half convention) at positions
    0..T-1; V ~ N(0,1) with 4 random channels per head scaled by 20;
    q ~ N(0,1), to be used at position T.
    """
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    p = nkv * hd
    Z = torch.randn(T, rank, generator=g, device=dev)
    W = torch.randn(rank, p, generator=g, device=dev) / math.sqrt(rank)
    E = torch.randn(T, p, generator=g, device=dev)
    k_n = (Z @ W + 0.01 * E).view(1, T, nkv, hd).permute(0, 2, 1, 3)
    inv_freq = rope_inv_freq(hd, theta).to(dev)
    ph = torch.arange(T, device=dev, dtype=torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat([ph, ph], dim=-1)
    k = k_n * emb.cos() + _rotate_half(k_n) * emb.sin()
    v = torch.randn(1, nkv, T, hd, generator=g, device=dev)
    for h in range(nkv):
        ch = torch.randperm(hd, generator=g, device=dev)[:4]
        v[:, h, :, ch] *= 20.0
    q = torch.randn(1, n_q, 1, hd, generator=g, device=dev)
    return k.half().contiguous(), v.half().contiguous(), q.half().contiguous()


def make_token(seed: int, device="cpu", nkv: int = N_KV, n_q: int = N_Q, hd: int = HEAD_DIM):
    """One decode-step worth of fresh (k, v) (1, nkv, 1, hd) and q (1, n_q, 1, hd), fp16."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    k = torch.randn(1, nkv, 1, hd, generator=g, device=dev)
    v = torch.randn(1, nkv, 1, hd, generator=g, device=dev)
    q = torch.randn(1, n_q, 1, hd, generator=g, device=dev)
    return k.half(), v.half(), q.half()


def random_compressed_layer(n_comp, device, seed, compress_start=4, n_sink=4, n_win=64, rank=192, nkv=N_KV,
                            hd=HEAD_DIM, gen_device=None):
    """A compressed layer with random codes, built directly on `device` (no prefill, no
    compression).  Decode cost does not depend on code values, so the multi-GPU
    benchmark workloads use this to set up many / very long caches quickly.  Returns the
    per-layer tensor dictionary in the product's format (kernel-side weights attached).
    With `gen_device="cpu"` the values are drawn by the CPU generator and then moved, which
    makes them identical on every rank whatever GPU it runs on."""
    from shard_b200.cache import attach_kernel_format
    dev = torch.device(device)
    gdev = dev if gen_device is None else torch.device(gen_device)
    g = torch.Generator(device=gdev).manual_seed(seed)
    p = nkv * hd
    basis_q = torch.randint(-127, 128, (p, rank), generator=g, device=gdev, dtype=torch.int8)
    basis_scale = (0.08 / 127 * (0.5 + torch.rand(rank, generator=g, device=gdev))).half()
    decay = torch.exp(-0.01 * torch.arange(rank, device=gdev, dtype=torch.float32))
    gc = {
        "k_coeffs": torch.randint(0, 256, (n_comp * rank // 2,), generator=g, device=gdev, dtype=torch.uint8),
        "k_coeff_scale": (decay * 0.4).half(),
        "k_coeffs_shape": (n_comp, rank),
        "k_basis_q": basis_q,
        "k_basis_scale": basis_scale,
        "k_basis_f16": (basis_q.half() * basis_scale).contiguous(),
        "k_mean": (torch.randn(p, generator=g, device=gdev) * 0.1).half(),
        "v_indices_u8": torch.randint(0, 256, (nkv, n_comp, hd // 4), generator=g, device=gdev, dtype=torch.uint8),
        "v_centroids_f16": (torch.randn(256, 4, generator=g, device=gdev) * 0.4).half(),
        "v_ch_f16": (0.5 + 3 * torch.rand(nkv, hd, generator=g, device=gdev)).half(),
        "sink_k": torch.randn(1, nkv, n_sink, hd, generator=g, device=gdev).half(),
        "sink_v": torch.randn(1, nkv, n_sink, hd, generator=g, device=gdev).half(),
        "win_k": torch.randn(1, nkv, n_win, hd, generator=g, device=gdev).half(),
        "win_v": torch.randn(1, nkv, n_win, hd, generator=g, device=gdev).half(),
        "n_compress": n_comp, "batch": 1, "compress_start": compress_start,
    }
    if gdev != dev:
        gc = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in gc.items()}
    gc["k_mean_f16"] = gc["k_mean"]
    gc["v_packed"] = gc["v_indices_u8"].view(-1)
    attach_kernel_format(gc, nkv)
    return gc


def random_cache(n_comp, layers, device, seed0, **kw):
    """A `Cache` whose layers are `random_compressed_layer`s (already 'compressed')."""
    from shard_b200.cache import Cache
    cache = Cache(num_layers=layers, rope_inv_freq=rope_inv_freq(), device=str(device))
    cache._streaming = True
    cache._compressed = True
    for li in range(layers):
        layer = cache.layers[li]
        layer._gpu_compressed = random_compressed_layer(n_comp, device, seed0 + li, **kw)
        layer._prefilled = True
        layer._needs_decompress = True
        layer._seq_len = kw.get("compress_start", 4) + n_comp + kw.get("n_win", 64)
    return cache
