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
