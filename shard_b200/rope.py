"""RoPE helpers and the host-side bit allocation of the K compressor.

Mirrors the parts of the reference's src/shard/rope.py that the compressed-KV
path uses.  The heavy lifting (RoPE removal over a whole prefill, the int4
quantiser) lives in CUDA; what is here is host control logic and the small
torch expressions of the non-fused read path.
"""
from __future__ import annotations

import torch


def rotate_half(x):
    """HF Llama convention: (x1, x2) -> (-x2, x1) on the two halves of the last dim."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def rope_cos_sin(positions, inv_freq):
    """cos/sin tables (T, hd) of fp32(pos) * fp32(inv_freq) duplicated over both halves."""
    ph = positions.to(torch.float32)[:, None] * inv_freq.to(positions.device, torch.float32)[None, :]
    emb = torch.cat([ph, ph], dim=-1)
    return emb.cos(), emb.sin()


def reapply_rope(keys, positions, inv_freq):
    """keys (..., T, hd) -> keys with RoPE at `positions` (reference: rope.py:26-30)."""
    cos, sin = rope_cos_sin(positions, inv_freq)
    return keys * cos + rotate_half(keys) * sin


def get_rope_inv_freq(model):
    """Find the model's rotary inv_freq table, else derive it from the config
    (reference: src/shard/rope.py:32-47)."""
    backbone = getattr(model, "model", getattr(model, "transformer", None))
    candidates = [backbone]
    layers = getattr(backbone, "layers", None) if backbone is not None else None
    if layers is not None and len(layers) > 0:
        candidates.append(layers[0])
    for owner in candidates:
        if owner is None:
            continue
        rot = getattr(owner, "rotary_emb", None)
        if rot is None:
            attn = getattr(owner, "self_attn", None)
            rot = getattr(attn, "rotary_emb", None) if attn is not None else None
        if rot is not None and hasattr(rot, "inv_freq"):
            return rot.inv_freq.detach().float().cpu()
    cfg = model.config
    hd = getattr(cfg, "head_dim", cfg.hidden_size // cfg.num_attention_heads)
    theta = getattr(cfg, "rope_theta", 10000.0)
    params = getattr(cfg, "rope_parameters", None)
    if isinstance(params, dict) and "rope_theta" in params:
        theta = params["rope_theta"]
    return 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))


_GROUP = 64                 # components share a bit width in groups of 64
_BIT_CHOICES = (0, 2, 4, 6, 8)
_DROP_PENALTY = 4.0         # a dropped group is charged 4x its variance
_COST_UNIT = 16             # budget is counted in units of 16 bits


def dp_bit_allocation(variances, total_budget):
    """Bits per PCA component by dynamic programming (reference: rope.py:49-84).

    Minimises sum_g err(g, bits_g) subject to sum_g ceil(size_g * bits_g / 16)
    <= total_budget // 16 + 1, with err = 4 * var for 0 bits and
    var / (3 * 4**bits) otherwise.  Ties keep the first (smallest) option.
    """
    v = variances.float().cpu()
    d = int(v.shape[0])
    n_groups = (d + _GROUP - 1) // _GROUP
    sizes = [min(_GROUP, d - g * _GROUP) for g in range(n_groups)]
    gvar = [v[g * _GROUP: g * _GROUP + sizes[g]].sum().item() for g in range(n_groups)]
    cap = total_budget // _COST_UNIT + 1
    inf = float("inf")
    best = [[inf] * (cap + 1) for _ in range(n_groups + 1)]
    pick = [[0] * (cap + 1) for _ in range(n_groups + 1)]
    best[0] = [0.0] * (cap + 1)

    def cost_of(g, bits):
        return 0 if bits == 0 else (sizes[g] * bits + _COST_UNIT - 1) // _COST_UNIT

    for g in range(n_groups):
        for b in range(cap + 1):
            for bits in _BIT_CHOICES:
                c = cost_of(g, bits)
                if c > b:
                    continue
                err = gvar[g] * _DROP_PENALTY if bits == 0 else gvar[g] / (3.0 * (1 << (2 * bits)))
                total = best[g][b - c] + err
                if total < best[g + 1][b]:
                    best[g + 1][b] = total
                    pick[g + 1][b] = bits
    b = min(range(cap + 1), key=lambda i: best[n_groups][i])
    alloc = [0] * d
    for g in range(n_groups - 1, -1, -1):
        bits = pick[g + 1][b]
        alloc[g * _GROUP: g * _GROUP + sizes[g]] = [bits] * sizes[g]
        b -= cost_of(g, bits)
    return alloc
