"""`Cache`: the reference's drop-in Hugging Face KV cache, backed by sm_100a kernels.

Same constructor, flags, state machine and per-layer tensor dictionary as the
reference's src/shard/cache.py (prefill keeps raw K/V; the first decode step
compresses every layer; later steps append to an 8-bit stream or an fp16
buffer), but every array-sized computation runs in libshard_b200.so:

* K: RoPE removal -> (PyTorch) low-rank SVD -> host bit allocation -> int8 basis
  -> projection kernel -> two-stage int4 quantiser + nibble packing;
* V: Hadamard + per-channel normalisation kernel -> k-means whose assignment step
  is the `vq_assign` kernel;
* decode append: the Lloyd-Max stream quantizer kernel.

What stays in PyTorch is what the reference also leaves to PyTorch: the
randomised SVD, the centroid update (`index_add_`) and small host-side logic.
There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

import math

import torch
from transformers.cache_utils import Cache as HFCache, CacheLayerMixin

from . import ops
from ._lib import ShardError
from .rope import dp_bit_allocation, get_rope_inv_freq, reapply_rope
from .streaming import get_codebook, stream_signs

KERNEL_HEAD_DIM = 128
KERNEL_RANK_STEP = 32
KERNEL_MAX_RANK = 192


def pca_fit(flat, mean, rank):
    """Top-`rank` principal directions of the rows of `flat` (n, p) around `mean`: the
    eigenvectors of the p x p covariance, largest eigenvalue first, and those eigenvalues.

    Replaces the reference's randomised `torch.svd_lowrank(flat - mean, q=rank, niter=24)`
    (src/shard/cache.py:376: 48 passes over the n x p matrix) by one pass -- the Gram matrix
    (flat - mean)^T (flat - mean), a p x p x n contraction in fp32 -- and a symmetric
    eigensolver on the small p x p matrix.  The subspace is the exact optimum the randomised
    method approximates, so it captures at least as much variance; individual vectors differ
    in sign and, within near-equal eigenvalues, by rotations, which the rest of the path is
    indifferent to (the basis is an input of everything downstream).
    """
    n, p = flat.shape
    xc = flat - mean
    # full-precision fp32 products whatever the global TF32 switch says: the trailing
    # eigenvalues are 1e-4 of the leading ones and decide the bit allocation
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        gram = xc.T @ xc
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    evals, evecs = torch.linalg.eigh(gram)
    order = torch.arange(p - 1, p - 1 - rank, -1, device=flat.device)
    basis = evecs[:, order].contiguous()
    eigvals = (evals[order].clamp(min=0) / n).float()
    return basis, eigvals


def hadamard(x):
    """Normalised Walsh-Hadamard transform on the last dim (self-inverse).

    Torch expression used only by the non-fused read path and by tests; the hot
    paths run the butterfly inside the kernels.
    """
    d = x.shape[-1]
    h = 1
    while h < d:
        y = x.unflatten(-1, (-1, 2 * h))
        lo, hi = y[..., :h], y[..., h:]
        x = torch.cat([lo + hi, lo - hi], dim=-1).flatten(-2)
        h *= 2
    return x / math.sqrt(d)


def kmeans(data, k, n_iter=30, seed=42, init=None):
    """Lloyd's algorithm as the reference runs it (src/shard/cache.py:21-39).

    Assignment and the per-centroid sums / counts come from one CUDA pass
    (`vq_assign_accumulate`); the division and the stopping rule stay in PyTorch.  Returns the updated centroids and the assignment made against the
    previous ones.  `init` overrides the seeded random initial centroids.
    """
    n = data.shape[0]
    dev = data.device
    if init is None:
        g = torch.Generator(device=dev).manual_seed(seed)
        centroids = data[torch.randperm(n, generator=g, device=dev)[:k]].clone()
    else:
        centroids = init.to(dev, data.dtype).clone()
    idx_u8 = None
    sums = torch.zeros_like(centroids)
    counts = torch.zeros(k, device=dev, dtype=data.dtype)
    for it in range(n_iter):
        # assignment and the sums / counts of the centroid update in one pass over the points
        idx_u8 = ops.vq_assign_accumulate(data, centroids, sums, counts)
        filled = counts > 0
        new = centroids.clone()
        new[filled] = sums[filled] / counts[filled].unsqueeze(1)
        moved = (new - centroids).abs().max().item()
        centroids = new
        if moved < 1e-4 and it >= 5:
            break
    return centroids, idx_u8


class CacheLayer(CacheLayerMixin):
    """One layer's K/V: raw after prefill, compressed (`_gpu_compressed`) afterwards."""

    def __init__(self, layer_idx):
        self.layer_idx = layer_idx
        self._keys = None
        self._values = None
        self._prefilled = False
        self._seq_len = 0
        self._cache_ref = None
        self._needs_decompress = False
        self._gpu_compressed = None
        self.is_initialized = False

    # -- lazy materialisation (non-fused reads) -------------------------------
    def _lazy_evict(self):
        c = self._cache_ref
        if c is None or not c._lazy_per_layer:
            return
        last = c._last_accessed_layer
        if last != -1 and last != self.layer_idx:
            prev = c.layers[last]
            if prev._gpu_compressed is not None:
                prev._keys = None
                prev._values = None
                prev._needs_decompress = True
        c._last_accessed_layer = self.layer_idx

    def _ensure_dequant(self):
        """Full fp16 K/V as [sink | middle | window | stream | fp16 decode buffer]
        (reference: src/shard/cache.py:87-124).  Off the hot path: used on the
        first decode step of layer 0, by non-Llama models and by multi-token
        continuation."""
        if not self._needs_decompress:
            return
        gc = self._gpu_compressed
        if gc is None:
            return
        c = self._cache_ref
        n_total, rank = gc["k_coeffs_shape"]
        packed = gc["k_coeffs"]
        lo = (packed & 0x0F).to(torch.float16) - 8.0
        hi = ((packed >> 4) & 0x0F).to(torch.float16) - 8.0
        coeffs = torch.stack([lo, hi], dim=1).flatten()[: n_total * rank].reshape(n_total, rank)
        coeffs = coeffs * gc["k_coeff_scale"].half()
        basis = gc["k_basis_q"].to(torch.float16) * gc["k_basis_scale"].half()
        recon = coeffs @ basis.T + gc["k_mean"].half()
        B, n_comp = gc["batch"], gc["n_compress"]
        nkv, hd = c._n_kv_heads, c.head_dim
        k_layer = recon.view(B, n_comp, nkv, hd).permute(0, 2, 1, 3)
        if c._rope_inv_freq is not None:
            pos = torch.arange(gc["compress_start"], gc["compress_start"] + n_comp, device=packed.device)
            k_mid = reapply_rope(k_layer, pos, c._rope_inv_freq).half()
        else:
            k_mid = k_layer.half()
        cb = gc["v_centroids_f16"].float()
        v_rot = cb[gc["v_indices_u8"].long()].reshape(nkv, n_comp, hd) * gc["v_ch_f16"].float().unsqueeze(1)
        v_mid = hadamard(v_rot).view(B, nkv, n_comp, hd).half()
        parts_k = [gc["sink_k"], k_mid, gc["win_k"]]
        parts_v = [gc["sink_v"], v_mid, gc["win_v"]]
        sk, sv = self._dequant_stream(gc)
        if sk is not None:
            parts_k.append(sk)
            parts_v.append(sv)
        if "decode_k" in gc:
            parts_k.append(gc["decode_k"])
            parts_v.append(gc["decode_v"])
        self._keys = torch.cat(parts_k, dim=2)
        self._values = torch.cat(parts_v, dim=2)
        self._needs_decompress = False

    @property
    def keys(self):
        self._lazy_evict()
        self._ensure_dequant()
        return self._keys

    @keys.setter
    def keys(self, v):
        self._keys = v

    @property
    def values(self):
        self._lazy_evict()
        self._ensure_dequant()
        return self._values

    @values.setter
    def values(self, v):
        self._values = v

    # -- HF entry point --------------------------------------------------------
    def update(self, key_states, value_states, *args, **kwargs):
        """Prefill stores raw K/V; the first decode step compresses; later steps append
        (reference: src/shard/cache.py:138-191)."""
        seq_new = key_states.shape[2]
        c = self._cache_ref
        if seq_new > 1 and not self._prefilled:
            self._prefilled = True
            self.is_initialized = True
            self._seq_len = seq_new
            self._keys = key_states
            self._values = value_states
            return key_states, value_states

        if self.layer_idx == 0 and c is not None and not c._compressed:
            c.compress()

        gc = self._gpu_compressed
        fused = bool(getattr(c, "_fused_decode_update", False))
        if fused and gc is not None and seq_new == 1 and c._streaming:
            # the decode hot path: the token is handed to the next decode launch, which quantises it
            # into its stream row; nothing is launched here
            if "_pending" in gc:
                self._flush_pending()
            s = gc.get("stream_n", 0)
            if "signs" not in gc or s >= gc["k_idx_buf"].shape[0]:
                self._grow_stream(gc, key_states, s + 1)
            k2, v2 = key_states, value_states
            if k2.stride(3) != 1 or k2.stride(1) != k2.shape[3] or v2.stride(3) != 1 or v2.stride(1) != v2.shape[3]:
                k2, v2 = k2.contiguous(), v2.contiguous()
            gc["_pending"] = (k2, v2, s)
            gc["stream_n"] = s + 1
            self._seq_len += 1
            self._needs_decompress = True
            c._last_accessed_layer = self.layer_idx
            return key_states, value_states

        self._lazy_evict()
        if gc is not None and c._streaming:
            for t in range(seq_new):
                # with the fused decode the last token is quantised inside the decode launch
                self._stream_append(key_states[:, :, t:t + 1, :], value_states[:, :, t:t + 1, :],
                                    self._seq_len + t, defer=fused and t == seq_new - 1)
            self._seq_len += seq_new
            self._needs_decompress = True
            if fused:
                return key_states, value_states
            self._ensure_dequant()
            return self._keys, self._values

        if gc is not None:
            # tokens a non-streaming cache keeps as they are: appended in place to a buffer allocated
            # ahead (doubling when full); gc["decode_k"] / ["decode_v"] are views of the rows in use
            n = gc["decode_k"].shape[2] if "decode_k" in gc else 0
            buf_k = gc.get("_dec_buf_k")
            if buf_k is None or n + seq_new > buf_k.shape[2] or buf_k.dtype != key_states.dtype:
                cap = max(c._decode_capacity, 2 * (n + seq_new))
                B, nkv, _, hd = key_states.shape
                new_k = torch.empty(B, nkv, cap, hd, dtype=key_states.dtype, device=key_states.device)
                new_v = torch.empty(B, nkv, cap, hd, dtype=value_states.dtype, device=value_states.device)
                if n:
                    new_k[:, :, :n].copy_(gc["decode_k"])
                    new_v[:, :, :n].copy_(gc["decode_v"])
                buf_k, gc["_dec_buf_k"], gc["_dec_buf_v"] = new_k, new_k, new_v
            buf_v = gc["_dec_buf_v"]
            buf_k[:, :, n:n + seq_new].copy_(key_states)
            buf_v[:, :, n:n + seq_new].copy_(value_states)
            gc["decode_k"] = buf_k[:, :, :n + seq_new]
            gc["decode_v"] = buf_v[:, :, :n + seq_new]
            self._seq_len += seq_new
            self._needs_decompress = True
            if fused:
                return key_states, value_states
            self._ensure_dequant()
            return self._keys, self._values

        self._ensure_dequant()
        self._seq_len += seq_new
        if self._keys is not None:
            self._keys = torch.cat([self._keys, key_states], dim=2)
            self._values = torch.cat([self._values, value_states], dim=2)
        else:
            self._keys = key_states
            self._values = value_states
        return self._keys, self._values

    # -- 8-bit stream -----------------------------------------------------------
    def _flush_pending(self):
        """Quantise a token whose append was left to the next decode launch and never got one."""
        gc = self._gpu_compressed
        pend = gc.pop("_pending", None) if gc is not None else None
        if pend is not None:
            k2, v2, slot = pend
            k2 = k2.reshape(-1, k2.shape[-1]).contiguous()       # (nkv, hd)
            v2 = v2.reshape(-1, v2.shape[-1]).contiguous()
            ops.stream_quantize(k2, v2, gc["signs"], get_codebook(k2.shape[-1], 8, k2.device),
                                gc["k_idx_buf"], gc["v_idx_buf"], gc["k_norm_buf"], gc["v_norm_buf"], slot)

    def _grow_stream(self, gc, k, need):
        """(Re)allocate the stream buffers for at least `need` rows: the cache's decode capacity at
        first, doubling afterwards (reference: src/shard/cache.py:220-230, which starts at 16 rows)."""
        c = self._cache_ref
        if c._stream_qjl:
            raise NotImplementedError("the QJL residual is not part of the CUDA stream path")
        if c._stream_bits != 8:
            raise NotImplementedError("the CUDA stream quantizer emits 8-bit codes only")
        B, heads, _, hd = k.shape
        if B != 1:
            raise NotImplementedError("one sequence per Cache (use one Cache per sequence)")
        if k.dtype != torch.float16:
            raise NotImplementedError("fp16 models only")
        dev = k.device
        if "signs" not in gc:
            gc["signs"] = stream_signs(self.layer_idx, hd, dev)
        cap = gc["k_idx_buf"].shape[0] if "k_idx_buf" in gc else 0
        if need <= cap:
            return
        new_cap = max(need, c._decode_capacity if cap == 0 else cap * 2)
        for key, shape, dtype in (("k_idx", (B, heads, hd), torch.uint8),
                                  ("v_idx", (B, heads, hd), torch.uint8),
                                  ("k_norm", (B, heads), torch.float16),
                                  ("v_norm", (B, heads), torch.float16)):
            new = torch.zeros((new_cap, *shape), device=dev, dtype=dtype)
            old = gc.get(f"{key}_buf")
            if old is not None:
                new[: old.shape[0]].copy_(old)
            gc[f"{key}_buf"] = new

    def _stream_append(self, k, v, position, defer=False):
        """Quantise one (1, nkv, 1, hd) token into the stream buffers
        (reference: src/shard/cache.py:193-241).  With `defer` the row is reserved and the
        token is handed to the next `decode_layer` call, whose kernel quantises it."""
        self._flush_pending()
        gc = self._gpu_compressed
        c = self._cache_ref
        if c._stream_qjl:
            raise NotImplementedError("the QJL residual is not part of the CUDA stream path")
        if c._stream_bits != 8:
            raise NotImplementedError("the CUDA stream quantizer emits 8-bit codes only")
        B, heads, _, hd = k.shape
        if B != 1:
            raise NotImplementedError("one sequence per Cache (use one Cache per sequence)")
        dev = k.device
        s = gc.get("stream_n", 0)
        if "signs" not in gc or s >= gc["k_idx_buf"].shape[0]:
            self._grow_stream(gc, k, s + 1)
        k2 = k.reshape(heads, hd)
        v2 = v.reshape(heads, hd)
        if k2.dtype != torch.float16:
            raise NotImplementedError("fp16 models only")
        if defer:
            gc["_pending"] = (k2.contiguous(), v2.contiguous(), s)
        else:
            ops.stream_quantize(k2.contiguous(), v2.contiguous(), gc["signs"], get_codebook(hd, 8, dev),
                                gc["k_idx_buf"], gc["v_idx_buf"], gc["k_norm_buf"], gc["v_norm_buf"], s)
        gc["stream_n"] = s + 1

    def _dequant_stream(self, gc=None, *unused):
        """fp16 (1, nkv, s, hd) K and V of the streamed tokens (reference: cache.py:243-279)."""
        if gc is None or gc is self._gpu_compressed:
            self._flush_pending()
        gc = self._gpu_compressed if gc is None else gc
        s = gc.get("stream_n", 0)
        if s == 0 or "k_idx_buf" not in gc:
            return None, None
        dev = gc["k_idx_buf"].device
        cb = get_codebook(self._cache_ref.head_dim, 8, dev)
        sk = ops.stream_dequant(gc["k_idx_buf"][:s], gc["k_norm_buf"][:s], gc["signs"], cb)
        sv = ops.stream_dequant(gc["v_idx_buf"][:s], gc["v_norm_buf"][:s], gc["signs"], cb)
        return sk.unsqueeze(0), sv.unsqueeze(0)

    # -- HF glue -----------------------------------------------------------------
    def get_seq_length(self, *args, **kwargs):
        return self._seq_len

    def get_max_cache_shape(self):
        return None

    def get_mask_sizes(self, query_length, *args, **kwargs):
        if not isinstance(query_length, int):
            query_length = int(query_length.shape[0])
        return self._seq_len + query_length, 0

    def lazy_initialization(self, *args, **kwargs):
        pass

    def reorder_cache(self, beam_idx):
        if self._needs_decompress:
            _ = self.keys
        if self._keys is not None:
            self._keys = self._keys.index_select(0, beam_idx.to(self._keys.device))
        if self._values is not None:
            self._values = self._values.index_select(0, beam_idx.to(self._values.device))


class Cache(HFCache):
    """Compressed KV cache with the reference's constructor and flags
    (src/shard/cache.py:295-336)."""

    def __init__(self, head_dim=128, num_layers=32, n_kv_heads=8, device="cuda",
                 k_target_cr=20.0, max_rank_k=192,
                 v_vq_group_size=4, v_vq_codebook_size=256,
                 sink_tokens=4, residual_window=64, rope_inv_freq=None, decode_capacity=256):
        self.head_dim = head_dim
        # rows the per-layer buffers of decoded tokens (8-bit stream, fp16 decode buffer) are
        # allocated for when the cache is compressed; they double when they run full
        self._decode_capacity = max(16, int(decode_capacity))
        self._num_layers = num_layers
        self._n_kv_heads = n_kv_heads
        self._per_layer_dim = n_kv_heads * head_dim
        self._k_target_cr = k_target_cr
        self._max_rank_k = max_rank_k
        self._v_vq_group_size = v_vq_group_size
        self._v_vq_codebook_size = v_vq_codebook_size
        self._sink_tokens = sink_tokens
        self._residual_window = residual_window
        self._rope_inv_freq = rope_inv_freq
        self._streaming = False
        self._stream_bits = 8
        self._stream_qjl = False
        self._lazy_per_layer = True
        self._full_fused = False
        # how the PCA basis of the keys is fitted: "eigh" (covariance + symmetric eigensolver on the
        # GPU) or "svd_lowrank" (the reference's randomised call)
        self._k_pca = "eigh"
        self._last_accessed_layer = -1
        self._compressed = False
        self._device = device
        self._decode_ws = None
        self._phase = None
        self._phase_key = None
        self._inv_freq_dev = None
        self.compress_seconds = None
        super().__init__(layers=[CacheLayer(i) for i in range(num_layers)])
        for layer in self.layers:
            layer._cache_ref = self

    @classmethod
    def from_model(cls, model, k_target_cr=16.0, **kwargs):
        cfg = model.config
        hd = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        return cls(head_dim=hd, num_layers=cfg.num_hidden_layers,
                   n_kv_heads=getattr(cfg, "num_key_value_heads", cfg.num_attention_heads),
                   device=str(next(model.parameters()).device),
                   k_target_cr=k_target_cr,
                   rope_inv_freq=get_rope_inv_freq(model), **kwargs)

    # -- compression ------------------------------------------------------------
    def _check_supported(self, k0):
        if not k0.is_cuda:
            raise ShardError("shard_b200.Cache compresses on a CUDA device; there is no CPU fallback")
        if self.head_dim != KERNEL_HEAD_DIM:
            raise NotImplementedError("kernels are built for head_dim 128")
        if self._v_vq_group_size != 4 or self._v_vq_codebook_size != 256:
            raise NotImplementedError("kernels are built for 256-entry codebooks of 4-channel sub-vectors")
        if k0.dtype != torch.float16:
            raise NotImplementedError("fp16 models only")
        if k0.shape[0] != 1:
            raise NotImplementedError("one sequence per Cache; batch by holding one Cache per sequence")
        if self._rope_inv_freq is None:
            raise NotImplementedError("rope_inv_freq is required by the compressed-score identity")

    def compress(self):
        """Compress every layer's prefill K/V (reference: src/shard/cache.py:338-366)."""
        if self._compressed:
            return
        k0 = self.layers[0]._keys
        if k0 is None:
            return
        B, _, seq, _ = k0.shape
        sink, win = self._sink_tokens, self._residual_window
        if seq <= sink + win + 4:
            return
        self._check_supported(k0)
        start, end = sink, seq - win
        ev0 = torch.cuda.Event(enable_timing=True)
        ev1 = torch.cuda.Event(enable_timing=True)
        ev0.record()
        for li in range(self._num_layers):
            torch.manual_seed(42 + li)
            layer = self.layers[li]
            k_full, v_full = layer._keys, layer._values
            kpart = self._compress_k(k_full[0, :, start:end, :], start)
            vpart = self._compress_v(v_full[0, :, start:end, :])
            self._build_gpu_format(layer, kpart, vpart,
                                   sink_k=k_full[:, :, :sink, :].clone(), sink_v=v_full[:, :, :sink, :].clone(),
                                   win_k=k_full[:, :, end:, :].clone(), win_v=v_full[:, :, end:, :].clone(),
                                   n_comp=end - start, batch=B, start=start)
        ev1.record()
        ev1.synchronize()
        self.compress_seconds = ev0.elapsed_time(ev1) / 1e3
        self._compressed = True

    def _compress_k(self, k_mid, pos_start, basis=None):
        """Un-rotate, fit a joint PCA over all KV heads, quantise basis to int8 and
        coefficients to int4 (reference: src/shard/cache.py:368-396, 416-420).

        k_mid: (nkv, n, hd) fp16 view.  `basis` (dim, rank) overrides the SVD (used by
        the parity tests, which take the basis as given).
        """
        dev = k_mid.device
        inv_freq = self._inv_freq(dev)
        flat = ops.undo_rope(k_mid, pos_start, inv_freq)
        n, p = flat.shape
        mean = flat.mean(dim=0)
        rank = min(self._max_rank_k, p, n - 1)
        if basis is None and self._k_pca == "svd_lowrank":
            # the reference's own call (src/shard/cache.py:376): randomised, 24 power iterations
            _, S, V = torch.svd_lowrank(flat - mean, q=rank, niter=24)
            basis = V[:, :rank]
            eigvals = (S[:rank].float() ** 2) / n
        elif basis is None:
            basis, eigvals = pca_fit(flat, mean, rank)
        else:
            basis = basis.to(dev, torch.float32)[:, :rank]
            eigvals = ((flat - mean) @ basis).pow(2).sum(dim=0) / n
        budget = max(64, int(self._per_layer_dim * 16 / self._k_target_cr))
        alloc = dp_bit_allocation(eigvals, budget)
        keep = sum(1 for b in alloc if b > 0)
        keep -= keep & 1
        if keep <= 0:
            raise ShardError("bit allocation kept no PCA component")
        basis = basis[:, :keep].contiguous()
        alloc = alloc[:keep]
        col_max = basis.abs().max(dim=0).values.clamp(min=1e-6)
        scale = col_max / 127.0
        basis_q = (basis / scale).round().clamp(-127, 127).to(torch.int8)
        w = (basis_q.float() * scale.float()).contiguous()
        proj = ops.k_project(flat, mean.float().contiguous(), w)
        packed, coeff_scale = ops.k_quantize_pack(proj, alloc)
        return {"k_basis_q": basis_q, "k_scale": scale.half(), "k_mean": mean.half(), "k_alloc": alloc,
                "k_coeffs": packed, "k_coeff_scale": coeff_scale, "k_n_total": n}

    def _compress_v(self, v_mid, init_centroids=None):
        """Hadamard-rotate, normalise per channel and vector-quantise 4-channel groups
        (reference: src/shard/cache.py:398-404, 41-52).  v_mid: (nkv, n, hd) fp16 view."""
        x, ch_max = ops.v_hadamard_normalise(v_mid)
        flat = x.view(-1, self._v_vq_group_size)
        centroids, idx_u8 = kmeans(flat, self._v_vq_codebook_size, n_iter=30, init=init_centroids)
        nkv, n, hd = v_mid.shape
        return {"centroids": centroids.half(), "packed": idx_u8, "ch_maxabs": ch_max.half(),
                "shape": (nkv, n, hd), "group_size": self._v_vq_group_size, "bits": 8,
                "n_orig": idx_u8.numel()}

    def _build_gpu_format(self, layer, k, v, sink_k, sink_v, win_k, win_v, n_comp, batch, start):
        """Assemble the per-layer tensor dictionary (reference: src/shard/cache.py:406-460)
        and the kernel-side prepared weights."""
        nkv, hd = self._n_kv_heads, self.head_dim
        keep = len(k["k_alloc"])
        ng = hd // v["group_size"]
        basis_f16 = (k["k_basis_q"].to(torch.float16) * k["k_scale"].to(torch.float16)).contiguous()
        coeff_scale_f16 = k["k_coeff_scale"].half()
        gc = {
            "k_coeffs": k["k_coeffs"],
            "k_coeff_scale": coeff_scale_f16,
            "k_coeffs_shape": (k["k_n_total"], keep),
            "k_basis_q": k["k_basis_q"],
            "k_basis_scale": k["k_scale"],
            "k_basis_f16": basis_f16,
            "k_mean": k["k_mean"],
            "k_mean_f16": k["k_mean"].to(torch.float16).contiguous(),
            "k_alloc": k["k_alloc"],
            "v_qdata": v,
            "v_packed": v["packed"],
            "v_indices_u8": v["packed"].view(nkv, n_comp, ng),
            "v_centroids_f16": v["centroids"].contiguous(),
            "v_ch_f16": v["ch_maxabs"].view(nkv, hd).contiguous(),
            "sink_k": sink_k, "sink_v": sink_v, "win_k": win_k, "win_v": win_v,
            "n_compress": n_comp, "batch": batch, "compress_start": start,
        }
        attach_kernel_format(gc, nkv)
        layer._gpu_compressed = gc
        layer._keys = None
        layer._values = None
        layer._needs_decompress = True

    def check(self):
        """Raise `ShardError` if a decode launch on this cache gave up on one of its bounded
        in-kernel waits since the last check (its output is then undefined).  Waits for the
        current stream; call it once per step or per request, not per layer."""
        if self._decode_ws is not None:
            ops.decode_status_check(self._decode_ws)

    def _inv_freq(self, dev):
        if self._inv_freq_dev is None or self._inv_freq_dev.device != torch.device(dev):
            self._inv_freq_dev = self._rope_inv_freq.to(dev, torch.float32).contiguous()
        return self._inv_freq_dev

    # -- accounting (reference: src/shard/cache.py:462-539) -------------------------
    @staticmethod
    def _nb(t):
        return t.nelement() * t.element_size()

    _STORAGE_KEYS = ("k_coeffs", "k_coeff_scale", "k_basis_q", "k_basis_scale", "k_mean", "v_packed",
                     "sink_k", "sink_v", "win_k", "win_v")

    def clean_memory_bytes(self):
        """Storage-only size of the compressed cache (no decode-time scratch)."""
        total, has = 0, False
        for layer in self.layers:
            gc = layer._gpu_compressed
            if gc is None:
                continue
            has = True
            total += sum(self._nb(gc[k]) for k in self._STORAGE_KEYS)
            total += self._nb(gc["v_qdata"]["ch_maxabs"]) + self._nb(gc["v_qdata"]["centroids"])
        if has:
            return total
        return sum(self._nb(l._keys) + self._nb(l._values) for l in self.layers if l._keys is not None)

    def memory_bytes(self):
        """Everything resident for the cache: storage, the decode-time copies this
        implementation keeps (fp16 basis, fragment-ordered weights) and the stream."""
        total, has = 0, False
        for layer in self.layers:
            gc = layer._gpu_compressed
            if gc is None:
                continue
            has = True
            total += sum(self._nb(gc[k]) for k in self._STORAGE_KEYS)
            total += self._nb(gc["v_qdata"]["ch_maxabs"]) + self._nb(gc["v_qdata"]["centroids"])
            for k in ("k_basis_f16", "k_mean_f16", "v_centroids_f16", "v_ch_f16", "k_wprep"):
                if k in gc:
                    total += self._nb(gc[k])
            if "k_coeffs_padded" in gc:
                total += self._nb(gc["k_coeffs_padded"])
            if "k_idx_buf" in gc:
                s = gc.get("stream_n", 0)
                bpv = self._stream_bits / 8.0
                for k in ("k_idx_buf", "v_idx_buf"):
                    total += int(gc[k][:s].nelement() * bpv)
                for k in ("k_norm_buf", "v_norm_buf"):
                    total += self._nb(gc[k][:s])
            if "decode_k" in gc:
                total += self._nb(gc["decode_k"]) + self._nb(gc["decode_v"])
        if has:
            return total
        return sum(self._nb(l._keys) + self._nb(l._values) for l in self.layers if l._keys is not None)

    def fp16_equivalent_bytes(self):
        gc = self.layers[0]._gpu_compressed
        if gc is not None:
            seq = gc["n_compress"] + self._sink_tokens + self._residual_window + gc.get("stream_n", 0)
        elif self.layers[0]._keys is not None:
            seq = self.layers[0]._keys.shape[2]
        else:
            return 0
        return seq * self._n_kv_heads * self.head_dim * 4 * self._num_layers

    def compress_ratio(self):
        return self.fp16_equivalent_bytes() / max(self.memory_bytes(), 1)

    def clean_compress_ratio(self):
        gc = self.layers[0]._gpu_compressed
        if gc is not None:
            seq = gc["n_compress"] + self._sink_tokens + self._residual_window
            fp16_bytes = seq * self._n_kv_heads * self.head_dim * 4 * self._num_layers
            return fp16_bytes / max(self.clean_memory_bytes(), 1)
        return self.compress_ratio()


def attach_kernel_format(gc, nkv):
    """Add what the decode kernel needs beyond the reference's dictionary: the
    fragment-ordered weights, and (only when the kept rank is not a multiple of 32) a
    copy of the coefficients padded with zero nibbles to the next multiple."""
    n_total, keep = gc["k_coeffs_shape"]
    basis = gc["k_basis_f16"]
    cscale = gc["k_coeff_scale"].to(torch.float16).contiguous()
    rank_k = ((keep + KERNEL_RANK_STEP - 1) // KERNEL_RANK_STEP) * KERNEL_RANK_STEP
    if rank_k > KERNEL_MAX_RANK:
        raise NotImplementedError("kernels support PCA ranks up to 192")
    coeffs = gc["k_coeffs"]
    if rank_k != keep:
        pad = rank_k - keep
        basis = torch.cat([basis, basis.new_zeros(basis.shape[0], pad)], dim=1).contiguous()
        cscale = torch.cat([cscale, cscale.new_zeros(pad)]).contiguous()
        rows = coeffs.view(n_total, keep // 2)
        coeffs = torch.cat([rows, rows.new_full((n_total, pad // 2), 0x88)], dim=1).contiguous().view(-1)
        gc["k_coeffs_padded"] = coeffs
    gc["k_rank_kernel"] = rank_k
    gc["k_coeffs_kernel"] = coeffs
    gc["k_wprep"] = ops.decode_prepare(basis, cscale, gc["k_mean_f16"], nkv, rank_k)
    gc["_fresh"] = True      # the next decode launch follows the kernels that wrote these tensors
    return gc
