"""Tensor-level wrappers of the C-ABI entry points.

Each function validates dtype / contiguity / device on the Python side, passes
raw device pointers and the current CUDA stream to libshard_b200.so and
returns torch tensors.  The names follow the reference's kernel wrappers
(src/shard/triton_kernels.py) where a counterpart exists.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import ShardDecodeShape, ShardSeq, check, cur_stream, ptr, require_cuda

HD = 128


def _c(t, dtype=None):
    if dtype is not None and t.dtype != dtype:
        raise _lib.ShardError(f"expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise _lib.ShardError("tensor must be contiguous")
    return t


# --------------------------------------------------------------------------- stream quantizer
def stream_quantize(new_k, new_v, signs, codebook, k_idx_buf, v_idx_buf, k_norm_buf, v_norm_buf, slot):
    """Append one token (nkv, 128) fp16 K/V as 8-bit codes + fp16 norms at row `slot`."""
    require_cuda(new_k, new_v, signs, codebook, k_idx_buf)
    nkv = new_k.shape[-2]
    seq = ShardSeq()
    seq.new_k, seq.new_v = ptr(_c(new_k, torch.float16)), ptr(_c(new_v, torch.float16))
    seq.signs = ptr(_c(signs, torch.float32))
    seq.st_k_idx, seq.st_v_idx = ptr(_c(k_idx_buf, torch.uint8)), ptr(_c(v_idx_buf, torch.uint8))
    seq.st_k_norm, seq.st_v_norm = ptr(_c(k_norm_buf, torch.float16)), ptr(_c(v_norm_buf, torch.float16))
    if slot >= k_idx_buf.shape[0]:
        raise _lib.ShardError("stream buffer full")
    check(_lib.load().shard_b200_stream_quantize(C.addressof(seq), 1, nkv, slot,
                                                 ptr(_c(codebook, torch.float32)), cur_stream()),
          "stream_quantize")


def stream_dequant(idx, norm, signs, codebook):
    """(s, nkv, 128) u8 codes + (s, nkv) fp16 norms -> (nkv, s, 128) fp16."""
    require_cuda(idx, norm, signs, codebook)
    s, nkv = idx.shape[0], idx.shape[-2]
    out = torch.empty(nkv, s, HD, dtype=torch.float16, device=idx.device)
    check(_lib.load().shard_b200_stream_dequant(ptr(_c(idx, torch.uint8)), ptr(_c(norm, torch.float16)),
                                                ptr(_c(signs, torch.float32)), ptr(_c(codebook, torch.float32)),
                                                s, nkv, ptr(out), cur_stream()), "stream_dequant")
    return out


# --------------------------------------------------------------------------- prefill compressor
def undo_rope(k, pos_start, inv_freq):
    """k: (nkv, n, 128) fp16 view (last dim contiguous) -> (n, nkv*128) fp32 without RoPE."""
    require_cuda(k, inv_freq)
    if k.dtype != torch.float16 or k.stride(-1) != 1:
        raise _lib.ShardError("undo_rope expects fp16 keys with a contiguous head dimension")
    nkv, n, _ = k.shape
    flat = torch.empty(n, nkv * HD, dtype=torch.float32, device=k.device)
    check(_lib.load().shard_b200_undo_rope(ptr(k), k.stride(0), k.stride(1), nkv, n, int(pos_start),
                                           ptr(_c(inv_freq, torch.float32)), ptr(flat), cur_stream()),
          "undo_rope")
    return flat


def k_project(flat, mean, w):
    """(flat - mean) @ w with fp32 accuracy on the tensor cores; flat (n, dim), mean (dim,), w (dim, keep)."""
    require_cuda(flat, mean, w)
    n, dim = flat.shape
    keep = w.shape[1]
    lib = _lib.load()
    wsb = lib.shard_b200_k_project_workspace_bytes(dim, keep)
    if wsb == 0:
        raise _lib.ShardError(f"k_project supports dim % 32 == 0, dim <= 1024, even keep <= 192 (got {dim}, {keep})")
    ws = torch.empty(wsb, dtype=torch.uint8, device=flat.device)
    proj = torch.empty(n, keep, dtype=torch.float32, device=flat.device)
    check(lib.shard_b200_k_project(ptr(_c(flat, torch.float32)), ptr(_c(mean, torch.float32)),
                                   ptr(_c(w, torch.float32)), n, dim, keep, ptr(proj), ptr(ws), wsb, cur_stream()),
          "k_project")
    return proj


def k_quantize_pack(proj, alloc):
    """Two-stage quantisation of projected keys to packed int4; returns (packed u8, coeff_scale fp32)."""
    require_cuda(proj)
    n, keep = proj.shape
    lib = _lib.load()
    alloc_t = torch.as_tensor(list(alloc), dtype=torch.int32).to(proj.device)
    wsb = lib.shard_b200_k_quantize_workspace_bytes(n, keep)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=proj.device)
    scale = torch.empty(keep, dtype=torch.float32, device=proj.device)
    packed = torch.empty(n * keep // 2, dtype=torch.uint8, device=proj.device)
    check(lib.shard_b200_k_quantize_pack(ptr(_c(proj, torch.float32)), ptr(alloc_t), n, keep, ptr(scale),
                                         ptr(packed), ptr(ws), wsb, cur_stream()), "k_quantize_pack")
    return packed, scale


def int4_pack(x):
    """Flat int8 in [-7, 7] -> nibbles (reference: triton_kernels.py:665-682)."""
    require_cuda(x)
    flat = _c(x.reshape(-1), torch.int8)
    out = torch.empty((flat.numel() + 1) // 2, dtype=torch.uint8, device=x.device)
    check(_lib.load().shard_b200_int4_pack(ptr(flat), flat.numel(), ptr(out), cur_stream()), "int4_pack")
    return out


def v_hadamard_normalise(v):
    """v: (nkv, n, 128) fp16 view -> (x (nkv, n, 128) fp32 = H(v)/ch_max, ch_max (nkv, 128) fp32)."""
    require_cuda(v)
    if v.dtype != torch.float16 or v.stride(-1) != 1:
        raise _lib.ShardError("v_hadamard_normalise expects fp16 values with a contiguous head dimension")
    nkv, n, _ = v.shape
    x = torch.empty(nkv, n, HD, dtype=torch.float32, device=v.device)
    ch = torch.empty(nkv, HD, dtype=torch.float32, device=v.device)
    check(_lib.load().shard_b200_v_hadamard_normalise(ptr(v), v.stride(0), v.stride(1), nkv, n, ptr(x),
                                                      ptr(ch), cur_stream()), "v_hadamard_normalise")
    return x, ch


def vq_assign(x, centroids, want_i64=True):
    """Nearest centroid of each row of x (N, 4); returns (idx u8, idx int64 or None)."""
    require_cuda(x, centroids)
    n = x.shape[0]
    if x.shape[1] != 4 or tuple(centroids.shape) != (256, 4):
        raise _lib.ShardError("vq_assign supports 4-dim sub-vectors and a 256-entry codebook")
    u8 = torch.empty(n, dtype=torch.uint8, device=x.device)
    i64 = torch.empty(n, dtype=torch.int64, device=x.device) if want_i64 else None
    check(_lib.load().shard_b200_vq_assign(ptr(_c(x, torch.float32)), ptr(_c(centroids, torch.float32)), n,
                                           ptr(u8), ptr(i64), cur_stream()), "vq_assign")
    return u8, i64


def vq_assign_accumulate(x, centroids, sums, counts):
    """vq_assign + per-centroid sums (256, 4) and counts (256,) of the same pass (both zeroed here);
    returns the u8 indices."""
    require_cuda(x, centroids, sums, counts)
    n = x.shape[0]
    if x.shape[1] != 4 or tuple(centroids.shape) != (256, 4):
        raise _lib.ShardError("vq_assign supports 4-dim sub-vectors and a 256-entry codebook")
    u8 = torch.empty(n, dtype=torch.uint8, device=x.device)
    sums.zero_()
    counts.zero_()
    check(_lib.load().shard_b200_vq_assign_accumulate(ptr(_c(x, torch.float32)), ptr(_c(centroids, torch.float32)), n,
                                                      ptr(u8), ptr(_c(sums, torch.float32)),
                                                      ptr(_c(counts, torch.float32)), cur_stream()),
          "vq_assign_accumulate")
    return u8


# --------------------------------------------------------------------------- decode
def phase_table_numel(n):
    """fp16 elements of the phase table of `n` tokens (tokens are padded to blocks of 32)."""
    return max(_lib.load().shard_b200_phase_table_bytes(int(n)) // 2, 128 * 32)


def phase_table(compress_start, pos_q, n, inv_freq, out=None):
    """fp16 cos / sin of fp32(compress_start + t - pos_q) * inv_freq for t < n, in the
    block-of-32-tokens plane layout the decode kernel reads (flat fp16 tensor)."""
    require_cuda(inv_freq)
    if out is None:
        out = torch.empty(phase_table_numel(n), dtype=torch.float16, device=inv_freq.device)
    elif out.numel() < phase_table_numel(n):
        raise _lib.ShardError("phase table buffer too small")
    check(_lib.load().shard_b200_phase_table(int(compress_start), int(pos_q), int(n),
                                             ptr(_c(inv_freq, torch.float32)), ptr(out), cur_stream()),
          "phase_table")
    return out


def decode_prepare(basis_f16, coeff_scale_f16, mean_f16, nkv, rank):
    require_cuda(basis_f16, coeff_scale_f16, mean_f16)
    lib = _lib.load()
    nbytes = lib.shard_b200_wprep_bytes(nkv, rank)
    if nbytes == 0:
        raise _lib.ShardError(f"unsupported PCA rank {rank}: must be a multiple of 32 in [32, 192]")
    out = torch.empty(nbytes, dtype=torch.uint8, device=basis_f16.device)
    check(lib.shard_b200_decode_prepare(ptr(_c(basis_f16, torch.float16)), ptr(_c(coeff_scale_f16, torch.float16)),
                                        ptr(_c(mean_f16, torch.float16)), nkv, rank, ptr(out), cur_stream()),
          "decode_prepare")
    return out


def make_shape(n_q, nkv, rank, n_comp, tok_begin, tok_end, n_sink, n_win, n_stream, pos_q, partial_out=False,
               append=False, n_dec=0):
    sh = ShardDecodeShape()
    sh.n_q, sh.nkv, sh.rank, sh.n_comp = n_q, nkv, rank, n_comp
    sh.tok_begin, sh.tok_end = tok_begin, tok_end
    sh.n_sink, sh.n_win, sh.n_stream = n_sink, n_win, n_stream
    sh.pos_q, sh.partial_out, sh.append = int(pos_q), int(bool(partial_out)), int(bool(append))
    sh.n_dec = int(n_dec)
    return sh


def decode_workspace_bytes(shape, batch=1):
    n = _lib.load().shard_b200_decode_workspace_bytes(C.byref(shape), batch)
    if n == 0:
        raise _lib.ShardError("decode shape rejected by the library")
    return n


def decode_attn(seq_or_table, batch, shape, inv_freq, codebook, workspace):
    """Launch the fused decode.  `seq_or_table` is a ShardSeq (batch 1) or a uint8 CUDA tensor
    holding `batch` ShardSeq records; `inv_freq` / `codebook` are tensors or raw device pointers."""
    lib = _lib.load()
    if batch == 1:
        seq_ptr = C.addressof(seq_or_table)
    else:
        seq_ptr = seq_or_table.data_ptr()
    inv = inv_freq if isinstance(inv_freq, int) else ptr(inv_freq)
    cb = codebook if isinstance(codebook, int) else ptr(codebook)
    rc = lib.shard_b200_decode_attn(seq_ptr, batch, C.byref(shape), inv, cb, workspace.data_ptr(),
                                    workspace.numel() * workspace.element_size(), cur_stream())
    if rc:
        check(rc, "decode_attn")


def decode_status(workspace=None):
    """Status word of the decode launches that used `workspace` (None: the library's built-in
    scratch on the current device): 0, or 1 if a bounded in-kernel wait gave up.  Waits for the
    current stream and clears a set word."""
    word = C.c_int32(0)
    check(_lib.load().shard_b200_decode_status(None if workspace is None else workspace.data_ptr(),
                                               C.byref(word), cur_stream()), "decode_status")
    return int(word.value)


def decode_status_check(workspace=None):
    if decode_status(workspace) != 0:
        raise _lib.ShardError("a decode launch gave up on a bounded in-kernel wait; its output is undefined")


def lse_merge(parts, out=None):
    """parts: (n_parts, n_q, 132) fp32 -> (n_q, 128) fp16."""
    require_cuda(parts)
    n_parts, n_q, stride = parts.shape
    if stride != _lib.PART_STRIDE:
        raise _lib.ShardError("partials must have 132 floats per head")
    if out is None:
        out = torch.empty(n_q, HD, dtype=torch.float16, device=parts.device)
    check(_lib.load().shard_b200_lse_merge(ptr(_c(parts, torch.float32)), n_parts, n_q, ptr(out), cur_stream()),
          "lse_merge")
    return out


def seq_table(seqs, device):
    """Pack a list of ShardSeq records into a CUDA byte tensor (the `batch > 1` table)."""
    raw = b"".join(bytes(s) for s in seqs)
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
