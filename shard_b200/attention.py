"""Decode attention over a compressed cache + the Llama attention hook.

`fused_attention_compressed` keeps the reference's signature
(src/shard/attention.py:270-343) and returns the same tensor, but the whole
computation -- scores on packed int4 PCA coefficients through the per-pair
relative-phase RoPE identity, the fp16 sink/window segments, the 8-bit streamed
tokens, one global softmax, the VQ-V weighted sum and the single inverse
Hadamard -- is one kernel launch of libshard_b200.so.
"""
from __future__ import annotations

import torch

from . import _lib, ops
from ._lib import ShardSeq, ptr
from .streaming import get_codebook

GQA = 4
# a forward over more new tokens than this after compression takes the dequantised path (one launch
# per query token would no longer pay)
MAX_FUSED_QUERY_TOKENS = 256


def _phase_for(cache, gc, pos_q, tok_begin, tok_end, dev):
    """cos/sin table of the step; all layers of a step share positions, so it is
    computed by the first layer that asks and reused by the others.  A forward over several
    new tokens needs one table per query position: `cache._phase_keep` tables are kept then
    (least recently made first out)."""
    key = (int(pos_q), gc["compress_start"], tok_begin, tok_end)
    if cache._phase_key == key:
        return cache._phase
    tabs = getattr(cache, "_phase_tabs", None)
    if tabs is None:
        tabs = cache._phase_tabs = {}
    tab = tabs.get(key)
    if tab is None:
        n = tok_end - tok_begin
        need = ops.phase_table_numel(n)
        keep = max(1, int(getattr(cache, "_phase_keep", 1)))
        tab = None
        while len(tabs) >= keep:                       # reuse the oldest table's memory
            old = tabs.pop(next(iter(tabs)))
            if tab is None and old.numel() >= need and old.device == dev:
                tab = old
        if tab is None:
            tab = torch.empty(need, dtype=torch.float16, device=dev)
        ops.phase_table(gc["compress_start"] + tok_begin, pos_q, n, cache._inv_freq(dev), out=tab)
        tabs[key] = tab
    cache._phase, cache._phase_key = tab, key
    return tab


def _seq_record(gc, dev):
    """ShardSeq of a layer: static pointers are filled once and cached in the dict."""
    seq = gc.get("_seq")
    if seq is None:
        seq = ShardSeq()
        seq.k_coeffs = ptr(gc["k_coeffs_kernel"])
        seq.k_wprep = ptr(gc["k_wprep"])
        seq.v_indices = ptr(gc["v_indices_u8"])
        seq.v_centroids = ptr(gc["v_centroids_f16"])
        seq.v_ch = ptr(gc["v_ch_f16"])
        for name in ("sink_k", "sink_v", "win_k", "win_v"):
            t = gc[name]
            if not t.is_contiguous():
                t = gc[name] = t.contiguous()
            setattr(seq, name, ptr(t) if t.numel() else None)
        gc["_seq"] = seq
    if "k_idx_buf" in gc:
        seq.st_k_idx, seq.st_v_idx = ptr(gc["k_idx_buf"]), ptr(gc["v_idx_buf"])
        seq.st_k_norm, seq.st_v_norm = ptr(gc["k_norm_buf"]), ptr(gc["v_norm_buf"])
        seq.signs = ptr(gc["signs"])
    return seq


class _Launch:
    """Per-layer launch state that does not change from step to step: the sequence record, the
    shape record (only n_stream / pos_q / append / n_dec are touched per step), workspace need
    and the constant device pointers."""
    __slots__ = ("key", "seq", "shape", "need", "inv_ptr", "cb", "cb_ptr", "dev", "dev_index", "kbuf")


def _launch_state(gc, cache, dev, nkv, n_q, t0, t1, with_fp16_segments, partial_out):
    n_sink = gc["sink_k"].shape[2] if with_fp16_segments else 0
    n_win = gc["win_k"].shape[2] if with_fp16_segments else 0
    key = (t0, t1, n_sink, n_win, bool(partial_out), gc["n_compress"], gc["k_rank_kernel"], dev)
    ls = gc.get("_launch")
    if ls is None or ls.key != key:
        _lib.require_cuda(gc["k_wprep"], gc["v_indices_u8"])       # same device as the query, and the current one
        if gc["k_wprep"].device != dev:
            raise _lib.ShardError(f"query on {dev} but the cache lives on {gc['k_wprep'].device}")
        ls = _Launch()
        ls.key = key
        ls.dev, ls.dev_index = dev, dev.index
        ls.seq = _seq_record(gc, dev)
        ls.kbuf = None
        ls.shape = ops.make_shape(n_q, nkv, gc["k_rank_kernel"], gc["n_compress"], t0, t1, n_sink, n_win, 0, 0,
                                  partial_out)
        # With a middle segment the scratch size does not depend on the number of rows (they ride
        # along in the middle's CTAs), only on whether there are any; without one it is asked for
        # per call.
        ls.need = 0
        if t1 > t0:
            probe = ops.make_shape(n_q, nkv, gc["k_rank_kernel"], gc["n_compress"], t0, t1, n_sink, n_win, 1, 0,
                                   partial_out)
            ls.need = ops.decode_workspace_bytes(probe, 1)
        ls.inv_ptr = ptr(cache._inv_freq(dev))
        ls.cb = get_codebook(128, 8, dev)
        ls.cb_ptr = ptr(ls.cb)
        gc["_launch"] = ls
    return ls


def decode_layer(q_rope, layer, pos_q, tok_range=None, partial_out=False, with_fp16_segments=True, out=None,
                 push=None, visible_new=None):
    """Run the fused decode for one layer.

    q_rope: (1, n_q, 1, 128) fp16 CUDA.  `tok_range` limits the middle segment to
    [begin, end) (sequence-split mode); `partial_out` returns the fp32
    (n_q, 132) record (max, sum-exp, 0, 0, acc[128]) instead of fp16 attention.
    `push` (a `parallel.PeerExchange`, with `partial_out`) makes the launch deliver that
    record into every rank's exchange buffer itself.  `visible_new` limits the decoded tokens
    (streamed rows, or rows of the fp16 decode buffer) the query attends to, to the first
    `visible_new` of them: the causal mask of a forward over several new tokens.

    A bounded wait that gives up inside the kernel leaves a status word in the cache's
    workspace; `Cache.check()` reads it (once per step or request, it synchronises).
    """
    gc = layer._gpu_compressed
    cache = layer._cache_ref
    if not q_rope.is_cuda:
        raise _lib.ShardError("shard_b200 kernels need CUDA tensors; there is no CPU fallback")
    B, n_q, s_q, hd = q_rope.shape
    nkv = cache._n_kv_heads
    if B != 1 or s_q != 1:
        raise NotImplementedError("decode kernel takes one query token of one sequence")
    if hd != 128 or n_q != GQA * nkv:
        raise NotImplementedError("decode kernel is built for head_dim 128 and 4 query heads per KV head")
    if q_rope.dtype != torch.float16:
        raise NotImplementedError("fp16 queries only")
    dev = q_rope.device
    t0, t1 = (0, gc["n_compress"]) if tok_range is None else tok_range
    ls = _launch_state(gc, cache, dev, nkv, n_q, t0, t1, with_fp16_segments, partial_out)
    # kernels go to the current device's current stream with raw pointers: the tensors must live there
    cur = torch.cuda.current_device()
    if cur != ls.dev_index:
        raise _lib.ShardError(f"tensor lives on cuda:{ls.dev_index} but the current device is cuda:{cur}; "
                              "make the tensor's device current (torch.cuda.device) before the call")
    n_stream = gc.get("stream_n", 0) if with_fp16_segments else 0
    if visible_new is not None and n_stream > 0:
        n_stream = min(n_stream, int(visible_new))
    pending = gc.pop("_pending", None)
    if pending is not None and (not with_fp16_segments or pending[2] != n_stream - 1):
        gc["_pending"] = pending
        layer._flush_pending()
        pending = None
    seq, shape = ls.seq, ls.shape
    if n_stream > 0:
        kbuf = gc["k_idx_buf"]
        if ls.kbuf is not kbuf:                        # the stream buffers were (re)allocated
            ls.kbuf = kbuf
            seq.st_k_idx, seq.st_v_idx = kbuf.data_ptr(), gc["v_idx_buf"].data_ptr()
            seq.st_k_norm, seq.st_v_norm = gc["k_norm_buf"].data_ptr(), gc["v_norm_buf"].data_ptr()
            seq.signs = gc["signs"].data_ptr()
    if pending is not None:
        seq.new_k, seq.new_v = pending[0].data_ptr(), pending[1].data_ptr()
    n_dec = dec_cap = 0
    if with_fp16_segments and "decode_k" in gc:
        # tokens a non-streaming cache appends as they are: views of the rows in use of buffers
        # (1, nkv, capacity, 128) allocated ahead, or plain (1, nkv, s, 128) tensors
        dk, dv = gc["decode_k"], gc["decode_v"]
        if dk.dtype != torch.float16:
            raise NotImplementedError("fp16 models only")
        if dk.stride(3) != 1 or dk.stride(2) != hd or dv.stride(3) != 1 or dv.stride(2) != hd or dv.stride(1) != dk.stride(1):
            dk, dv = gc["decode_k"], gc["decode_v"] = dk.contiguous(), dv.contiguous()
        n_dec = dk.shape[2]
        dec_cap = dk.stride(1) // hd if nkv > 1 else n_dec   # rows allocated per KV head
        if visible_new is not None:
            n_dec = min(n_dec, int(visible_new))
        seq.dec_k, seq.dec_v = dk.data_ptr(), dv.data_ptr()
    q2 = q_rope
    if q2.stride(3) != 1 or q2.stride(1) != hd:
        q2 = q_rope.reshape(n_q, hd).contiguous()
    if push is not None and not partial_out:
        raise _lib.ShardError("a launch that delivers to the peers emits the partial record")
    if out is None and push is None:
        out = (torch.empty(n_q, _lib.PART_STRIDE, dtype=torch.float32, device=dev) if partial_out
               else torch.empty(n_q, hd, dtype=torch.float16, device=dev))
    elif out is not None and (not out.is_contiguous() or out.numel() != n_q * (_lib.PART_STRIDE if partial_out else hd)):
        raise _lib.ShardError("out must be a contiguous (n_q, 128) fp16 or (n_q, 132) fp32 tensor")
    # with `push` and no `out` the record only goes to the exchange buffers
    seq.q, seq.out = q2.data_ptr(), (None if out is None else out.data_ptr())
    seq.phase = _phase_for(cache, gc, pos_q, t0, t1, dev).data_ptr() if t1 > t0 else None
    shape.n_stream, shape.pos_q, shape.append = n_stream, int(pos_q), int(pending is not None)
    shape.n_dec, shape.dec_cap = n_dec, dec_cap
    # the first launch on a freshly built dictionary follows the kernels that wrote its codes and
    # weights: it must not start early behind them
    shape.no_overlap = int(gc.pop("_fresh", False))
    need = ls.need
    if t1 == t0:                                       # rows only: scratch grows with the rows
        need = ops.decode_workspace_bytes(shape, 1)
    ws = cache._decode_ws
    if ws is None or ws.numel() < need or ws.device != dev:
        # zero-filled: the header's status word and arrival counters must start at zero
        ws = cache._decode_ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=dev)
    if push is not None:
        push.launch_decode(seq, shape, ls.inv_ptr, ls.cb_ptr if n_stream > 0 else None, ws)
    else:
        ops.decode_attn(seq, 1, shape, ls.inv_ptr, ls.cb_ptr if n_stream > 0 else None, ws)
    return out


def fused_attention_compressed(q_rope, layer, pos_q, inv_freq=None, attn_mask=None, out=None):
    """Attention of the new query token(s) over the layer's compressed cache; returns
    (1, n_q, s, hd) in q's dtype, or None if the layer is not compressed.

    One query token (s = 1, the decode step) is one kernel launch.  For s > 1 -- a forward over
    several new tokens after compression, which the reference serves by dequantising the whole
    cache (src/shard/attention.py:357-362, src/shard/cache.py:87-124) -- `pos_q` is the position
    of the LAST query; query j attends to everything before the s new tokens plus the first j + 1
    of them (causal), one launch per query token, nothing dequantised.  The new tokens must
    already have been appended (`update`).

    `attn_mask` is accepted for signature compatibility: for one sequence without padding the
    causal mask is what the above implements (the reference's own fused variant skips it for the
    same reason, src/shard/attention.py:254).  `inv_freq` is taken from the cache the layer
    belongs to.  `out` (not in the reference's signature) lets the caller name a contiguous
    (1, n_q, s, hd) fp16 tensor to write into.
    """
    gc = getattr(layer, "_gpu_compressed", None)
    if gc is None:
        return None
    _, n_q, s_q, hd = q_rope.shape
    if s_q == 1:
        res = decode_layer(q_rope, layer, pos_q, out=None if out is None else out.view(n_q, hd))
        return res.view(1, n_q, 1, hd)
    cache = layer._cache_ref
    layer._flush_pending()                             # every new token is in its row before the first query looks
    n_new_total = gc.get("stream_n", 0) if "k_idx_buf" in gc else (gc["decode_k"].shape[2] if "decode_k" in gc else 0)
    if n_new_total < s_q:
        raise _lib.ShardError("append the new tokens (update) before attending with them")
    res = torch.empty(s_q, n_q, hd, dtype=torch.float16, device=q_rope.device)
    prev_keep = getattr(cache, "_phase_keep", 1)
    cache._phase_keep = max(prev_keep, min(s_q, 8))    # the layers of this forward share the tables
    try:
        for j in range(s_q):
            decode_layer(q_rope[:, :, j:j + 1, :], layer, pos_q - (s_q - 1) + j, out=res[j],
                         visible_new=n_new_total - (s_q - 1) + j)
    finally:
        cache._phase_keep = prev_keep
    res = res.permute(1, 0, 2).unsqueeze(0)            # (1, n_q, s, hd)
    if out is not None:
        out.copy_(res)
        return out
    return res


def enable_llama_fused_attention(model=None):
    """Route LlamaAttention.forward through the fused decode kernel whenever the
    cache is a compressed `shard_b200.Cache` and exactly one new token is processed
    (reference: src/shard/attention.py:345-414).  Returns False if transformers'
    Llama is unavailable."""
    from .cache import Cache
    try:
        from transformers.models.llama import modeling_llama as ml
    except ImportError:
        return False
    attn_cls = ml.LlamaAttention
    if getattr(attn_cls, "_shard_b200_patched", False):
        return True
    stock_forward = attn_cls.forward

    def forward(self, hidden_states, position_embeddings=None, attention_mask=None,
                past_key_values=None, **kwargs):
        cache = past_key_values
        layer = cache.layers[self.layer_idx] if isinstance(cache, Cache) else None
        bsz, q_len = hidden_states.shape[:2]
        if (layer is not None and self.layer_idx == 0 and not cache._compressed and layer._prefilled
                and bsz == 1 and cache._rope_inv_freq is not None):
            # the first forward after the prefill: the reference compresses inside layer 0's update and
            # serves that layer from the dequantised cache once; compressing before layer 0 attends
            # lets every layer of this step take the fused kernel
            cache.compress()
        use_fused = (layer is not None and layer._gpu_compressed is not None
                     and 1 <= q_len <= MAX_FUSED_QUERY_TOKENS and bsz == 1
                     and cache._rope_inv_freq is not None)
        if not use_fused:
            return stock_forward(self, hidden_states, position_embeddings=position_embeddings,
                                 attention_mask=attention_mask, past_key_values=past_key_values, **kwargs)
        shape = (bsz, q_len, -1, self.head_dim)
        q = self.q_proj(hidden_states).view(shape).transpose(1, 2)
        k = self.k_proj(hidden_states).view(shape).transpose(1, 2)
        v = self.v_proj(hidden_states).view(shape).transpose(1, 2)
        cos, sin = position_embeddings
        q, k = ml.apply_rotary_pos_emb(q, k, cos, sin)
        cache._fused_decode_update = True
        try:
            cache.update(k, v, self.layer_idx, {"sin": sin, "cos": cos})
        finally:
            cache._fused_decode_update = False
        pos_q = layer.get_seq_length() - 1
        out = fused_attention_compressed(q, layer, pos_q, cache._rope_inv_freq, attention_mask)
        out = out.transpose(1, 2).reshape(bsz, q_len, -1)
        return self.o_proj(out), None

    attn_cls.forward = forward
    attn_cls._shard_b200_patched = True
    return True
