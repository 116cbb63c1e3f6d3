"""Multi-GPU execution of the compressed-KV decode: batch sharding and sequence split.

The reference is single-GPU; both modes are additions that keep its per-layer
tensor dictionary as the unit of work.

* batch-sharded: sequences are independent caches, so rank r simply owns a
  contiguous block of them -- no communication on the data path.
  `BatchedDecoder` launches one kernel per layer for all local sequences.
* sequence-split: one long sequence's compressed middle is cut into contiguous
  token ranges, one per rank.  Every rank runs the fused decode on its range and
  emits per query head (max, sum-exp, acc[128]); the records (16.9 KB per rank and
  layer) travel over NVLink peer memory -- delivered by the decode launch itself and
  merged by a kernel that is already polling (`PeerExchange`) -- or, without peer
  access, are all-gathered over NCCL and combined with the same log-sum-exp kernel
  that merges the split-KV partials inside one GPU.  Rank 0 also owns the fp16
  sink/window and the streamed tokens.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib, ops
from ._lib import ShardSeq, ptr

TOKEN_ALIGN = 128  # decode tiles are 128 tokens; ranges start on tile boundaries


def split_ranges(n_comp: int, world: int, align: int = TOKEN_ALIGN):
    """Contiguous [begin, end) token ranges of the middle segment, one per rank.

    Boundaries are multiples of `align`; sizes differ by at most `align`; a rank may
    get an empty range when there are fewer tiles than ranks.
    """
    if world < 1:
        raise ValueError("world must be >= 1")
    tiles = (n_comp + align - 1) // align
    base, extra = divmod(tiles, world)
    out, t = [], 0
    for r in range(world):
        nt = base + (1 if r < extra else 0)
        b, e = min(t * align, n_comp), min((t + nt) * align, n_comp)
        out.append((b, e))
        t += nt
    return out


def batch_shard(n_seqs: int, rank: int, world: int):
    """Indices of the sequences rank `rank` owns (contiguous block, sizes differ by <= 1)."""
    base, extra = divmod(n_seqs, world)
    lo = rank * base + min(rank, extra)
    return list(range(lo, lo + base + (1 if rank < extra else 0)))


def shard_layer_tokens(gc: dict, rank: int, world: int) -> dict:
    """A rank's slice of one layer's dictionary for sequence-split decode.

    Keeps rows [begin, end) of the packed coefficients and VQ codes, shifts
    `compress_start` so that positions stay absolute, replicates the small tensors
    (basis, mean, codebook, channel scales).  Only rank 0 keeps the fp16 segments.
    Pure tensor slicing: works on any device.
    """
    begin, end = split_ranges(gc["n_compress"], world)[rank]
    n_total, keep = gc["k_coeffs_shape"]
    rows = gc["k_coeffs"].view(n_total, keep // 2)[begin:end]
    out = {k: v for k, v in gc.items() if not k.startswith("_") and k not in (
        "k_wprep", "k_coeffs_kernel", "k_coeffs_padded", "k_rank_kernel", "v_qdata", "v_packed")}
    out["k_coeffs"] = rows.contiguous().view(-1)
    out["k_coeffs_shape"] = (end - begin, keep)
    out["v_indices_u8"] = gc["v_indices_u8"][:, begin:end].contiguous()
    out["v_packed"] = out["v_indices_u8"].view(-1)
    out["n_compress"] = end - begin
    out["compress_start"] = gc["compress_start"] + begin
    out["token_range"] = (begin, end)
    if rank != 0:
        for name in ("sink_k", "sink_v", "win_k", "win_v"):
            out[name] = gc[name][:, :, :0]
        for name in list(out):
            if name.endswith("_buf") or name in ("stream_n", "signs"):
                del out[name]
    return out


def all_gather_partials(part: torch.Tensor, group=None, out: torch.Tensor | None = None):
    """All-gather one (n_q, 132) fp32 partial per rank into (world, n_q, 132), rank order."""
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world, *part.shape), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(out.view(-1), part.contiguous().view(-1), group=group)
    return out


class PeerExchange:
    """Exchange buffers of the ranks of one node, opened over CUDA IPC, and the epoch counter of
    `shard_b200_seqsplit_merge`: the partial records of a sequence-split decode step travel as
    plain peer stores over NVLink and are merged by the same kernel that sent them, instead of an
    NCCL all-gather followed by a merge launch.  All ranks must call `merge` the same number of
    times, in the same order.  Needs every rank on its own GPU of one node with peer access."""

    def __init__(self, nkv: int, group=None, device=None, timeout_us: int = 0):
        import ctypes as C
        self.group = group
        self.timeout_us = int(timeout_us)      # bound of the in-kernel flag wait; 0 = library default (0.2 s)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.nkv = nkv
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        lib = _lib.load()
        nbytes = lib.shard_b200_peer_buffer_bytes(self.world, nkv)
        if nbytes == 0:
            raise _lib.ShardError("unsupported world size for the peer exchange (1..16 ranks)")
        own = C.c_void_p()
        handle = C.create_string_buffer(64)
        with torch.cuda.device(self.dev):
            _lib.check(lib.shard_b200_peer_alloc(nbytes, C.byref(own), handle), "peer_alloc")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self._own = own.value
            self._opened = []
            ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    ptrs.append(self._own)
                    continue
                p = C.c_void_p()
                hbuf = C.create_string_buffer(handles[r], 64)
                _lib.check(lib.shard_b200_peer_open(hbuf, C.byref(p)), "peer_open")
                self._opened.append(p.value)
                ptrs.append(p.value)
        self._ptrs = (C.c_void_p * self.world)(*ptrs)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.epoch = 0
        self.fused_out = None
        dist.barrier(group=group)            # every buffer is zeroed and opened before the first store

    def merge(self, part: torch.Tensor, out: torch.Tensor | None = None):
        """part: this rank's (n_q, 132) fp32 record -> (n_q, 128) fp16 merged over all ranks."""
        n_q = 4 * self.nkv
        if out is None:
            out = torch.empty(n_q, 128, dtype=torch.float16, device=part.device)
        self.epoch += 1
        _lib.check(_lib.load().shard_b200_seqsplit_merge(part.data_ptr(), self._ptrs, self.rank, self.world, self.nkv,
                                                         self.epoch, out.data_ptr(), self.status.data_ptr(),
                                                         self.timeout_us, _lib.cur_stream()), "seqsplit_merge")
        return out

    # -- fused form: the decode launch delivers, a polling kernel merges -----------------------
    def launch_decode(self, seq, shape, inv_ptr, cb_ptr, ws):
        """Called by `decode_layer(..., push=self)`: the decode launch of the NEXT epoch, whose
        combining CTAs store the rank's record into every rank's buffer and publish the epoch.
        With `self.fused_out` set (by `decode_merge`) the same CTAs also wait for all ranks' records
        and write the merged output there: the step is one launch."""
        import ctypes as C
        fused = self.fused_out
        _lib.check(_lib.load().shard_b200_decode_attn_seqsplit(
            C.addressof(seq), C.byref(shape), inv_ptr, cb_ptr, ws.data_ptr(), ws.numel() * ws.element_size(),
            self._ptrs, self.rank, self.world, self.epoch + 1,
            None if fused is None else fused.data_ptr(), self.status.data_ptr(), self.timeout_us,
            _lib.cur_stream()), "decode_attn_seqsplit")
        if fused is not None:
            self.epoch += 1

    def decode_merge(self, q_rope, layer, pos_q, out: torch.Tensor | None = None, with_fp16_segments=True):
        """One launch: decode this rank's slice, deliver the record to every rank, wait for theirs,
        merge.  Returns the (n_q, 128) fp16 output (identical on all ranks)."""
        from .attention import decode_layer
        n_q = 4 * self.nkv
        if out is None:
            out = torch.empty(n_q, 128, dtype=torch.float16, device=self.dev)
        self.fused_out = out
        try:
            decode_layer(q_rope, layer, pos_q, partial_out=True, with_fp16_segments=with_fp16_segments, push=self)
        finally:
            self.fused_out = None
        return out

    def wait_merge(self, out: torch.Tensor | None = None):
        """Wait for every rank's record of the epoch `launch_decode` delivered and merge them."""
        n_q = 4 * self.nkv
        if out is None:
            out = torch.empty(n_q, 128, dtype=torch.float16, device=self.dev)
        self.epoch += 1
        _lib.check(_lib.load().shard_b200_seqsplit_wait_merge(self._ptrs, self.rank, self.world, self.nkv, self.epoch,
                                                              out.data_ptr(), self.status.data_ptr(),
                                                              self.timeout_us, _lib.cur_stream()),
                   "seqsplit_wait_merge")
        return out

    def check(self):
        """Raise if a bounded wait inside a merge gave up (synchronises the device)."""
        if int(self.status.item()) != 0:
            raise _lib.ShardError("sequence-split merge timed out waiting for a peer's records")

    def close(self):
        lib = _lib.load()
        torch.cuda.synchronize(self.dev)
        dist.barrier(group=self.group)       # nobody is still storing into a buffer that goes away
        for p in self._opened:
            lib.shard_b200_peer_close(p)
        self._opened = []
        if self._own:
            lib.shard_b200_peer_free(self._own)
            self._own = None


def neutral_partial(n_q: int, device):
    """The record of a rank that has nothing to attend to: max = -inf, sum-exp = 0, acc = 0.
    Every merge gives it weight zero."""
    part = torch.zeros(n_q, _lib.PART_STRIDE, dtype=torch.float32, device=device)
    part[:, 0] = float("-inf")
    return part


def seqsplit_decode(q_rope, layer, pos_q, group=None, gather_buf=None, timing=None, peer=None, out=None,
                    part_buf=None):
    """Sequence-split decode of one layer whose dictionary was cut by `shard_layer_tokens`.

    Every rank calls this with the same query; all ranks return the same
    (1, n_q, 1, hd) fp16 tensor (the combine runs in fixed rank order).  With `peer`
    (a `PeerExchange`) the decode launch delivers its record into every rank's exchange
    buffer over NVLink and a merge kernel that is already polling finishes the step;
    without it the records go through an NCCL all-gather followed by `lse_merge`.
    A rank whose range is empty (fewer tiles than ranks) and that owns no fp16 / streamed
    rows launches no decode and contributes the neutral record.
    `timing`, if given, is a dict receiving CUDA events around the merge step.
    """
    from .attention import decode_layer
    rank = dist.get_rank(group)
    gc = layer._gpu_compressed
    n_q = q_rope.shape[1]
    first = rank == 0
    n_rows = 0
    if first:
        n_rows = gc["sink_k"].shape[2] + gc["win_k"].shape[2] + gc.get("stream_n", 0)
        n_rows += gc["decode_k"].shape[2] if "decode_k" in gc else 0
    idle = gc["n_compress"] == 0 and n_rows == 0
    out2 = None if out is None else out.view(n_q, q_rope.shape[3])
    if peer is not None and not idle:
        if timing is None:
            res = peer.decode_merge(q_rope, layer, pos_q, out2, with_fp16_segments=first)   # one launch
        else:
            decode_layer(q_rope, layer, pos_q, partial_out=True, with_fp16_segments=first, out=part_buf, push=peer)
            timing["merge_start"].record()
            res = peer.wait_merge(out2)
    else:
        part = (neutral_partial(n_q, q_rope.device) if idle else
                decode_layer(q_rope, layer, pos_q, partial_out=True, with_fp16_segments=first, out=part_buf))
        if timing is not None:
            timing["merge_start"].record()
        if peer is not None:
            res = peer.merge(part, out2)
        else:
            parts = all_gather_partials(part, group, gather_buf)
            res = ops.lse_merge(parts, out2)
    if timing is not None:
        timing["merge_end"].record()
    return res.view(1, n_q, 1, q_rope.shape[3])


class BatchedDecoder:
    """Decode step over many independent single-sequence caches with one launch per layer.

    All caches must be compressed with identical geometry (n_comp, rank, heads) and
    advance in lock step (same query position), which is what a batch of equal-length
    prompts does.  Stream buffers are allocated once with `stream_capacity` rows so the
    device pointer tables never change.
    """

    def __init__(self, caches, stream_capacity=512):
        from .streaming import get_codebook, stream_signs
        if not caches:
            raise ValueError("no caches")
        self.caches = caches
        c0 = caches[0]
        self.n_layers = c0._num_layers
        self.nkv = c0._n_kv_heads
        self.n_q = 4 * self.nkv
        self.hd = c0.head_dim
        g0 = c0.layers[0]._gpu_compressed
        self.dev = g0["k_coeffs"].device
        self.n_comp = g0["n_compress"]
        self.rank_k = g0["k_rank_kernel"]
        self.compress_start = g0["compress_start"]
        self.n_sink, self.n_win = g0["sink_k"].shape[2], g0["win_k"].shape[2]
        self.S = len(caches)
        self.capacity = stream_capacity
        self.n_stream = 0
        S, dev = self.S, self.dev
        self.q = torch.zeros(self.n_layers, S, self.n_q, self.hd, dtype=torch.float16, device=dev)
        self.out = torch.zeros(self.n_layers, S, self.n_q, self.hd, dtype=torch.float16, device=dev)
        self.new_k = torch.zeros(self.n_layers, S, self.nkv, self.hd, dtype=torch.float16, device=dev)
        self.new_v = torch.zeros(self.n_layers, S, self.nkv, self.hd, dtype=torch.float16, device=dev)
        self.codebook = get_codebook(self.hd, 8, dev)
        self.inv_freq = c0._inv_freq(dev)
        self.phase = torch.empty(ops.phase_table_numel(self.n_comp), dtype=torch.float16, device=dev)
        self.tables = []
        self._keep = []
        for li in range(self.n_layers):
            seqs = []
            for si, c in enumerate(caches):
                gc = c.layers[li]._gpu_compressed
                if (gc["n_compress"], gc["k_rank_kernel"]) != (self.n_comp, self.rank_k):
                    raise ValueError("caches of a batch must share n_comp and PCA rank")
                bufs = {
                    "k_idx": torch.zeros(stream_capacity, self.nkv, self.hd, dtype=torch.uint8, device=dev),
                    "v_idx": torch.zeros(stream_capacity, self.nkv, self.hd, dtype=torch.uint8, device=dev),
                    "k_norm": torch.zeros(stream_capacity, self.nkv, dtype=torch.float16, device=dev),
                    "v_norm": torch.zeros(stream_capacity, self.nkv, dtype=torch.float16, device=dev),
                    "signs": stream_signs(li, self.hd, dev),
                }
                self._keep.append(bufs)
                gc["batched_stream"] = bufs
                s = ShardSeq()
                s.k_coeffs, s.k_wprep = ptr(gc["k_coeffs_kernel"]), ptr(gc["k_wprep"])
                s.v_indices, s.v_centroids, s.v_ch = ptr(gc["v_indices_u8"]), ptr(gc["v_centroids_f16"]), ptr(gc["v_ch_f16"])
                for name in ("sink_k", "sink_v", "win_k", "win_v"):
                    t = gc[name] if gc[name].is_contiguous() else gc[name].contiguous()
                    gc[name] = t
                    setattr(s, name, ptr(t) if t.numel() else None)
                s.st_k_idx, s.st_v_idx = ptr(bufs["k_idx"]), ptr(bufs["v_idx"])
                s.st_k_norm, s.st_v_norm = ptr(bufs["k_norm"]), ptr(bufs["v_norm"])
                s.signs = ptr(bufs["signs"])
                s.phase = ptr(self.phase)
                s.q, s.out = ptr(self.q[li, si]), ptr(self.out[li, si])
                s.new_k, s.new_v = ptr(self.new_k[li, si]), ptr(self.new_v[li, si])
                seqs.append(s)
            self.tables.append(ops.seq_table(seqs, dev) if S > 1 else seqs[0])
        shape = self._shape(0, self.capacity)
        self.ws = torch.zeros(ops.decode_workspace_bytes(shape, S), dtype=torch.uint8, device=dev)

    def _shape(self, pos_q, n_stream, append=False):
        return ops.make_shape(self.n_q, self.nkv, self.rank_k, self.n_comp, 0, self.n_comp,
                              self.n_sink, self.n_win, n_stream, pos_q, False, append=append)

    def step(self, pos_q):
        """Append self.new_k/new_v (all layers, all sequences) to the streams, then attend
        with self.q; results land in self.out.  Launches 1 + n_layers kernels: the phase table,
        then per layer one kernel that appends, attends and combines."""
        if self.n_stream >= self.capacity:
            raise _lib.ShardError("stream capacity exhausted")
        lib = _lib.load()
        st = _lib.cur_stream()
        ops.phase_table(self.compress_start, pos_q, self.n_comp, self.inv_freq, out=self.phase)
        shape = self._shape(pos_q, self.n_stream + 1, append=True)
        import ctypes as C
        for li in range(self.n_layers):
            tab = self.tables[li]
            tptr = tab.data_ptr() if self.S > 1 else C.addressof(tab)
            _lib.check(lib.shard_b200_decode_attn(tptr, self.S, C.byref(shape), ptr(self.inv_freq),
                                                  ptr(self.codebook), ptr(self.ws), self.ws.numel(), st),
                       "decode_attn")
        self.n_stream += 1
        return self.out

    def check(self):
        """Raise `ShardError` if a launch of this decoder gave up on a bounded in-kernel wait since
        the last check.  Waits for the current stream: once per step or request, not per layer."""
        ops.decode_status_check(self.ws)
