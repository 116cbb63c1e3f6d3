"""Sequence-split decode on ONE GPU: the exchange + merge kernels with several 'ranks' emulated
as launches on one stream over local exchange buffers, and the bounded waits running out.

Nothing here needs a second GPU or CUDA IPC: a rank is a (rank index, exchange buffer) pair, and
the launches run in an order in which nobody has to wait for a launch that comes later.  The
time-out tests leave one rank's flag unset on purpose; the kernel gives up after the stated bound,
reports through its status word and returns -- no trap, no fault, the context stays usable.
"""
import ctypes as C
import time

import numpy as np
import pytest
import torch

from conftest import tol_ok
from oracle import shard_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


class _LocalRank:
    """What `decode_layer(..., push=...)` needs from a `PeerExchange`, over local buffers."""

    def __init__(self, ptrs, rank, world, nkv=8):
        self._ptrs, self.rank, self.world, self.nkv, self.epoch = ptrs, rank, world, nkv, 0
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def launch_decode(self, seq, shape, inv_ptr, cb_ptr, ws):
        from shard_b200 import _lib
        fused = getattr(self, "fused_out", None)
        _lib.check(_lib.load().shard_b200_decode_attn_seqsplit(
            C.addressof(seq), C.byref(shape), inv_ptr, cb_ptr, ws.data_ptr(), ws.numel(), self._ptrs, self.rank,
            self.world, self.epoch + 1, None if fused is None else fused.data_ptr(), self.status.data_ptr(), 50000,
            _lib.cur_stream()), "decode_attn_seqsplit")
        if fused is not None:
            self.epoch += 1

    def wait_merge(self, out, timeout_us=0):
        from shard_b200 import _lib
        self.epoch += 1
        _lib.check(_lib.load().shard_b200_seqsplit_wait_merge(self._ptrs, self.rank, self.world, self.nkv, self.epoch,
                                                              out.data_ptr(), self.status.data_ptr(), timeout_us,
                                                              _lib.cur_stream()), "seqsplit_wait_merge")


def _exchange_buffers(world, nkv=8):
    from shard_b200 import _lib
    nbytes = _lib.load().shard_b200_peer_buffer_bytes(world, nkv)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
    return bufs, (C.c_void_p * world)(*[b.data_ptr() for b in bufs])


@pytest.mark.parametrize("world", [1, 2, 4])
def test_decode_launch_delivers_and_polling_kernel_merges(world):
    """Every 'rank' decodes its slice with a launch that delivers the record itself, then every
    rank's polling kernel merges: equal to whole-sequence decode, identical on all ranks, and
    identical to the exchange-and-merge kernel fed with the same partial records, over several
    steps (both buffer slots are reused)."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from gpu_helpers import FakeCache, FakeLayer, gc_to_device, random_gc, random_query
    from shard_b200 import _lib, ops
    from shard_b200.attention import decode_layer
    from shard_b200.cache import attach_kernel_format
    from shard_b200.parallel import shard_layer_tokens
    lib = _lib.load()
    n_comp, pos_q = 3000, 3200
    gc_np = random_gc(n_comp, seed=61)
    inv = torch.from_numpy(O.default_inv_freq())
    full = FakeLayer(gc_to_device(gc_np), FakeCache(inv))
    slices = []
    for r in range(world):
        sub = shard_layer_tokens(full._gpu_compressed, r, world)
        attach_kernel_format(sub, 8)
        slices.append(FakeLayer(sub, FakeCache(inv)))
    bufs, ptrs = _exchange_buffers(world)
    bufs2, ptrs2 = _exchange_buffers(world)
    ranks = [_LocalRank(ptrs, r, world) for r in range(world)]
    status2 = torch.zeros(1, dtype=torch.int32, device=DEV)
    for step in range(4):
        q_np = random_query(seed=70 + step)
        q = torch.from_numpy(q_np).to(DEV).view(1, 32, 1, 128)
        whole = decode_layer(q, full, pos_q).cpu().numpy()
        parts = []
        for r in range(world):
            part = torch.empty(32, 132, dtype=torch.float32, device=DEV)
            decode_layer(q, slices[r], pos_q, partial_out=True, with_fp16_segments=(r == 0), out=part,
                         push=ranks[r])
            parts.append(part)
        outs = [torch.full((32, 128), float("nan"), dtype=torch.float16, device=DEV) for _ in range(world)]
        for r in range(world):
            ranks[r].wait_merge(outs[r])
        torch.cuda.synchronize()
        got = [o.cpu().numpy() for o in outs]
        assert all(int(rk.status.item()) == 0 for rk in ranks)
        assert all(np.array_equal(g, got[0]) for g in got)
        assert np.abs(got[0].astype(np.float32) - whole.astype(np.float32)).max() <= 2e-3
        exact, *_ = O.attention_exact(q_np, gc_np, pos_q, O.default_inv_freq())
        assert tol_ok(got[0], exact, atol=1.5e-3, rtol=5e-3)
        # the same records through the kernel that stores, publishes, waits and merges in one launch,
        # and through lse_merge: same operations in the same order
        assert np.array_equal(ops.lse_merge(torch.stack(parts)).cpu().numpy(), got[0])
        alt = [torch.empty(32, 128, dtype=torch.float16, device=DEV) for _ in range(world)]
        # all ranks but the last would wait for a later launch: give them the records first
        # (the last rank's launch finds every flag in place; the others are re-run after it)
        for r in list(range(world)) + list(range(world - 1)):
            rc = lib.shard_b200_seqsplit_merge(parts[r].data_ptr(), ptrs2, r, world, 8, step + 1, alt[r].data_ptr(),
                                               status2.data_ptr(), 50000 if r < world - 1 else 0, _lib.cur_stream())
            assert rc == 0
        torch.cuda.synchronize()
        assert all(np.array_equal(a.cpu().numpy(), got[0]) for a in alt)
        status2.zero_()          # the first pass of ranks 0 .. world-2 ran out of time by design


def test_one_launch_step_with_a_world_of_one_and_its_wait_running_out():
    """The one-launch form (the delivering CTAs also wait and merge): with a world of one it must
    reproduce the plain decode bit for bit; with a world of two whose other rank never delivers, its
    bounded wait gives up, reports through the status word and leaves the output alone."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from gpu_helpers import FakeCache, FakeLayer, gc_to_device, random_gc, random_query
    from shard_b200.attention import decode_layer
    gc_np = random_gc(2000, seed=81)
    layer = FakeLayer(gc_to_device(gc_np), FakeCache(torch.from_numpy(O.default_inv_freq())))
    q = torch.from_numpy(random_query(seed=82)).to(DEV).view(1, 32, 1, 128)
    plain = decode_layer(q, layer, 2100).cpu().numpy()
    bufs, ptrs = _exchange_buffers(1)
    rk = _LocalRank(ptrs, 0, 1)
    for step in range(3):                                # both slots, reused
        rk.fused_out = torch.full((32, 128), float("nan"), dtype=torch.float16, device=DEV)
        decode_layer(q, layer, 2100, partial_out=True, push=rk)
        torch.cuda.synchronize()
        assert int(rk.status.item()) == 0
        assert np.array_equal(rk.fused_out.cpu().numpy(), plain)
    bufs2, ptrs2 = _exchange_buffers(2)
    lone = _LocalRank(ptrs2, 0, 2)
    lone.fused_out = torch.full((32, 128), 7.0, dtype=torch.float16, device=DEV)
    t0 = time.perf_counter()
    decode_layer(q, layer, 2100, partial_out=True, push=lone)   # rank 1 never delivers: 50 ms bound
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.045 <= waited < 0.6, waited
    assert int(lone.status.item()) == 1 and bool((lone.fused_out == 7.0).all())
    assert np.array_equal(decode_layer(q, layer, 2100).cpu().numpy(), plain)   # the context is fine


@pytest.mark.parametrize("kernel", ["exchange_merge", "wait_merge"])
def test_bounded_wait_runs_out_and_reports(kernel):
    """World of two, only rank 0 is ever launched: rank 1's flag stays unset, the wait gives up
    after the bound passed in, the status word reads 1 and the output is left alone."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from shard_b200 import _lib
    lib = _lib.load()
    bufs, ptrs = _exchange_buffers(2)
    part = torch.zeros(32, 132, dtype=torch.float32, device=DEV)
    part[:, 1] = 1.0
    out = torch.full((32, 128), 7.0, dtype=torch.float16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    limit_us = 20000
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    if kernel == "exchange_merge":
        rc = lib.shard_b200_seqsplit_merge(part.data_ptr(), ptrs, 0, 2, 8, 1, out.data_ptr(), status.data_ptr(),
                                           limit_us, _lib.cur_stream())
    else:
        rc = lib.shard_b200_seqsplit_wait_merge(ptrs, 0, 2, 8, 1, out.data_ptr(), status.data_ptr(), limit_us,
                                                _lib.cur_stream())
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert limit_us * 1e-6 * 0.9 <= waited < 0.5, waited      # gave up after the bound, well within half a second
    assert int(status.item()) == 1
    assert bool((out == 7.0).all())
    # the context is still usable and the same buffers work once both ranks deliver
    status.zero_()
    for r in (0, 1, 0):
        lib.shard_b200_seqsplit_merge(part.data_ptr(), ptrs, r, 2, 8, 2, out.data_ptr(), status.data_ptr(),
                                      limit_us, _lib.cur_stream())
    torch.cuda.synchronize()
    assert bool((out == 0.0).all())


def test_decode_status_word_is_reported_and_cleared():
    """`shard_b200_decode_status` reads the word at the head of a workspace and clears it."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from shard_b200 import _lib, ops
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    assert ops.decode_status(ws) == 0
    ws[:4].view(torch.int32).fill_(1)            # what a launch that gave up leaves behind
    assert ops.decode_status(ws) == 1
    assert ops.decode_status(ws) == 0
    ws[:4].view(torch.int32).fill_(1)
    with pytest.raises(_lib.ShardError, match="gave up"):
        ops.decode_status_check(ws)
