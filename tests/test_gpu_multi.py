"""Two-GPU test of the sequence-split decode: every rank attends to its slice of the compressed
middle, the per-head (max, sum-exp, acc) records travel through NCCL or through peer memory, and the merged result
equals single-GPU attention over the whole cache.  Skipped on boxes with fewer than 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import REPO

pytestmark = pytest.mark.gpu

_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
from gpu_helpers import FakeCache, FakeLayer, gc_to_device, random_gc, random_query
from oracle import shard_oracle as O
from conftest import tol_ok
from shard_b200.cache import attach_kernel_format
from shard_b200.parallel import PeerExchange, seqsplit_decode, shard_layer_tokens
from shard_b200.attention import decode_layer

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
gc_np = random_gc(5000, seed=3)
q_np = random_query(seed=4)
inv = torch.from_numpy(O.default_inv_freq())
full = FakeLayer(gc_to_device(gc_np, f"cuda:{rank}"), FakeCache(inv))
q = torch.from_numpy(q_np).to(f"cuda:{rank}").view(1, 32, 1, 128)
whole = decode_layer(q, full, 5100).clone()
sub = shard_layer_tokens(full._gpu_compressed, rank, world)
attach_kernel_format(sub, 8)
mine = FakeLayer(sub, FakeCache(inv))
out = seqsplit_decode(q, mine, 5100)
torch.cuda.synchronize()
got, ref = out.cpu().numpy()[0, :, 0, :], whole.cpu().numpy()
assert np.abs(got.astype(np.float32) - ref.astype(np.float32)).max() <= 2e-3
exact, *_ = O.attention_exact(q_np, gc_np, 5100, O.default_inv_freq())
assert tol_ok(got, exact, atol=1.5e-3, rtol=5e-3)
gathered = [None] * world
dist.all_gather_object(gathered, got.tobytes())
assert all(x == gathered[0] for x in gathered)      # bitwise identical on every rank
# the same exchange over NVLink peer memory inside the merge kernel: bit-identical to the NCCL path,
# also when the two buffer slots are reused over several steps
peer = PeerExchange(8)
for step in range(6):
    # odd steps: one launch per rank (the delivering CTAs wait and merge); even steps: the decode
    # launch delivers and a second, already polling launch merges
    timing = None if step % 2 else {"merge_start": torch.cuda.Event(), "merge_end": torch.cuda.Event()}
    out2 = seqsplit_decode(q, mine, 5100, peer=peer, timing=timing)
    torch.cuda.synchronize()
    peer.check()
    assert out2.cpu().numpy()[0, :, 0, :].tobytes() == got.tobytes(), step
# fewer tiles than ranks: rank 1's range is empty, it launches no decode and contributes the neutral record
tiny_np = random_gc(100, seed=8)
tiny_full = FakeLayer(gc_to_device(tiny_np, f"cuda:{rank}"), FakeCache(inv))
tiny_whole = decode_layer(q, tiny_full, 200).cpu().numpy()
tiny_sub = shard_layer_tokens(tiny_full._gpu_compressed, rank, world)
assert (tiny_sub["n_compress"] == 0) == (rank == 1)
if tiny_sub["n_compress"]:
    attach_kernel_format(tiny_sub, 8)
tiny = FakeLayer(tiny_sub, FakeCache(inv))
for p_ in (None, peer):
    o = seqsplit_decode(q, tiny, 200, peer=p_).cpu().numpy()[0, :, 0, :]
    assert np.abs(o.astype(np.float32) - tiny_whole.astype(np.float32)).max() <= 2e-3
peer.check()
peer.close()
dist.barrier()
# one process driving two GPUs: the kernel's shared-memory opt-in and the SM count are per device
other = 1 - rank
with torch.cuda.device(other):
    layer_o = FakeLayer(gc_to_device(gc_np, f"cuda:{other}"), FakeCache(inv))
    q_o = q.to(f"cuda:{other}")
    got_o = decode_layer(q_o, layer_o, 5100).cpu().numpy()
assert np.array_equal(got_o, ref)
try:
    decode_layer(q_o, full, 5100)            # tensors of two different devices in one call
    raise SystemExit("a tensor of another device was accepted")
except Exception as e:
    assert "cuda:" in str(e) and ("current device" in str(e) or "lives on" in str(e)), e
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
'''


def test_sequence_split_decode_over_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29700 + os.getpid() % 200),
               WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), REPO], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE) for r in range(2)]
    for p in procs:
        out, err = p.communicate(timeout=300)
        assert p.returncode == 0, err.decode()[-1500:]
