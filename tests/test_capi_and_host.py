"""CPU-only checks: the C-ABI library loads and exports what the header declares;
host-side partitioning logic; the multi-rank merge path over gloo."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import REPO, gc_from_golden, load_golden
from oracle import shard_oracle as O


def _declared_symbols():
    text = open(os.path.join(REPO, "include", "shard_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(shard_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from shard_b200 import _lib, build
    build.build()
    lib = _lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(_lib.symbols()) == declared
    assert lib.shard_b200_abi_version() == 3
    assert lib.shard_b200_status_string(-1).decode().startswith("invalid argument")


def test_struct_layouts_match_header():
    import ctypes as C
    from shard_b200 import _lib
    assert C.sizeof(_lib.ShardSeq) == 21 * 8
    assert C.sizeof(_lib.ShardDecodeShape) == 15 * 4


def test_argument_validation_without_gpu():
    """Rejected arguments return before any CUDA call, so this runs without a device."""
    import ctypes as C
    from shard_b200 import _lib, ops
    lib = _lib.load()
    sh = ops.make_shape(32, 8, 100, 1000, 0, 1000, 4, 64, 0, 1068)          # rank not a multiple of 32
    assert lib.shard_b200_decode_workspace_bytes(C.byref(sh), 1) == 0
    sh = ops.make_shape(32, 8, 192, 1000, 0, 1001, 4, 64, 0, 1068)          # range past the end
    assert lib.shard_b200_decode_workspace_bytes(C.byref(sh), 1) == 0
    sh = ops.make_shape(32, 8, 192, 32700, 0, 32700, 4, 64, 255, 33023)
    need = lib.shard_b200_decode_workspace_bytes(C.byref(sh), 1)
    assert 0 < need < (8 << 20)
    assert lib.shard_b200_wprep_bytes(8, 192) == 8 * 4 * 16384
    assert lib.shard_b200_wprep_bytes(8, 200) == 0
    seq = _lib.ShardSeq()
    assert lib.shard_b200_decode_attn(C.addressof(seq), 1, C.byref(sh), None, None, None, 0, None) == -1
    assert lib.shard_b200_k_quantize_pack(None, None, 10, 4, None, None, None, 0, None) == -1
    assert lib.shard_b200_k_project_workspace_bytes(1024, 192) == 16 + 32 * 2 * 192 * 128
    assert lib.shard_b200_k_project_workspace_bytes(1000, 192) == 0 and lib.shard_b200_k_project_workspace_bytes(1024, 194) == 0
    assert lib.shard_b200_k_project(None, None, None, 10, 1024, 64, None, None, 0, None) == -1
    assert lib.shard_b200_lse_merge(None, 2, 32, None, None) == -1
    # sequence-split exchange: buffer = flags (2 slots x world x nkv u32, rounded to 256 B) + 2 slots of records
    assert lib.shard_b200_peer_buffer_bytes(2, 8) == 256 + 2 * 2 * 32 * 132 * 4
    assert lib.shard_b200_peer_buffer_bytes(17, 8) == 0
    assert lib.shard_b200_seqsplit_merge(None, None, 0, 2, 8, 1, None, None, 0, None) == -1
    assert lib.shard_b200_seqsplit_wait_merge(None, 0, 2, 8, 1, None, None, 0, None) == -1
    sh1 = ops.make_shape(32, 8, 192, 1000, 0, 1000, 4, 64, 0, 1068, partial_out=False)
    bufs = (C.c_void_p * 2)(1, 1)
    assert lib.shard_b200_decode_attn_seqsplit(C.addressof(seq), C.byref(sh1), None, None, None, 0, bufs, 0, 2, 1,
                                               None, None, 0, None) == -1   # the record that travels is the partial one
    assert lib.shard_b200_decode_status(None, None, None) == -1
    assert lib.shard_b200_vq_assign_accumulate(None, None, 10, None, None, None, None) == -1
    assert lib.shard_b200_phase_table_bytes(33) == 64 * 256


def test_ops_refuse_cpu_tensors():
    from shard_b200 import _lib, ops
    with pytest.raises(_lib.ShardError):
        ops.vq_assign(torch.zeros(8, 4), torch.zeros(256, 4))
    with pytest.raises(_lib.ShardError):
        ops.undo_rope(torch.zeros(8, 4, 128, dtype=torch.float16), 0, torch.zeros(64))


def test_split_ranges_cover_and_align():
    from shard_b200.parallel import batch_shard, split_ranges
    for n in (0, 1, 15, 16, 17, 444, 1980, 32700, 131004):
        for w in (1, 2, 3, 4, 8):
            r = split_ranges(n, w)
            assert len(r) == w and r[0][0] == 0 and r[-1][1] == n
            for (a, b), (c, d) in zip(r[:-1], r[1:]):
                assert b == c and a <= b
            assert all(a % 128 == 0 for a, _ in r if a < n)
            sizes = [b - a for a, b in r]
            assert max(sizes) - min(sizes) <= 128 + 127
    for n in (1, 7, 64):
        for w in (1, 2, 4, 8):
            got = sum((batch_shard(n, r, w) for r in range(w)), [])
            assert got == list(range(n))


def test_host_tables_match_reference_fixtures():
    """The product's own host-side tables -- Lloyd-Max codebook, per-layer sign vectors, DP bit
    allocation -- against the values the reference produced (the kernels take them as inputs)."""
    import json
    from shard_b200.rope import dp_bit_allocation
    from shard_b200.streaming import lloyd_max_codebook, stream_signs
    g = load_golden("codebook.npz")
    cb = lloyd_max_codebook(128, 8)
    assert cb.dtype == torch.float32 and np.array_equal(cb.numpy(), g["codebook"])
    for li in range(4):
        assert np.array_equal(stream_signs(li, 128, "cpu").numpy(), g["signs"][li])
    with open(os.path.join(REPO, "tests", "golden", "dp_alloc.json")) as f:
        cases = json.load(f)
    assert len(cases) >= 3
    for c in cases:
        assert list(dp_bit_allocation(torch.tensor(c["eig"], dtype=torch.float32), c["budget"])) == c["alloc"]


def test_wrappers_refuse_tensors_of_another_device():
    """Launches go to the current device's stream with raw pointers: a tensor of another GPU is
    refused on the host (checked here with a stand-in tensor; no GPU needed)."""
    from shard_b200 import _lib

    class Dev:
        index = 1

    class T:
        is_cuda = True
        device = Dev()

    _lib.require_cuda(T(), None, current=1)
    with pytest.raises(_lib.ShardError, match="current device"):
        _lib.require_cuda(T(), current=0)


def test_empty_rank_contributes_neutral_record():
    """Fewer tiles than ranks: the idle ranks' record (max = -inf, sum-exp = 0) gets weight zero."""
    from shard_b200.parallel import neutral_partial, split_ranges
    r = split_ranges(200, 4)
    assert r == [(0, 128), (128, 200), (200, 200), (200, 200)]
    rng = np.random.default_rng(0)
    real = np.zeros((2, 32, 132), np.float32)
    real[:, :, 0] = rng.standard_normal((2, 32))
    real[:, :, 1] = 1 + rng.random((2, 32))
    real[:, :, 4:] = rng.standard_normal((2, 32, 128))
    idle = neutral_partial(32, "cpu").numpy()
    assert np.isneginf(idle[:, 0]).all() and not idle[:, 1:].any()
    parts = np.concatenate([real, idle[None], idle[None]])
    a = O.lse_merge(real[:, :, 0], real[:, :, 1], real[:, :, 4:])
    b = O.lse_merge(parts[:, :, 0], parts[:, :, 1], parts[:, :, 4:])
    assert np.array_equal(a, b)


def test_shard_layer_tokens_slices(golden_chain512):
    from shard_b200.parallel import shard_layer_tokens
    g = golden_chain512
    gc = {k: (torch.from_numpy(v) if isinstance(v, np.ndarray) else v) for k, v in gc_from_golden(g).items()}
    for k in ("sink_k", "sink_v", "win_k", "win_v"):
        gc[k] = gc[k].unsqueeze(0)
    n, keep = gc["k_coeffs_shape"]
    rows = gc["k_coeffs"].view(n, keep // 2)
    seen = 0
    for r in range(3):
        sub = shard_layer_tokens(gc, r, 3)
        b, e = sub["token_range"]
        assert sub["compress_start"] == gc["compress_start"] + b and sub["n_compress"] == e - b
        assert torch.equal(sub["k_coeffs"].view(e - b, keep // 2), rows[b:e])
        assert torch.equal(sub["v_indices_u8"], gc["v_indices_u8"][:, b:e])
        assert (sub["sink_k"].shape[2] > 0) == (r == 0)
        seen += e - b
    assert seen == n


_GLOO_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from conftest import gc_from_golden, load_golden
from oracle import shard_oracle as O
from shard_b200.parallel import all_gather_partials, split_ranges

dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}",
                        rank=int(sys.argv[3]), world_size=int(sys.argv[4]))
rank, world = dist.get_rank(), dist.get_world_size()
g = load_golden("chain512.npz")
gc = gc_from_golden(g)
inv_freq = O.default_inv_freq()
q = g["q"][0, :, 0, :]
b, e = split_ranges(gc["n_compress"], world)[rank]
_, m, l, acc = O.attention_exact(q, gc, 512, inv_freq, tok_range=(b, e), with_fp16_segments=False)
if rank == 0:   # rank 0 also owns sink + window: fold them in as a second local part
    gc0 = dict(gc); gc0["n_compress"] = 0
    _, m2, l2, acc2 = O.attention_exact(q, gc, 512, inv_freq, tok_range=(0, 0), with_fp16_segments=True)
    M = np.maximum(m, m2); w1, w2 = np.exp(m - M), np.exp(m2 - M)
    m, l, acc = M, w1 * l + w2 * l2, w1[:, None] * acc + w2[:, None] * acc2
part = np.zeros((32, 132), np.float32)
part[:, 0], part[:, 1], part[:, 4:] = m, l, acc
parts = all_gather_partials(torch.from_numpy(part)).numpy()
merged = O.lse_merge(parts[:, :, 0], parts[:, :, 1], parts[:, :, 4:])
whole, *_ = O.attention_exact(q, gc, 512, inv_freq)
assert np.allclose(merged, whole, atol=2e-5), np.abs(merged - whole).max()
gathered = [None] * world
dist.all_gather_object(gathered, merged.tobytes())
assert all(x == gathered[0] for x in gathered)          # bitwise identical on all ranks
dist.destroy_process_group()
print("ok", rank)
'''


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_split_merge_over_gloo(world, tmp_path):
    """World-size-N CPU ranks: each computes the oracle partial of its token range, the
    partials travel through the product's all-gather helper, and the log-sum-exp
    combine reproduces whole-sequence attention identically on every rank."""
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    port = 29500 + (os.getpid() % 2000) + world
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([REPO, os.path.join(REPO, "tests")]))
    procs = [subprocess.Popen([sys.executable, str(script), os.path.join(REPO, "tests"), str(port), str(r),
                               str(world)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
             for r in range(world)]
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0, err.decode()[-2000:]


def test_hf_glue_short_prompt_on_cpu():
    """Prompts too short to compress (<= sink + window + 4 tokens) run through the stock
    attention with our Cache acting as a plain KV store -- exercises the HF-facing glue
    (update / get_seq_length / get_mask_sizes) without a GPU."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from shard_b200 import Cache, enable_llama_fused_attention
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=1, head_dim=128, vocab_size=128, rope_theta=500000.0)
    model = LlamaForCausalLM(cfg).eval()
    assert enable_llama_fused_attention(model)
    ids = torch.randint(0, 128, (1, 20), generator=torch.Generator().manual_seed(1))
    cache = Cache.from_model(model)
    cache._streaming = True
    with torch.no_grad():
        out = model.generate(ids, max_new_tokens=6, do_sample=False, past_key_values=cache, pad_token_id=0)
        ref = model.generate(ids, max_new_tokens=6, do_sample=False, pad_token_id=0)
    assert torch.equal(out, ref)
    assert not cache._compressed and cache.get_seq_length() == 25
    assert cache.memory_bytes() == 2 * 2 * 25 * 128 * 4      # raw fp32 K and V of 2 layers
    assert torch.allclose(cache._rope_inv_freq, 1.0 / (500000.0 ** (torch.arange(0, 128, 2).float() / 128)))
