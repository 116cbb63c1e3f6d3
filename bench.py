"""Benchmark of the compressed-KV decode attention path (BASELINE.json metric).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-triton]
                    [--workload cfg1|cfg2|cfg3|cfg4] [--merge peer|nccl] [--ctx T] [--layers L]

A *step* is one decode step: every layer appends one new (K, V) token to its
8-bit stream and attends with one query token over
[sink | compressed middle | window | stream].  Default workload (cfg2): one
32768-token sequence on the Llama-3.1-8B geometry, 32 layers, synthetic K/V
(rank-192 keys before RoPE, outlier-channel values), compressed by this
package's own prefill compressor before the timed region.

Metric: microseconds per sequence-layer-step (at one GPU and one sequence this is
"us/step/layer").  With N > 1 GPUs each rank owns its own sequences (batch
sharding, no data-path communication); the value is the aggregate
ms_per_step / (layers * total sequences), time is the max over ranks.  In the same
run the N > 1 line also carries `seqsplit` (one 131072-token sequence split by token
range over the N GPUs, records exchanged over NVLink, with a parity check against
unsplit decode that fails the run on a mismatch) and `batch64` (64 x 8K sequences
sharded by batch).

One JSON line is printed by rank 0.  `--impl reference` times the reference's own
CPU implementation (its unmodified Python package, run from oracle/_ref when
oracle/make_ref.py has put it there; otherwise the numpy port of it, saying so) on the
host cores.  `--impl reference-triton` times the reference's Triton path on the GPU,
for context only.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(1, os.path.join(HERE, "tests"))          # synth.py: the seeded synthetic K/V generator

N_Q, N_KV, HD, RANK, SINK, WIN = 32, 8, 128, 192, 4, 64
METRIC = "compressed_kv_decode_attn_us_per_step_per_layer"
TRAFFIC_SUMMARY = os.path.join("profiles", "decode_partial_pipe_kernel_cfg2_full.md")


def algorithmic_bytes(n_comp, n_stream, rank=RANK, n_sink=SINK, n_win=WIN):
    """Bytes one layer-step must touch, every operand counted once: packed int4
    coefficients + VQ codes per middle token, fp16 basis, mean, scales, codebook,
    fp16 sink/window K and V, stream codes + norms, query in, output out."""
    per_tok = rank // 2 + N_KV * 32
    fixed = 2 * rank * N_KV * HD + 2 * N_KV * HD + 2 * rank + 256 * 4 * 2 + 2 * N_KV * HD
    fixed += (n_sink + n_win) * N_KV * HD * 2 * 2 + N_Q * HD * 2 * 2
    return n_comp * per_tok + fixed + n_stream * (2 * N_KV * HD + 2 * 2 * N_KV)


def algorithmic_flops(n_comp):
    """K reconstruction [n x 192] . [192 x 1024] plus scores and P.V of the middle segment."""
    return 2 * n_comp * RANK * N_KV * HD + 4 * N_Q * HD * n_comp


def workload_string(T, L, seqs_per_gpu):
    """One description of the headline workload, used by both arms."""
    return (f"cfg2: Llama-3.1-8B geometry ({N_Q}/{N_KV} heads, head_dim {HD}), {T}-token context, {L} layers, "
            f"{seqs_per_gpu} sequence(s) per GPU, one query token per step, 8-bit stream growing by one token per step")


def measured_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of one decode launch on the cfg2 geometry, read
    from the committed ncu summary (a line `dram_bytes_per_launch = N`); (None, None) if absent."""
    try:
        text = open(os.path.join(HERE, TRAFFIC_SUMMARY)).read()
        m = re.search(r"dram_bytes_per_launch\s*=\s*(\d+)", text)
        return (int(m.group(1)), TRAFFIC_SUMMARY) if m else (None, None)
    except OSError:
        return None, None


def measured_peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, bf16 TFLOP/s sustained, kind)."""
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        burst = float(d.get("bf16_tflops", 0))
        return float(d["hbm_gbs"]), burst, float(d.get("bf16_tflops_sustained", burst)), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while running."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), parts[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm))
        return out


# ----------------------------------------------------------------------------- reference arm / CPU baseline
def reference_path():
    from oracle.make_ref import ref_path
    return ref_path()


def reference_layer_with_random_codes(n_comp, dev, seed=0):
    """One layer of the REFERENCE's own `Cache` (imported from oracle/_ref) whose per-layer dictionary
    is built by hand with random codes, as the reference's own kernel test does
    (benchmarks/kernel_test.py:206-221); decode cost does not depend on code values."""
    import torch
    from shard.cache import Cache as RefCache
    g = torch.Generator().manual_seed(seed)
    p = N_KV * HD
    inv = 1.0 / (500000.0 ** (torch.arange(0, HD, 2, dtype=torch.float32) / HD))
    cache = RefCache(num_layers=1, device=str(dev), rope_inv_freq=inv)
    cache._streaming = True
    basis_q = torch.randint(-127, 128, (p, RANK), generator=g, dtype=torch.int8)
    bscale = (0.08 / 127 * (0.5 + torch.rand(RANK, generator=g))).half()
    idx = torch.randint(0, 256, (N_KV * n_comp * 32,), generator=g, dtype=torch.uint8)
    cent = (torch.randn(256, 4, generator=g) * 0.4).half()
    ch = (0.5 + 3 * torch.rand(N_KV, HD, generator=g)).half()
    gc = {
        "k_coeffs": torch.randint(0, 256, (n_comp * RANK // 2,), generator=g, dtype=torch.uint8),
        "k_coeffs_shape": (n_comp, RANK),
        "k_coeff_scale": (torch.exp(-0.01 * torch.arange(RANK)) * 0.4).half(),
        "k_basis_q": basis_q, "k_basis_scale": bscale, "k_basis_f16": basis_q.half() * bscale,
        "k_mean": (torch.randn(p, generator=g) * 0.1).half(),
        "v_qdata": {"centroids": cent, "packed": idx, "ch_maxabs": ch, "shape": (N_KV, n_comp, HD),
                    "group_size": 4, "bits": 8, "n_orig": idx.numel()},
        "v_indices_u8": idx.view(N_KV, n_comp, 32), "v_centroids_f16": cent, "v_ch_f16": ch,
        "sink_k": torch.randn(1, N_KV, SINK, HD, generator=g).half(),
        "sink_v": torch.randn(1, N_KV, SINK, HD, generator=g).half(),
        "win_k": torch.randn(1, N_KV, WIN, HD, generator=g).half(),
        "win_v": torch.randn(1, N_KV, WIN, HD, generator=g).half(),
        "n_compress": n_comp, "batch": 1, "compress_start": SINK,
    }
    gc["k_mean_f16"] = gc["k_mean"]
    move = lambda d: {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in d.items()}  # noqa: E731
    gc = move(gc)
    gc["v_qdata"] = move(gc["v_qdata"])
    layer = cache.layers[0]
    layer._gpu_compressed = gc
    return layer, inv


def time_reference_layer_steps(n_comp, repeats, warmup, dev="cpu"):
    """Seconds per layer-step of the reference's own decode path -- `CacheLayer._stream_append` +
    `fused_attention_compressed`, unmodified, imported from oracle/_ref -- on `dev`."""
    import torch
    ref = reference_path()
    if ref is None:
        raise RuntimeError("oracle/_ref is absent")
    if ref not in sys.path:
        sys.path.insert(0, ref)
    from shard.attention import fused_attention_compressed as ref_attn
    is_cuda = str(dev).startswith("cuda")
    if not is_cuda:
        torch.set_num_threads(os.cpu_count() or 1)       # do not inherit OMP_NUM_THREADS=1 from a launcher
    layer, inv = reference_layer_with_random_codes(n_comp, dev)
    g = torch.Generator().manual_seed(1)
    pos0 = SINK + n_comp + WIN
    times = []
    for it in range(warmup + repeats):
        q = torch.randn(1, N_Q, 1, HD, generator=g).half().to(dev)
        k = torch.randn(1, N_KV, 1, HD, generator=g).half().to(dev)
        v = torch.randn(1, N_KV, 1, HD, generator=g).half().to(dev)
        if is_cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        layer._stream_append(k, v, pos0 + it)
        out = ref_attn(q, layer, pos0 + it, inv, None)
        if is_cuda:
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert out.shape == (1, N_Q, 1, HD)
        if it >= warmup:
            times.append(dt)
    return sum(times) / len(times), (torch.get_num_threads() if not is_cuda else 0)


def synthetic_compressed_layer_numpy(n_comp, seed=0):
    """A compressed layer with random codes for the numpy port."""
    import numpy as np
    rng = np.random.default_rng(seed)
    p = N_KV * HD
    nib = rng.integers(1, 16, size=(n_comp, RANK), dtype=np.uint8)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8).reshape(-1)
    basis_q = rng.integers(-127, 128, size=(p, RANK)).astype(np.int8)
    basis_scale = (0.08 / 127 * (0.5 + rng.random(RANK))).astype(np.float16)
    mean = (rng.standard_normal(p) * 0.1).astype(np.float16)
    return {
        "k_coeffs": packed, "k_coeffs_shape": (n_comp, RANK),
        "k_coeff_scale": (np.exp(-0.01 * np.arange(RANK)) * 0.4).astype(np.float16),
        "k_basis_q": basis_q, "k_basis_scale": basis_scale,
        "k_basis_f16": (basis_q.astype(np.float16) * basis_scale).astype(np.float16),
        "k_mean": mean, "k_mean_f16": mean,
        "v_indices_u8": rng.integers(0, 256, size=(N_KV, n_comp, 32)).astype(np.uint8),
        "v_centroids_f16": (rng.standard_normal((256, 4)) * 0.4).astype(np.float16),
        "v_ch_f16": (0.5 + rng.random((N_KV, HD)) * 3).astype(np.float16),
        "sink_k": rng.standard_normal((N_KV, SINK, HD)).astype(np.float16),
        "sink_v": rng.standard_normal((N_KV, SINK, HD)).astype(np.float16),
        "win_k": rng.standard_normal((N_KV, WIN, HD)).astype(np.float16),
        "win_v": rng.standard_normal((N_KV, WIN, HD)).astype(np.float16),
        "n_compress": n_comp, "batch": 1, "compress_start": SINK,
    }


def time_cpu_port(n_comp, repeats, warmup, n_stream=8):
    """Seconds per layer-step of the numpy port of the reference's decode (used only when
    oracle/_ref is absent), including the stream append."""
    import numpy as np
    from oracle import shard_oracle as O
    gc = synthetic_compressed_layer_numpy(n_comp)
    inv = O.default_inv_freq()
    cb = O.lloyd_max_codebook(HD, 8)
    signs = O.stream_signs(0)
    rng = np.random.default_rng(1)
    sk = rng.standard_normal((n_stream, N_KV, HD)).astype(np.float16)
    sv = rng.standard_normal((n_stream, N_KV, HD)).astype(np.float16)
    ki, kn, vi, vn = O.stream_quantize(sk, sv, signs, cb)
    times = []
    for it in range(warmup + repeats):
        q = rng.standard_normal((N_Q, HD)).astype(np.float16)
        nk = rng.standard_normal((1, N_KV, HD)).astype(np.float16)
        nv = rng.standard_normal((1, N_KV, HD)).astype(np.float16)
        t0 = time.perf_counter()
        a, b, c, d = O.stream_quantize(nk, nv, signs, cb)
        stream = dict(k_idx=np.concatenate([ki, a]), v_idx=np.concatenate([vi, c]),
                      k_norm=np.concatenate([kn, b]), v_norm=np.concatenate([vn, d]),
                      signs=signs, codebook=cb)
        O.fused_attention_compressed(q, gc, SINK + n_comp + WIN + n_stream, inv, stream=stream)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    return sum(times) / len(times), os.cpu_count() or 1


def cpu_baseline(n_comp, repeats, warmup, n_sample=None):
    """(seconds per layer-step scaled to n_comp tokens, cores, kind, what was sampled)."""
    n_sample = n_comp if n_sample is None else n_sample
    if reference_path() is not None:
        sec, cores = time_reference_layer_steps(n_sample, repeats, warmup)
        kind, what = "reference", ("the reference's own fused_attention_compressed + _stream_append "
                                   "(unmodified package from oracle/_ref), CPU fp16 tensors, hand-built "
                                   "per-layer dictionary with random codes")
    else:
        sec, cores = time_cpu_port(n_sample, repeats, warmup)
        kind, what = "port", "numpy port of the reference's CPU path (oracle/_ref is absent), random codes"
    scale = n_comp / n_sample
    sample = (f"{repeats} timed layer-steps ({warmup} warm-up) of ONE layer; "
              + (f"whole middle segment, n_comp={n_comp}" if n_sample == n_comp else
                 f"{n_sample} of the {n_comp} middle tokens per step, time scaled by {scale:.2f}")
              + f"; {what}")
    return sec * scale, cores, kind, sample, sec


def run_reference(args):
    """The reference arm: the reference's own CPU implementation of one layer-step on all host
    cores.  A timed step is ONE layer-step (a bounded sample of the 32-layer decode step); with
    many steps a step attends to a contiguous share of the middle tokens (cost is linear in the
    tokens) so that the run ends within about two minutes.  `value` is the time of a whole
    layer-step; `ms_per_step` is what a timed step really took."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.ctx
    n_comp = T - SINK - WIN
    K = max(1, args.steps)
    W = max(1, min(args.warmup, 2))
    budget_s, est_full_s = 120.0, 0.6 * n_comp / 32700.0
    n_sample = n_comp if (K + W) * est_full_s <= budget_s else max(1024, int(n_comp * budget_s / ((K + W) * est_full_s)))
    sec, cores, kind, sample, sec_sample = cpu_baseline(n_comp, K, W, n_sample)
    us = sec * 1e6
    line = {
        "impl": "reference", "metric": METRIC, "value": us, "unit": "us", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec_sample * 1e3,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": workload_string(T, args.layers, args.seqs),
                   "sampled_as": "one layer-step per timed step; value = microseconds per sequence-layer-step "
                                 "on the host cores (it does not depend on the number of GPUs)"},
        "cpu_baseline": {"value": us, "unit": "us", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference_triton(args):
    """Context only: the reference's GPU path (its Triton kernels + eager PyTorch, unmodified, from
    oracle/_ref) on this GPU, microseconds per layer-step at 32K and 8K."""
    import torch
    res = {"impl": "reference-triton", "unit": "us per layer-step"}
    try:
        if reference_path() is None:
            raise RuntimeError("oracle/_ref is absent")
        torch.cuda.set_device(0)
        for T in (8192, 32768):
            sec, _ = time_reference_layer_steps(T - SINK - WIN, 20, 5, dev="cuda:0")
            res[f"ctx_{T}"] = sec * 1e6
        import shard.triton_kernels as tk
        res["triton"] = bool(tk.HAS_TRITON)
    except Exception as e:                                    # reported, never fatal: context only
        res["unavailable"] = f"{type(e).__name__}: {e}"[:300]
    print(json.dumps(res), flush=True)


# ----------------------------------------------------------------------------- our arm
def build_cache(T, layers, seed0, dev):
    import torch
    import synth
    from shard_b200 import Cache
    cache = Cache(num_layers=layers, rope_inv_freq=synth.rope_inv_freq())
    cache._streaming = True
    for li in range(layers):
        k, v, _ = synth.make_kvq(T, seed0 + li, device=dev)
        cache.layers[li].update(k, v)
    cache.compress()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return cache


class _Dist:
    """Rank bookkeeping + barrier shared by the workloads."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1 and not dist.is_initialized():
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        import torch
        import torch.distributed as dist
        t = torch.tensor(values, device=self.dev, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def close(self):
        import torch.distributed as dist
        if self.world > 1 and dist.is_initialized():
            dist.destroy_process_group()


def time_batched(D, caches, T, L, K, W, sampler=None):
    """Device-resident timing of K decode steps of `caches` (one launch per layer for all local
    sequences); returns (ms_total max over ranks, streamed rows at the end, decoder)."""
    import torch
    from shard_b200.parallel import BatchedDecoder
    S = len(caches)
    bd = BatchedDecoder(caches, stream_capacity=2 * (K + W) + 8)
    total = K + W
    g = torch.Generator(device=D.dev).manual_seed(1234 + D.rank)
    q_pool = torch.randn(total, L, S, N_Q, HD, generator=g, device=D.dev).half()
    k_pool = torch.randn(total, L, S, N_KV, HD, generator=g, device=D.dev).half()
    v_pool = torch.randn(total, L, S, N_KV, HD, generator=g, device=D.dev).half()

    def one_step(j):
        bd.q.copy_(q_pool[j])
        bd.new_k.copy_(k_pool[j])
        bd.new_v.copy_(v_pool[j])
        bd.step(T + j)

    for j in range(W):
        one_step(j)
    D.barrier()
    if sampler is not None:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    D.barrier()
    ev0.record()
    for j in range(W, W + K):
        one_step(j)
    ev1.record()
    D.barrier()
    bd.check()                                    # no launch gave up on a bounded wait
    (ms_total,) = D.max_over_ranks([ev0.elapsed_time(ev1)])
    return ms_total, bd.n_stream, bd


def measure_batch64(D, L, K, W):
    """BASELINE configs[3]: 64 independent 8192-token sequences sharded by batch over the ranks."""
    import torch
    import synth
    T, total_seqs = 8192, 64
    if total_seqs % D.world:
        return {"skipped": f"{D.world} GPUs do not divide 64 sequences"}
    S = total_seqs // D.world
    n_comp = T - SINK - WIN
    caches = [synth.random_cache(n_comp, L, D.dev, 5000 + 100 * (D.rank * S + s)) for s in range(S)]
    ms_total, s_now, bd = time_batched(D, caches, T, L, K, W)
    ms_per_step = ms_total / K
    bytes_step = algorithmic_bytes(n_comp, W + K // 2) * L * S
    del bd, caches
    torch.cuda.empty_cache()
    return {"workload": f"cfg3: 64 sequences x {T} tokens, {L} layers, {S} per GPU (random codes), one launch per "
                        "layer for all local sequences, no communication",
            "steps": K, "ms_per_step": ms_per_step, "tokens_per_s": total_seqs / (ms_per_step * 1e-3),
            "us_per_sequence_layer": ms_per_step * 1e3 / (L * total_seqs),
            "hbm_gbs_per_gpu": bytes_step / (ms_per_step * 1e-3) / 1e9}


def seqsplit_parity(D, peer):
    """Merged output of a 5000-token layer split over the ranks vs the same GPU decoding the whole
    (unsplit) layer, through the peer-memory path and the NCCL path; identical bytes on all ranks.
    Returns (max abs difference, bitwise equal across ranks and paths)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import synth
    from gpu_helpers import FakeCache, FakeLayer
    from shard_b200.attention import decode_layer
    from shard_b200.cache import attach_kernel_format
    from shard_b200.parallel import seqsplit_decode, shard_layer_tokens
    inv = synth.rope_inv_freq()
    full_gc = synth.random_compressed_layer(5000, D.dev, 4242, gen_device="cpu")
    full = FakeLayer(full_gc, FakeCache(inv))
    q = torch.randn(1, N_Q, 1, HD, generator=torch.Generator().manual_seed(99)).half().to(D.dev)
    whole = decode_layer(q, full, 5100).float().cpu().numpy()
    sub = shard_layer_tokens(full_gc, D.rank, D.world)
    if sub["n_compress"]:
        attach_kernel_format(sub, N_KV)
    mine = FakeLayer(sub, FakeCache(inv))
    outs = []
    for p_ in ([peer] if peer is not None else []) + [None]:
        if D.world == 1 and p_ is None:
            part = decode_layer(q, mine, 5100, partial_out=True)
            from shard_b200 import ops
            o = ops.lse_merge(part.unsqueeze(0))
        else:
            o = seqsplit_decode(q, mine, 5100, peer=p_)
        outs.append(o.reshape(N_Q, HD).cpu().numpy())
    torch.cuda.synchronize()
    max_abs = max(float(np.abs(o.astype(np.float32) - whole).max()) for o in outs)
    blobs = [o.tobytes() for o in outs]
    same = all(b == blobs[0] for b in blobs)
    if D.world > 1:
        gathered = [None] * D.world
        dist.all_gather_object(gathered, blobs[0])
        same = same and all(x == gathered[0] for x in gathered)
    return max_abs, same


def measure_seqsplit(D, L, K, W, T=131072, merge="peer", with_n1=True):
    """BASELINE configs[4]: one T-token sequence, the compressed middle cut into contiguous token
    ranges (one per GPU).  Every rank decodes its range; with `merge="peer"` the decode launch
    itself delivers the per-head (max, sum-exp, acc) record into every rank's exchange buffer over
    NVLink and a polling kernel merges; with "nccl" the records are all-gathered and merged by a
    separate launch.  Rank 0 also owns sink, window and stream."""
    import torch
    import torch.distributed as dist
    import synth
    from shard_b200 import ops
    from shard_b200.attention import decode_layer
    from shard_b200.parallel import PeerExchange, seqsplit_decode, split_ranges

    n_comp = T - SINK - WIN
    begin, end = split_ranges(n_comp, D.world)[D.rank]
    first = D.rank == 0
    cache = synth.random_cache(end - begin, L, D.dev, 9000, compress_start=SINK + begin,
                               n_sink=SINK if first else 0, n_win=WIN if first else 0)
    total = K + W
    g = torch.Generator(device=D.dev).manual_seed(77)          # same queries on every rank
    q_pool = torch.randn(total, L, 1, N_Q, 1, HD, generator=g, device=D.dev).half()
    k_pool = torch.randn(total, L, 1, N_KV, 1, HD, generator=g, device=D.dev).half()
    v_pool = torch.randn(total, L, 1, N_KV, 1, HD, generator=g, device=D.dev).half()
    parts = torch.empty(D.world, N_Q, 132, dtype=torch.float32, device=D.dev)
    part = torch.empty(N_Q, 132, dtype=torch.float32, device=D.dev)
    out = torch.empty(L, N_Q, HD, dtype=torch.float16, device=D.dev)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K * L)]
    peer = PeerExchange(N_KV) if (D.world > 1 and merge in ("peer", "both")) else None

    def step(j, events, use_peer):
        pos = T + j
        cache._fused_decode_update = True
        for li in range(L):
            layer = cache.layers[li]
            if first:
                layer.update(k_pool[j, li], v_pool[j, li])           # stream append (rank 0 owns the stream)
            e = ev[(j - W) * L + li] if events else None
            if e: e[0].record()
            if use_peer and not events:
                peer.decode_merge(q_pool[j, li], layer, pos, out[li], with_fp16_segments=first)   # one launch
            elif use_peer:
                decode_layer(q_pool[j, li], layer, pos, partial_out=True, with_fp16_segments=first, push=peer)
                e[1].record()
                peer.wait_merge(out[li])
            else:
                decode_layer(q_pool[j, li], layer, pos, partial_out=True, with_fp16_segments=first, out=part)
                if e: e[1].record()
                if D.world > 1:
                    dist.all_gather_into_tensor(parts.view(-1), part.view(-1))
                else:
                    parts[0].copy_(part)
                ops.lse_merge(parts, out=out[li])
            if e: e[2].record()
        cache._fused_decode_update = False

    def timed_run(use_peer, steps, events):
        """ms per step (max over ranks) of `steps` decode steps; with `events` also the decode / merge
        split per step from CUDA events around every launch (an event record between two launches
        keeps the second from starting early behind the first, so the split is taken in a pass of
        its own and the headline number in a pass without events)."""
        for j in range(W):
            step(j, False, use_peer)
        D.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        D.barrier()
        ev0.record()
        for j in range(W, W + steps):
            step(j, events, use_peer)
        ev1.record()
        D.barrier()
        ms_total = ev0.elapsed_time(ev1)
        dec_ms = mrg_ms = 0.0
        if events:
            used = ev[: steps * L]
            dec_ms = sum(e[0].elapsed_time(e[1]) for e in used) / steps
            mrg_ms = sum(e[1].elapsed_time(e[2]) for e in used) / steps
        return D.max_over_ranks([ms_total / steps, dec_ms, mrg_ms])

    res = {"workload": f"cfg4: one {T}-token sequence, {L} layers, compressed middle split into {D.world} contiguous "
                       "token range(s) (random codes); rank 0 also owns sink, window and stream", "steps": K}
    kb = min(K, 8)
    ms_step, _, _ = timed_run(peer is not None, K, False)
    ms_b, dec_ms, mrg_ms = timed_run(peer is not None, kb, True)
    res.update(us_per_layer=ms_step * 1e3 / L,
               breakdown={"steps": kb, "us_per_layer": ms_b * 1e3 / L, "decode_us_per_layer": dec_ms * 1e3 / L,
                          "merge_us_per_layer": mrg_ms * 1e3 / L,
                          "note": "pass with CUDA events around every launch (no launch overlap)"},
               decode_us_per_layer=dec_ms * 1e3 / L, merge_us_per_layer=mrg_ms * 1e3 / L,
               merge="one launch per rank: the decode launch delivers its record over NVLink peer memory, waits for "
                     "the others' and merges (the breakdown pass uses a second, polling launch for the merge)"
               if peer is not None
               else ("NCCL all-gather + merge launch" if D.world > 1 else "single GPU: merge launch only"))
    if D.world > 1 and merge == "both":
        # the NCCL path beside it (the stream keeps growing meanwhile: well under 1 us per layer on rank 0)
        k2 = min(K, 16)
        ms2, _, _ = timed_run(False, k2, False)
        _, dec2, mrg2 = timed_run(False, kb, True)
        res["nccl"] = {"us_per_layer": ms2 * 1e3 / L, "decode_us_per_layer": dec2 * 1e3 / L,
                       "merge_us_per_layer": mrg2 * 1e3 / L, "steps": k2}
    n_local = end - begin
    bytes_ls = algorithmic_bytes(n_local, W + K // 2)
    res["hbm_gbs_per_gpu"] = bytes_ls / (res["us_per_layer"] * 1e-6) / 1e9
    res["tokens_per_rank"] = n_local
    max_abs, same = seqsplit_parity(D, peer)
    res["parity_max_abs"], res["bitwise_equal_across_ranks"] = max_abs, bool(same)
    cache.check()
    if peer is not None:
        peer.check()
        peer.close()
    del cache
    torch.cuda.empty_cache()
    if with_n1 and D.world > 1:
        # the same sequence on ONE GPU (rank 0 alone; the others wait), for the speed-up
        t1 = [0.0]
        if first:
            whole = synth.random_cache(n_comp, L, D.dev, 9000)
            k1 = min(K, 8)
            for rep in range(2):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for j in range(k1):
                    whole._fused_decode_update = True
                    for li in range(L):
                        whole.layers[li].update(k_pool[j, li], v_pool[j, li])
                        decode_layer(q_pool[j, li], whole.layers[li], T + j, out=out[li])
                    whole._fused_decode_update = False
                e1.record()
                torch.cuda.synchronize()
                t1 = [e0.elapsed_time(e1) / k1]
            del whole
            torch.cuda.empty_cache()
        (ms1,) = D.max_over_ranks(t1)
        res["n1_us_per_layer"] = ms1 * 1e3 / L
        res["speedup_vs_n1"] = ms1 / ms_step
    return res


def run_ours(args):
    import torch
    from shard_b200 import fused_attention_compressed

    D = _Dist()
    world, rank, dev = D.world, D.rank, D.dev
    T, L = args.ctx, args.layers
    K, W = args.steps, max(args.warmup, 3)
    seqs_per_gpu = args.seqs
    n_comp = T - SINK - WIN

    t0 = time.perf_counter()
    caches = [build_cache(T, L, 100 + 1000 * (rank * seqs_per_gpu + s), dev) for s in range(seqs_per_gpu)]
    compress_s = sum(c.compress_seconds for c in caches) / len(caches)
    ratio = caches[0].clean_compress_ratio()
    build_s = time.perf_counter() - t0

    # ---- device-resident timing -------------------------------------------------
    sampler = ClockSampler(D.local) if rank == 0 else None
    ms_total, s_now, bd = time_batched(D, caches, T, L, K, W, sampler)
    # dominant kernel: the timed region is K * L launches of the decode kernel plus K launches of the
    # ~5 us phase-table kernel, back to back on one stream, so the decode kernel's average launch
    # duration is the region's event time over K * L (the phase table adds 1/L of its time to each)
    kern_ms = ms_total / (K * L)
    clocks = sampler.stop() if rank == 0 else None
    del bd

    # ---- end to end through the public API, host buffers ----------------------------
    e2e_steps = min(K, 64)
    cache = caches[0]
    hq = torch.randn(L, 1, N_Q, 1, HD).half().pin_memory()
    hk = torch.randn(L, 1, N_KV, 1, HD).half().pin_memory()
    hv = torch.randn(L, 1, N_KV, 1, HD).half().pin_memory()
    hout = torch.empty(L, 1, N_Q, 1, HD, dtype=torch.float16).pin_memory()
    dq = torch.empty_like(hq, device=dev)
    dk = torch.empty_like(hk, device=dev)
    dv = torch.empty_like(hv, device=dev)
    dout = torch.empty_like(hout, device=dev)
    inv = cache._rope_inv_freq

    def e2e_step(pos):
        for c in caches:
            dq.copy_(hq, non_blocking=True)
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
            c._fused_decode_update = True
            for li in range(L):
                layer = c.layers[li]
                layer.update(dk[li], dv[li])
                fused_attention_compressed(dq[li], layer, pos, inv, None, out=dout[li])
            c._fused_decode_update = False
            hout.copy_(dout, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    pos = cache.layers[0].get_seq_length()
    for j in range(3):
        e2e_step(pos + j)
    D.barrier()
    t0 = time.perf_counter()
    for j in range(e2e_steps):
        e2e_step(pos + 3 + j)
    D.barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    for c in caches:
        c.check()

    ms_total, e2e_ms, kern_ms = D.max_over_ranks([ms_total, e2e_ms, kern_ms])
    ms_per_step = ms_total / K
    n_seq_total = seqs_per_gpu * world
    us = ms_per_step * 1e3 / (L * n_seq_total)

    # ---- the two sharded BASELINE configs ride along when there is more than one GPU ----------
    extra = {}
    if world > 1 and args.multi_extras:
        del caches, cache
        torch.cuda.empty_cache()
        extra["seqsplit"] = measure_seqsplit(D, L, min(K, 32), 3, merge="both")
        extra["batch64"] = measure_batch64(D, L, min(K, 16), 3)

    if rank == 0:
        hbm_peak, tf_burst, tf_sustained, peak_kind = measured_peaks()
        s_mid = W + K // 2
        bytes_ls = algorithmic_bytes(n_comp, s_mid)
        flops_ls = algorithmic_flops(n_comp)
        kern_bytes = algorithmic_bytes(n_comp, s_now) * seqs_per_gpu
        kern_flops = flops_ls * seqs_per_gpu
        achieved = kern_bytes / (kern_ms * 1e-3) / 1e9
        tf = kern_flops / (kern_ms * 1e-3) / 1e12
        traffic, traffic_src = measured_traffic() if (T == 32768 and seqs_per_gpu == 1) else (None, None)
        line = {
            "metric": METRIC, "value": us, "unit": "us", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {
                "workload": workload_string(T, L, seqs_per_gpu),
                "stream": f"8-bit stream grows {W}->{W + K} tokens",
                "l2": "inputs larger than L2: one step touches %.0f MB of cache per GPU"
                      % (bytes_ls * L * seqs_per_gpu / 1e6),
                "parallelism": "batch-sharded, no communication" if world > 1 else "single GPU",
            },
            "hbm_gbs_per_gpu": bytes_ls * L * seqs_per_gpu / (ms_per_step * 1e-3) / 1e9,
            "hbm_frac_of_8TBs": bytes_ls * L * seqs_per_gpu / (ms_per_step * 1e-3) / 8e12,
            "tensor_tflops_per_gpu": flops_ls * L * seqs_per_gpu / (ms_per_step * 1e-3) / 1e12,
            "decode_tokens_per_s": n_seq_total / (ms_per_step * 1e-3),
            "prefill_compress_s_per_sequence": compress_s, "setup_s": build_s,
            "clean_compress_ratio": ratio,
            # 31 FLOP per byte of cache touched: the reconstruction GEMM, not HBM, bounds this path
            "roofline": {"kernel": "decode_partial_pipe_kernel (one decode_attn call: append + split-KV pass + combine)",
                         "bound": "tensor", "achieved": tf, "peak": tf_burst, "unit": "TFLOP/s",
                         "frac": tf / tf_burst,
                         "peak_kind": peak_kind + " (cuBLAS bf16 burst; the timed region runs at full clocks "
                                                  "without a power cap)",
                         "frac_of_sustained": tf / tf_sustained, "peak_sustained": tf_sustained,
                         "traffic": traffic, "traffic_source": traffic_src,
                         "us_per_launch": kern_ms * 1e3,
                         "algorithmic_flops_per_launch": kern_flops, "algorithmic_bytes_per_launch": kern_bytes,
                         "hbm_achieved_gbs": achieved, "hbm_peak_gbs": hbm_peak, "hbm_frac": achieved / hbm_peak},
            "e2e": {"value": e2e_ms * 1e3 / (L * n_seq_total), "unit": "us",
                    "h2d_bytes_per_step": seqs_per_gpu * L * (N_Q + 2 * N_KV) * HD * 2,
                    "d2h_bytes_per_step": seqs_per_gpu * L * N_Q * HD * 2,
                    "ms_per_step": e2e_ms, "api": "Cache.layers[i].update + fused_attention_compressed"},
            "gpu_launches": K * (1 + L),
            "clocks": clocks,
        }
        line.update(extra)
        if args.cpu_baseline:
            sec, cores, kind, sample, _ = cpu_baseline(n_comp, 8, 2)
            line["cpu_baseline"] = {"value": sec * 1e6, "unit": "us", "cores": cores, "kind": kind, "sample": sample}
        if args.reference_triton and world == 1:
            try:
                r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-triton"],
                                   capture_output=True, text=True, timeout=600)
                line["reference_triton"] = json.loads(r.stdout.strip().splitlines()[-1])
            except Exception as e:
                line["reference_triton"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        print(json.dumps(line), flush=True)
    bad = None
    if "seqsplit" in extra:
        sp = extra["seqsplit"]
        if not (sp["parity_max_abs"] <= 2e-3 and sp["bitwise_equal_across_ranks"]):
            bad = f"sequence-split parity check failed: {sp['parity_max_abs']}, {sp['bitwise_equal_across_ranks']}"
    D.close()
    if bad:
        raise SystemExit(bad)


def run_batch64(args):
    D = _Dist()
    res = measure_batch64(D, args.layers, args.steps, max(args.warmup, 3))
    if D.rank == 0:
        line = {"metric": METRIC, "value": res.get("us_per_sequence_layer"), "unit": "us", "n_gpus": D.world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": res.get("ms_per_step"),
                "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic", "config": {"workload": res.get("workload")}, "batch64": res,
                "e2e": {"value": None, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": args.steps * (1 + args.layers)}
        print(json.dumps(line), flush=True)
    D.close()


def run_seqsplit(args):
    D = _Dist()
    T = 131072 if args.ctx == 32768 else args.ctx
    W = max(args.warmup, 3)
    sampler = ClockSampler(D.local) if D.rank == 0 else None
    if sampler:
        sampler.start()
    res = measure_seqsplit(D, args.layers, args.steps, W, T=T, merge=args.merge)
    clocks = sampler.stop() if sampler else None
    if D.rank == 0:
        line = {"metric": METRIC, "value": res["us_per_layer"], "unit": "us", "n_gpus": D.world, "steps": args.steps,
                "warmup": W, "ms_per_step": res["us_per_layer"] * args.layers / 1e3, "higher_is_better": False,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": res["workload"], "parallelism": f"sequence-split x{D.world}"},
                "seqsplit": res,
                "e2e": {"value": None, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": args.steps * (1 + args.layers * 2), "clocks": clocks}
        print(json.dumps(line), flush=True)
    ok = res["parity_max_abs"] <= 2e-3 and res["bitwise_equal_across_ranks"]
    D.close()
    if not ok:
        raise SystemExit("sequence-split parity check failed")


def run_compress_profile(args):
    """Prefill compressor, one layer of a T-token sequence: CUDA-event time of every kernel family run
    on its own (median of 7 after 3 warm-ups), with its algorithmic bytes / FLOPs against the measured
    peaks, and the whole `Cache.compress()` of the layer.  One GPU."""
    import torch
    import synth
    from shard_b200 import Cache, ops
    from shard_b200.cache import kmeans, pca_fit
    from shard_b200.streaming import get_codebook, stream_signs

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    T = args.ctx
    n = T - SINK - WIN
    hbm_peak, tf_burst, tf_sustained, peak_kind = measured_peaks()
    k, v, _ = synth.make_kvq(T, 100, device=dev)
    inv = synth.rope_inv_freq().to(dev)

    def timed(fn, reps=7, warm=3):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    k_mid, v_mid = k[0, :, SINK:T - WIN, :], v[0, :, SINK:T - WIN, :]
    rows = []

    def row(name, ms, nbytes=None, flops=None, note=""):
        r = {"kernel": name, "ms": ms, "note": note}
        if nbytes:
            r.update(algorithmic_bytes=nbytes, gbs=nbytes / ms / 1e6, hbm_frac=nbytes / ms / 1e6 / hbm_peak)
        if flops:
            r.update(algorithmic_flops=flops, tflops=flops / ms / 1e9)
        rows.append(r)

    flat = ops.undo_rope(k_mid, SINK, inv)
    row("undo_rope_kernel", timed(lambda: ops.undo_rope(k_mid, SINK, inv)), nbytes=n * 1024 * (2 + 4),
        note="reads fp16 keys, writes fp32")
    mean = flat.mean(dim=0).contiguous()
    basis, eig = pca_fit(flat, mean, RANK)
    row("pca_fit (torch: Gram matrix GEMM + eigh)", timed(lambda: pca_fit(flat, mean, RANK), reps=3, warm=1),
        flops=2 * n * 1024 * 1024, note="library GEMM + cuSOLVER eigensolver on 1024 x 1024")
    scale = basis.abs().amax(0).clamp(min=1e-6) / 127.0
    w = ((basis / scale).round().clamp(-127, 127) * scale).contiguous()
    proj = ops.k_project(flat, mean, w)
    ms = timed(lambda: ops.k_project(flat, mean, w))
    row("k_project_tc_kernel (+ weight split)", ms, nbytes=n * 1024 * 4 + n * RANK * 4, flops=2 * n * 1024 * RANK,
        note="3 tf32 MMAs per k-step: tensor work is 3x the algorithmic FLOPs; frac_of_tf32_peak uses half the bf16 peak")
    rows[-1]["tensor_frac_of_tf32_peak"] = 3 * 2 * n * 1024 * RANK / ms / 1e9 / (tf_burst / 2)
    alloc = [4] * RANK
    row("kq_* (min/max, max-abs, scale, pack)", timed(lambda: ops.k_quantize_pack(proj, alloc)),
        nbytes=3 * n * RANK * 4 + n * RANK // 2, note="three passes over the fp32 projection, writes packed int4")
    x, ch = ops.v_hadamard_normalise(v_mid)
    row("v_rotate / v_clamp / v_normalise", timed(lambda: ops.v_hadamard_normalise(v_mid)),
        nbytes=n * 1024 * (2 + 4 + 4 + 4), note="reads fp16 values, writes fp32, normalises in place")
    flat_v = x.view(-1, 4)
    g = torch.Generator(device=dev).manual_seed(42)
    cent = flat_v[torch.randperm(flat_v.shape[0], generator=g, device=dev)[:256]].clone()
    sums, counts = torch.zeros_like(cent), torch.zeros(256, device=dev)
    nsub = flat_v.shape[0]
    ms = timed(lambda: ops.vq_assign_accumulate(flat_v, cent, sums, counts))
    row("vq_assign_kernel<true> (one k-means pass)", ms, nbytes=nsub * 17, flops=12 * 256 * nsub,
        note="fp32 CUDA cores: 256 distances of 4 subtractions, 4 multiply-adds ... per sub-vector")
    row("kmeans (30 iterations at most)", timed(lambda: kmeans(flat_v, 256, n_iter=30), reps=3, warm=1), note="whole V codebook fit")
    cb, signs = get_codebook(HD, 8, dev), stream_signs(0, HD, dev)
    bufs = [torch.zeros(16, N_KV, HD, dtype=torch.uint8, device=dev) for _ in range(2)] + \
           [torch.zeros(16, N_KV, dtype=torch.float16, device=dev) for _ in range(2)]
    tk, tv = k[0, :, 0, :].contiguous(), v[0, :, 0, :].contiguous()
    row("stream_quantize_kernel", timed(lambda: ops.stream_quantize(tk, tv, signs, cb, *bufs, 0)), nbytes=2 * N_KV * HD * 3,
        note="one token: launch latency")
    cache = Cache(num_layers=1, rope_inv_freq=synth.rope_inv_freq())
    cache.layers[0].update(k, v)
    cache.compress()
    line = {"metric": "prefill_compress_s_per_layer", "value": cache.compress_seconds, "unit": "s", "n_gpus": 1,
            "steps": 1, "warmup": 0, "ms_per_step": cache.compress_seconds * 1e3, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"prefill compression of one layer, {T}-token sequence (n_comp = {n}), Llama-3.1-8B geometry"},
            "peaks": {"hbm_gbs": hbm_peak, "bf16_tflops_burst": tf_burst, "kind": peak_kind}, "kernels": rows,
            "e2e": {"value": None, "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": len(rows)}
    print(json.dumps(line), flush=True)


def run_generate(args):
    """BASELINE configs[1]: a random-init Llama-3.1-8B-shape decoder driven through HF `generate`
    semantics -- prefill 8192 synthetic ids, compress the cache, decode greedily with the 8-bit
    stream -- through `Cache` + `enable_llama_fused_attention`.  One GPU."""
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM
    import shard_b200.attention as A
    from shard_b200 import Cache, enable_llama_fused_attention

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    L = args.layers
    T = 8192 if args.ctx == 32768 else args.ctx
    n_new = min(args.steps, 128)
    cfg = LlamaConfig(hidden_size=4096, intermediate_size=14336, num_hidden_layers=L, num_attention_heads=N_Q,
                      num_key_value_heads=N_KV, head_dim=HD, vocab_size=128256, rope_theta=500000.0,
                      max_position_embeddings=T + 1024)
    torch.manual_seed(0)
    torch.set_default_dtype(torch.float16)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg)
    torch.set_default_dtype(torch.float32)
    model.eval()
    enable_llama_fused_attention(model)
    ids = torch.randint(0, 128256, (1, T), generator=torch.Generator().manual_seed(0)).to(dev)
    cache = Cache.from_model(model)
    cache._streaming = True

    attn_ev = []
    real = A.fused_attention_compressed

    def timed(*a, **k):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = real(*a, **k)
        e1.record()
        attn_ev.append((e0, e1))
        return out

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    with torch.no_grad():
        ev[0].record()
        logits = model(ids, past_key_values=cache, use_cache=True).logits[:, -1]
        ev[1].record()
        cache.compress()
        ev[2].record()
        tok = logits.argmax(-1, keepdim=True)
        # first decode step (not timed)
        tok = model(tok, past_key_values=cache, use_cache=True).logits[:, -1].argmax(-1, keepdim=True)
        A.fused_attention_compressed = timed
        sampler = ClockSampler(0)
        sampler.start()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n_new):
            tok = model(tok, past_key_values=cache, use_cache=True).logits[:, -1].argmax(-1, keepdim=True)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        clocks = sampler.stop()
        A.fused_attention_compressed = real
    cache.check()
    attn_us = sum(a.elapsed_time(b) for a, b in attn_ev) * 1e3 / max(len(attn_ev), 1)
    line = {
        "metric": METRIC, "value": attn_us, "unit": "us", "n_gpus": 1, "steps": n_new, "warmup": 1,
        "ms_per_step": wall * 1e3 / n_new, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"cfg1: random-init Llama-3.1-8B-shape decoder ({L} layers), prefill {T} synthetic ids, "
                               f"compress, {n_new} greedy decode steps with the 8-bit stream, through "
                               "Cache + enable_llama_fused_attention (whole model forward per step)",
                   "note": "value = mean CUDA-event time around fused_attention_compressed per layer and step "
                           "(events recorded from Python inside the model forward, so it includes launch gaps); "
                           "ms_per_step = whole decode step of the model"},
        "prefill_ms": ev[0].elapsed_time(ev[1]), "prefill_compress_s": ev[1].elapsed_time(ev[2]) / 1e3,
        "decode_tokens_per_s": n_new / wall,
        "compress_ratio": cache.compress_ratio(), "clean_compress_ratio": cache.clean_compress_ratio(),
        "e2e": {"value": None, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": len(attn_ev), "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-triton"])
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seqs", type=int, default=1, help="sequences per GPU (cfg2)")
    ap.add_argument("--workload", default="cfg2", choices=["cfg1", "cfg2", "cfg3", "cfg4", "compress"],
                    help="cfg1: Llama-8B-shape decoder, 8K prefill + greedy decode through the HF hook (1 GPU); "
                         "cfg2: one 32K sequence per GPU (headline; at N > 1 the line also carries cfg4 and cfg3 "
                         "records); cfg3: 64 x 8K sequences sharded by batch; "
                         "cfg4: one 131072-token sequence split by token range; "
                         "compress: per-kernel timing of the prefill compressor on one layer (1 GPU)")
    ap.add_argument("--merge", default="peer", choices=["peer", "nccl", "both"],
                    help="cfg4 at N > 1: deliver the partial records over peer memory from inside the decode "
                         "launch (default), or NCCL all-gather followed by a merge launch, or time both")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--no-reference-triton", dest="reference_triton", action="store_false")
    ap.add_argument("--no-multi-extras", dest="multi_extras", action="store_false",
                    help="at N > 1 skip the sequence-split and 64-sequence records")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-triton":
        run_reference_triton(args)
    elif args.workload == "cfg4":
        run_seqsplit(args)
    elif args.workload == "cfg3":
        run_batch64(args)
    elif args.workload == "cfg1":
        run_generate(args)
    elif args.workload == "compress":
        run_compress_profile(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
