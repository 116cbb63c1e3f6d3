"""Benchmark of the compressed-KV decode attention path (BASELINE.json metric).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
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
ms_per_step / (layers * total sequences), time is the max over ranks.

One JSON line is printed by rank 0.  `--impl reference` times the CPU port of the
reference's algorithm (the numpy oracle) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

N_Q, N_KV, HD, RANK, SINK, WIN = 32, 8, 128, 192, 4, 64
METRIC = "compressed_kv_decode_attn_us_per_step_per_layer"


def algorithmic_bytes(n_comp, n_stream, rank=RANK, n_sink=SINK, n_win=WIN):
    """Bytes one layer-step must touch, every operand counted once: packed int4
    coefficients + VQ codes per middle token, fp16 basis, mean, scales, codebook,
    fp16 sink/window K and V, stream codes + norms, query in, output out."""
    per_tok = rank // 2 + N_KV * 32
    fixed = 2 * rank * N_KV * HD + 2 * N_KV * HD + 2 * rank + 256 * 4 * 2 + 2 * N_KV * HD
    fixed += (n_sink + n_win) * N_KV * HD * 2 * 2 + N_Q * HD * 2 * 2
    return n_comp * per_tok + fixed + n_stream * (2 * N_KV * HD + 2 * 2 * N_KV)


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_partial_pipe_kernel launch on the
# cfg2 geometry (ncu capture summarised under profiles/); None for other workloads
TRAFFIC_BYTES_PER_LAUNCH = 20858624


def measured_peaks():
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 0))), "measured"
    return 6650.0, 1590.0, "fallback"


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
def synthetic_compressed_layer_numpy(n_comp, seed=0):
    """A compressed layer with random codes (decode cost does not depend on code values)."""
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
    """Seconds per layer-step of the CPU port (numpy oracle) of the reference's decode,
    including the stream append, on all host cores numpy's BLAS uses."""
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


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.ctx
    n_comp = T - SINK - WIN
    # A step is one layer-step of the CPU port (about 1.5 s at 32K on 16 cores).  To keep K steps
    # within about two minutes a step attends to a contiguous share of the middle tokens when K is
    # large; the cost is linear in the tokens, so the time is scaled back to the whole layer.
    K = max(1, args.steps)
    budget_s, est_full_s = 120.0, 1.5 * n_comp / 32700.0
    n_sample = n_comp if K * est_full_s <= budget_s else max(1024, int(n_comp * budget_s / (K * est_full_s)))
    sec, cores = time_cpu_port(n_sample, K, max(1, min(args.warmup, 1)))
    sec *= n_comp / n_sample
    us = sec * 1e6
    sample = (f"1 layer-step per timed step (of {args.layers} layers), random codes, numpy port; "
              + (f"whole middle segment, n_comp={n_comp}" if n_sample == n_comp else
                 f"{n_sample} of the {n_comp} middle tokens per step, time scaled by {n_comp / n_sample:.2f}"))
    line = {
        "impl": "reference", "metric": METRIC, "value": us, "unit": "us", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * args.layers,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"cfg2: Llama-3.1-8B geometry, {T}-token context, {args.layers} layers, batch 1"},
        "cpu_baseline": {"value": us, "unit": "us", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm
def build_cache(T, layers, seed0, dev):
    import torch
    from shard_b200 import Cache, synth
    cache = Cache(num_layers=layers, rope_inv_freq=synth.rope_inv_freq())
    cache._streaming = True
    for li in range(layers):
        k, v, _ = synth.make_kvq(T, seed0 + li, device=dev)
        cache.layers[li].update(k, v)
    cache.compress()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return cache


def run_ours(args):
    import torch
    import torch.distributed as dist
    from shard_b200 import fused_attention_compressed
    from shard_b200.parallel import BatchedDecoder

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    T, L = args.ctx, args.layers
    K, W = args.steps, max(args.warmup, 3)
    seqs_per_gpu = args.seqs
    cfg3 = args.workload == "cfg3"
    if cfg3:
        T = 8192 if args.ctx == 32768 else args.ctx
        total_seqs = 64
        if total_seqs % world:
            raise SystemExit("cfg3 needs a GPU count that divides 64")
        seqs_per_gpu = total_seqs // world
    n_comp = T - SINK - WIN

    t0 = time.perf_counter()
    if cfg3:
        # 64 x 32 layer caches: random codes built on the device (decode cost is data independent)
        from shard_b200 import synth as _synth
        caches = [_synth.random_cache(n_comp, L, dev, 5000 + 100 * (rank * seqs_per_gpu + s))
                  for s in range(seqs_per_gpu)]
        compress_s, ratio = None, None
    else:
        caches = [build_cache(T, L, 100 + 1000 * (rank * seqs_per_gpu + s), dev) for s in range(seqs_per_gpu)]
        compress_s = sum(c.compress_seconds for c in caches) / len(caches)
        ratio = caches[0].clean_compress_ratio()
    build_s = time.perf_counter() - t0

    bd = BatchedDecoder(caches, stream_capacity=2 * (K + W) + 8)
    total = K + W
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    q_pool = torch.randn(total, L, seqs_per_gpu, N_Q, HD, generator=g, device=dev).half()
    k_pool = torch.randn(total, L, seqs_per_gpu, N_KV, HD, generator=g, device=dev).half()
    v_pool = torch.randn(total, L, seqs_per_gpu, N_KV, HD, generator=g, device=dev).half()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step(j):
        bd.q.copy_(q_pool[j])
        bd.new_k.copy_(k_pool[j])
        bd.new_v.copy_(v_pool[j])
        bd.step(T + j)

    # ---- device-resident timing -------------------------------------------------
    for j in range(W):
        one_step(j)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for j in range(W, W + K):
        one_step(j)
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)

    # ---- dominant kernel: the timed region is K * L launches of the decode kernel plus K launches
    # of the 5.6 us phase-table kernel, back to back on one stream, so its average launch duration
    # is the region's event time over K * L (the phase table adds 1/L of its time to each)
    s_now = bd.n_stream
    kern_ms = ms_total / (K * L)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the public API, host buffers ----------------------------
    e2e_steps = min(K, 4 if cfg3 else 64)
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
    barrier()
    t0 = time.perf_counter()
    for j in range(e2e_steps):
        e2e_step(pos + 3 + j)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps

    # ---- reduce over ranks ---------------------------------------------------------
    vals = torch.tensor([ms_total, e2e_ms, kern_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, kern_ms = (float(x) for x in vals.tolist())
    ms_per_step = ms_total / K
    n_seq_total = seqs_per_gpu * world
    us = ms_per_step * 1e3 / (L * n_seq_total)

    if rank == 0:
        hbm_peak, tf_peak, peak_kind = measured_peaks()
        s_mid = W + K // 2
        bytes_ls = algorithmic_bytes(n_comp, s_mid)
        flops_ls = 2 * n_comp * RANK * N_KV * HD + 4 * N_Q * HD * n_comp
        kern_bytes = algorithmic_bytes(n_comp, s_now) * seqs_per_gpu
        kern_flops = flops_ls * seqs_per_gpu
        achieved = kern_bytes / (kern_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": us, "unit": "us", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong" if cfg3 else "weak",
            "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {
                "workload": (f"{args.workload}: Llama-3.1-8B geometry ({N_Q}/{N_KV} heads, head_dim {HD}), "
                             f"{T}-token context, {L} layers, {seqs_per_gpu} sequence(s) per GPU"
                             + (f" ({seqs_per_gpu * world} in total, random codes)" if cfg3 else "")
                             + f", 8-bit stream grows {W}->{W + K} tokens"),
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
                         "bound": "tensor", "achieved": kern_flops / (kern_ms * 1e-3) / 1e12, "peak": tf_peak,
                         "unit": "TFLOP/s", "frac": kern_flops / (kern_ms * 1e-3) / 1e12 / tf_peak,
                         "peak_kind": peak_kind + " (cuBLAS bf16, sustained)", "traffic": TRAFFIC_BYTES_PER_LAUNCH if (args.workload == "cfg2" and T == 32768 and seqs_per_gpu == 1) else None,
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
        if args.cpu_baseline:
            sec, cores = time_cpu_port(n_comp, 2, 1)
            line["cpu_baseline"] = {"value": sec * 1e6, "unit": "us", "cores": cores, "kind": "port",
                                    "sample": f"3 layer-steps (1 warm-up) of one layer, n_comp={n_comp}, "
                                              "numpy port of the reference's CPU path"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_seqsplit(args):
    """cfg4: one long sequence, its compressed middle cut into contiguous token ranges (one per
    GPU); every rank decodes its range, the per-head (max, sum-exp, acc) records are all-gathered
    over NCCL and merged by the log-sum-exp kernel.  Rank 0 also owns sink, window and stream."""
    import torch
    import torch.distributed as dist
    from shard_b200 import ops, synth
    from shard_b200.attention import decode_layer
    from shard_b200.parallel import split_ranges

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T = 131072 if args.ctx == 32768 else args.ctx
    L, K, W = args.layers, args.steps, max(args.warmup, 3)
    n_comp = T - SINK - WIN
    begin, end = split_ranges(n_comp, world)[rank]
    first = rank == 0
    cache = synth.random_cache(end - begin, L, dev, 9000, compress_start=SINK + begin,
                               n_sink=SINK if first else 0, n_win=WIN if first else 0)
    total = K + W
    g = torch.Generator(device=dev).manual_seed(77)          # same queries on every rank
    q_pool = torch.randn(total, L, 1, N_Q, 1, HD, generator=g, device=dev).half()
    k_pool = torch.randn(total, L, 1, N_KV, 1, HD, generator=g, device=dev).half()
    v_pool = torch.randn(total, L, 1, N_KV, 1, HD, generator=g, device=dev).half()
    parts = torch.empty(world, N_Q, 132, dtype=torch.float32, device=dev)
    part = torch.empty(N_Q, 132, dtype=torch.float32, device=dev)
    out = torch.empty(L, N_Q, HD, dtype=torch.float16, device=dev)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K * L)]
    peer = None
    if world > 1 and args.merge == "peer":
        from shard_b200.parallel import PeerExchange
        peer = PeerExchange(N_KV)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(j, timed):
        pos = T + j
        cache._fused_decode_update = True
        for li in range(L):
            layer = cache.layers[li]
            if first:
                layer.update(k_pool[j, li], v_pool[j, li])           # stream append (rank 0 owns the stream)
            e = ev[(j - W) * L + li] if timed else None
            if e: e[0].record()
            decode_layer(q_pool[j, li], layer, pos, partial_out=True, with_fp16_segments=first, out=part)
            if e: e[1].record()
            if peer is not None:
                peer.merge(part, out=out[li])                        # peer stores + flags + merge, one kernel
            else:
                if world > 1:
                    dist.all_gather_into_tensor(parts.view(-1), part.view(-1))
                else:
                    parts[0].copy_(part)
                ops.lse_merge(parts, out=out[li])
            if e: e[2].record()
        cache._fused_decode_update = False

    for j in range(W):
        step(j, False)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for j in range(W, W + K):
        step(j, True)
    ev1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = ev0.elapsed_time(ev1)
    dec_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / K
    mrg_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / K
    vals = torch.tensor([ms_total, dec_ms, mrg_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms_total, dec_ms, mrg_ms = (float(x) for x in vals.tolist())
    ms_per_step = ms_total / K
    if rank == 0:
        hbm_peak, tf_peak, peak_kind = measured_peaks()
        n_local = end - begin
        bytes_ls = algorithmic_bytes(n_local, W + K // 2)
        flops_l = 2 * n_local * RANK * N_KV * HD + 4 * N_Q * HD * n_local
        line = {
            "metric": METRIC, "value": ms_per_step * 1e3 / L, "unit": "us", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"cfg4: one {T}-token sequence, {L} layers, compressed middle split into "
                                   f"{world} contiguous token range(s) (random codes), log-sum-exp merge "
                                   + ("over NVLink peer memory inside the merge kernel" if peer is not None
                                      else "after an NCCL all-gather" if world > 1 else "on one GPU"),
                       "l2": "inputs larger than L2: one step touches %.0f MB of cache per GPU" % (bytes_ls * L / 1e6),
                       "parallelism": f"sequence-split x{world}"},
            "decode_us_per_layer": dec_ms * 1e3 / L, "merge_us_per_layer": mrg_ms * 1e3 / L,
            "merge_overhead_frac": mrg_ms / max(dec_ms + mrg_ms, 1e-9),
            "hbm_gbs_per_gpu": bytes_ls * L / (ms_per_step * 1e-3) / 1e9,
            "roofline": {"kernel": "decode_partial_pipe_kernel", "bound": "tensor",
                         "achieved": flops_l / (dec_ms / L * 1e-3) / 1e12, "peak": tf_peak, "unit": "TFLOP/s",
                         "frac": flops_l / (dec_ms / L * 1e-3) / 1e12 / tf_peak,
                         "peak_kind": peak_kind + " (cuBLAS bf16, sustained)", "traffic": None,
                         "hbm_achieved_gbs": bytes_ls / (dec_ms / L * 1e-3) / 1e9, "hbm_peak_gbs": hbm_peak},
            "e2e": {"value": None, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": K * (1 + L * 2), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if peer is not None:
        peer.check()
        peer.close()
    if world > 1:
        dist.destroy_process_group()


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
        # first decode step: layer 0 goes through the stock path once (its update is what would have
        # triggered the compression); not timed
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
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seqs", type=int, default=1, help="sequences per GPU (cfg2)")
    ap.add_argument("--workload", default="cfg2", choices=["cfg1", "cfg2", "cfg3", "cfg4"],
                    help="cfg1: Llama-8B-shape decoder, 8K prefill + greedy decode through the HF hook (1 GPU); "
                         "cfg2: one 32K sequence per GPU (headline); cfg3: 64 x 8K sequences sharded by batch; "
                         "cfg4: one 131072-token sequence split by token range, merged over NCCL")
    ap.add_argument("--merge", default="peer", choices=["peer", "nccl"],
                    help="cfg4 at N > 1: exchange the partial records over peer memory inside the merge "
                         "kernel (default) or with an NCCL all-gather followed by a merge launch")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "cfg4":
        run_seqsplit(args)
    elif args.workload == "cfg1":
        run_generate(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
