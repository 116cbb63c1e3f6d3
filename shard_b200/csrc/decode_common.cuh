// Pieces shared by the decode kernels: launch plan, per-CTA query staging, the
// warp-per-token path for fp16 / streamed rows, and the CTA-level merge that emits one
// (max, sum-exp, acc[128]) record per query head.
#pragma once

#include "common.cuh"
#include "peer_layout.cuh"

namespace shard {

constexpr int ROWS_PER_CTA = 32;        // rows per CTA when a launch has no middle segment
constexpr int MAX_ROW_CTAS = 18;

// Sequence-split decode: where the launch's result goes when it is delivered straight into the
// exchange buffers of all ranks (layout in peer_layout.cuh).  world == 0: no delivery.
struct PeerPush {
  unsigned char* bufs[PEER_MAX_WORLD];
  int rank, world;
  unsigned int epoch;
  void* merged_out;              // fp16 [n_q][128]: if set, the delivering CTA also waits for all ranks' records and merges
  int* status;                   // set to 1 when that wait gives up (may be null)
  unsigned long long wait_ns;    // its bound
};

struct DecodeParams {
  ShardSeq one;
  const ShardSeq* table;
  ShardDecodeShape sh;
  const float* inv_freq;
  const float* codebook;
  float* ws;
  int* status;          // device word set non-zero when a bounded wait gave up
  int* tickets;         // [batch][nkv] arrival counters of the fused combine (zero between calls)
  int n_chunks;         // CTAs (per KV head) that walk the compressed middle (0: there is no middle)
  int tiles_per_chunk;
  int tiles_rem;        // the first tiles_rem chunks walk one tile more
  int n_row_parts;      // CTAs (per KV head) that share the fp16 / streamed rows: the chunk CTAs
                        // themselves when there is a middle, else CTAs of their own; 0: no rows
  int n_parts;          // records per (sequence, query head): n_chunks rotated-space + n_row_parts standard
  int n_ctas;           // CTAs per (sequence, KV head) = gridDim.x
  PeerPush push;        // sequence-split: deliver the combined record to every rank's exchange buffer
};

struct SoftmaxState {
  float m[GQA];
  float l[GQA];       // lane-local partial sums (see call sites)
  float acc[GQA][4];  // lane owns channels 4*lane .. 4*lane+3
};

__device__ __forceinline__ void softmax_init(SoftmaxState& st) {
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    st.m[h] = neg_inf();
    st.l[h] = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) st.acc[h][c] = 0.f;
  }
}

// one streamed token: fp16 value of channels 4*lane..+3 exactly as the reference's
// dequantize_per_token + norm scaling produce it
__device__ __forceinline__ void stream_dequant_lane4(const uint8_t* __restrict__ idx_row, float nrm,
                                                     const float* __restrict__ cbs, const float4 sg, int lane,
                                                     float (&o)[4]) {
  // L2-coherent load: the row may have been written by this CTA a moment ago (fused append)
  const uint32_t codes = __ldcg(reinterpret_cast<const unsigned int*>(idx_row + 4 * lane));
  float x[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = cbs[(codes >> (8 * i)) & 0xff];
  fwht128_lane4(x, lane);
  const float sgn[4] = {sg.x, sg.y, sg.z, sg.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half unit = __float2half_rn(__fmul_rn(__fdiv_rn(x[i], SQRT_HD), sgn[i]));
    o[i] = __half2float(__float2half_rn(__fmul_rn(__half2float(unit), nrm)));
  }
}

// online-softmax update with one token whose 4 scores are warp-uniform
__device__ __forceinline__ void row_update(SoftmaxState& st, const float (&s)[GQA], const float (&v)[4]) {
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    const float mn = fmaxf(st.m[h], s[h]);
    const float alpha = (st.m[h] == neg_inf()) ? 0.f : exp2f((st.m[h] - mn) * LOG2E);
    const float pr = exp2f((s[h] - mn) * LOG2E);
    st.m[h] = mn;
    st.l[h] = st.l[h] * alpha + pr;
#pragma unroll
    for (int c = 0; c < 4; ++c) st.acc[h][c] = st.acc[h][c] * alpha + pr * v[c];
  }
}


// Un-rotated query (fp16 arithmetic, as the reference does it) and the query as given,
// for the 4 heads of KV group `kv`; thread d < 128 handles channel d.
__device__ __forceinline__ void stage_query(const ShardSeq& sq, int kv, int pos_q, const float* __restrict__ inv_freq,
                                            int d, float* __restrict__ qn, float* __restrict__ qr) {
  const int i = d & 63;
  const float phase = __fmul_rn((float)pos_q, inv_freq[i]);
  float sn, cs;
  sincosf(phase, &sn, &cs);
  const __half c16 = __float2half_rn(cs), s16 = __float2half_rn(sn);
  const __half* qg = reinterpret_cast<const __half*>(sq.q) + (size_t)kv * GQA * HD;
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    const __half x = qg[h * HD + d];
    const __half other = qg[h * HD + (d ^ 64)];
    const __half rot = (d < 64) ? __hneg(other) : other;
    const __half un = __hsub(__hmul(x, c16), __hmul(rot, s16));
    qn[h * HD + d] = __half2float(un);
    qr[h * HD + d] = __half2float(x);
  }
}

// Fused append: the CTA that owns streamed row n_stream-1 first quantises the step's new
// K/V vector of its KV head into that row (one warp each for K and V).  The caller synchronises
// the CTA afterwards; the rows are then read back with L2-coherent loads.
__device__ __forceinline__ void append_new_token(const ShardSeq& sq, const ShardDecodeShape& sh, int kv,
                                                 const float* __restrict__ cbs, bool is_v, int lane) {
  const size_t row = (size_t)(sh.n_stream - 1) * sh.nkv + kv;
  const __half* src = reinterpret_cast<const __half*>(is_v ? sq.new_v : sq.new_k) + kv * HD;
  uint8_t* idx_out = (is_v ? sq.st_v_idx : sq.st_k_idx) + row * HD;
  __half* norm_out = reinterpret_cast<__half*>(is_v ? sq.st_v_norm : sq.st_k_norm) + row;
  quantize_vec_warp(src, sq.signs, cbs, idx_out, norm_out, lane);
}

// Rows outside the compressed middle, in one index space: u < n_sink + n_win + n_dec is an fp16
// row (sink rows first, then window, then the fp16 decode buffer), the rest are streamed rows.  A warp takes rows u_first, u_first + u_step, ...;
// lane owns channels 4*lane..+3.  `qr` is the query as given (fp32 copy in shared memory), `cbs`
// the stream codebook in shared memory (needed for streamed rows only).
__device__ __forceinline__ void process_rows(SoftmaxState& st, const ShardSeq& sq, const ShardDecodeShape& sh,
                                             int kv, int u_first, int u_step,
                                             const float* __restrict__ qr, const float* __restrict__ cbs, int lane) {
  const int n_sw = sh.n_sink + sh.n_win, n_fp = n_sw + sh.n_dec, n_rows = n_fp + sh.n_stream;
  if (u_first >= n_rows) return;
  float4 sg = make_float4(0.f, 0.f, 0.f, 0.f);
  if (sh.n_stream > 0) sg = *reinterpret_cast<const float4*>(sq.signs + 4 * lane);
  float4 qv[GQA];
#pragma unroll
  for (int h = 0; h < GQA; ++h) qv[h] = *reinterpret_cast<const float4*>(qr + h * HD + 4 * lane);
  for (int u = u_first; u < n_rows; u += u_step) {
    float kx[4], vx[4];
    if (u < n_fp) {
      const bool in_sink = u < sh.n_sink, in_dec = u >= n_sw;
      const int r = in_sink ? u : (in_dec ? u - n_sw : u - sh.n_sink);
      const int rows = in_sink ? sh.n_sink : (in_dec ? (sh.dec_cap > 0 ? sh.dec_cap : sh.n_dec) : sh.n_win);
      const __half* kb = reinterpret_cast<const __half*>(in_sink ? sq.sink_k : (in_dec ? sq.dec_k : sq.win_k));
      const __half* vb = reinterpret_cast<const __half*>(in_sink ? sq.sink_v : (in_dec ? sq.dec_v : sq.win_v));
      const size_t off = ((size_t)kv * rows + r) * HD + 4 * lane;
      const uint2 kr = *reinterpret_cast<const uint2*>(kb + off);
      const uint2 vr = *reinterpret_cast<const uint2*>(vb + off);
      const float2 k01 = __half22float2(*reinterpret_cast<const __half2*>(&kr.x));
      const float2 k23 = __half22float2(*reinterpret_cast<const __half2*>(&kr.y));
      const float2 v01 = __half22float2(*reinterpret_cast<const __half2*>(&vr.x));
      const float2 v23 = __half22float2(*reinterpret_cast<const __half2*>(&vr.y));
      kx[0] = k01.x; kx[1] = k01.y; kx[2] = k23.x; kx[3] = k23.y;
      vx[0] = v01.x; vx[1] = v01.y; vx[2] = v23.x; vx[3] = v23.y;
    } else {
      const size_t row = (size_t)(u - n_fp) * sh.nkv + kv;
      const float kn = __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(sq.st_k_norm) + row)));
      const float vn = __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(sq.st_v_norm) + row)));
      stream_dequant_lane4(sq.st_k_idx + row * HD, kn, cbs, sg, lane, kx);
      stream_dequant_lane4(sq.st_v_idx + row * HD, vn, cbs, sg, lane, vx);
    }
    float s[GQA];
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      float d = qv[h].x * kx[0];
      d = fmaf(qv[h].y, kx[1], d);
      d = fmaf(qv[h].z, kx[2], d);
      d = fmaf(qv[h].w, kx[3], d);
      s[h] = warp_sum(d) * INV_SQRT_HD;
    }
    row_update(st, s, vx);
  }
}

// Merge of per-warp softmax states (lane owns channels 4*lane..+3, m/l are warp-uniform) into one
// record per head, in two steps with a barrier of the caller's choice in between:
// partial_store by every one of the NWARPS warps (index `w`), then partial_merge by 128 threads
// (d = 0..127).  `scratch` needs NWARPS*4*130 floats.
template <int NWARPS>
__device__ __forceinline__ void partial_store(const SoftmaxState& st, float* __restrict__ scratch, int w, int lane) {
  float* mw = scratch;
  float* lw = mw + NWARPS * GQA;
  float* aw = lw + NWARPS * GQA;
  if (lane == 0) {
#pragma unroll
    for (int h = 0; h < GQA; ++h) { mw[w * GQA + h] = st.m[h]; lw[w * GQA + h] = st.l[h]; }
  }
#pragma unroll
  for (int h = 0; h < GQA; ++h)
    *reinterpret_cast<float4*>(aw + (w * GQA + h) * HD + 4 * lane) =
        make_float4(st.acc[h][0], st.acc[h][1], st.acc[h][2], st.acc[h][3]);
}

template <int NWARPS>
__device__ __forceinline__ void partial_merge(const float* scratch, float* __restrict__ rec_base, int d) {
  const float* mw = scratch;
  const float* lw = mw + NWARPS * GQA;
  const float* aw = lw + NWARPS * GQA;
#pragma unroll
  for (int h = 0; h < GQA; ++h) {
    float M = neg_inf();
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, mw[w * GQA + h]);
    float L = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float mwv = mw[w * GQA + h];
      const float wt = (mwv == neg_inf()) ? 0.f : exp2f((mwv - M) * LOG2E);
      L = fmaf(wt, lw[w * GQA + h], L);
      a = fmaf(wt, aw[(w * GQA + h) * HD + d], a);
    }
    float* rec = rec_base + h * PART;
    if (d == 0) { rec[0] = M; rec[1] = L; rec[2] = 0.f; rec[3] = 0.f; }
    rec[4 + d] = a;
  }
}

// Fused combine.  Every CTA of one (sequence, KV head) calls this after its record is written
// (`released`: the caller has already issued __threadfence + __syncthreads after those writes).
// Each takes a ticket; the CTA that draws the last one sees all records of that KV head
// (release/acquire through the fences around the ticket), merges them for the head's four
// query heads exactly as decode_combine_kernel does (same order, same operations), and puts
// the counter back to zero for the next call.  `sm` needs GQA*HD + 2*GQA*n_parts floats that
// are free; NTHREADS >= GQA*HD.  Thread tid handles head tid/128, channel tid%128.
template <int NTHREADS>
__device__ __forceinline__ void ticket_combine(const DecodeParams& p, const ShardSeq& sq, int kv, int b,
                                               float* sm_raw, int tid, bool released = false) {
  volatile float* sm = sm_raw;   // exchanged between threads: every access must reach shared memory
  static_assert(NTHREADS >= GQA * HD, "one thread per (head, channel)");
  __shared__ int last_s;
  if (!released) {               // the caller has not yet fenced its record writes and synchronised the CTA
    __threadfence();
    __syncthreads();
  }
  if (tid == 0) {
    int* ctr = p.tickets + b * p.sh.nkv + kv;
    const int last = atomicAdd(ctr, 1) == p.n_ctas - 1;
    if (last) atomicExch(ctr, 0);
    last_s = last;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  const bool active = tid < GQA * HD;
  const int n_q = p.sh.n_q, n_parts = p.n_parts, n_rot = p.n_chunks;
  const int hl = (tid >> 7) & (GQA - 1), h = kv * GQA + hl, d = tid & (HD - 1);
  const float* base0 = p.ws + ((size_t)b * n_parts * n_q + (size_t)kv * GQA) * PART;
  const size_t pstride = (size_t)n_q * PART;
  // This CTA is on the critical path of the launch: nobody else is left.
  float M = neg_inf(), L = 0.f, rot = 0.f, stdv = 0.f;
  const float* accp = base0 + hl * PART + 4 + d;
  if (n_parts <= 64) {
    // Every load goes out before anything is waited for, so the merge costs one round trip to L2
    // and no shared memory: lane j of a warp fetches (max, sum-exp) of parts j and j + 32 of the
    // warp's head -- the same for all its lanes -- and every thread its channel of every part (a
    // launch over one sequence of a model with 8 KV heads has 36 parts).
    constexpr int COMBINE_BATCH = 36;
    const int lane = tid & 31;
    float a0[COMBINE_BATCH];
#pragma unroll
    for (int pi = 0; pi < COMBINE_BATCH; ++pi) a0[pi] = (active && pi < n_parts) ? __ldcg(accp + pi * pstride) : 0.f;
    float mj[2], lj[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int pj = lane + 32 * k;
      const float* rec = base0 + pj * pstride + hl * PART;
      mj[k] = (active && pj < n_parts) ? __ldcg(rec) : neg_inf();
      lj[k] = (active && pj < n_parts) ? __ldcg(rec + 1) : 0.f;
    }
    if (active) {                                      // whole warps: tid < GQA * HD
      M = warp_max(fmaxf(mj[0], mj[1]));
      float wj[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) wj[k] = (mj[k] == neg_inf()) ? 0.f : exp2f((mj[k] - M) * LOG2E);
      // (parts in ascending order, the same operations as decode_combine_kernel)
#pragma unroll
      for (int pi = 0; pi < COMBINE_BATCH; ++pi) {
        const float wt = __shfl_sync(0xffffffffu, wj[pi >> 5], pi & 31);
        const float lp = __shfl_sync(0xffffffffu, lj[pi >> 5], pi & 31);
        if (pi < n_parts) {
          L = fmaf(wt, lp, L);
          if (pi < n_rot) rot = fmaf(wt, a0[pi], rot); else stdv = fmaf(wt, a0[pi], stdv);
        }
      }
      for (int pi = COMBINE_BATCH; pi < n_parts; ++pi) {
        const float wt = __shfl_sync(0xffffffffu, wj[pi >> 5], pi & 31);
        const float lp = __shfl_sync(0xffffffffu, lj[pi >> 5], pi & 31);
        const float a = __ldcg(accp + pi * pstride);
        L = fmaf(wt, lp, L);
        if (pi < n_rot) rot = fmaf(wt, a, rot); else stdv = fmaf(wt, a, stdv);
      }
    }
  } else {
    // many parts: (max, sum-exp) of every part of the four heads staged in shared memory
    volatile float* ms = sm + GQA * HD;                 // [GQA][n_parts]
    volatile float* ls = ms + GQA * n_parts;            // [GQA][n_parts]
    for (int idx = tid; idx < GQA * n_parts; idx += NTHREADS) {
      const int hh = idx / n_parts, pi = idx - hh * n_parts;
      const float* rec = base0 + pi * pstride + hh * PART;
      ms[idx] = __ldcg(rec);
      ls[idx] = __ldcg(rec + 1);
    }
    __syncthreads();
    if (active) {
      for (int pi = 0; pi < n_parts; ++pi) M = fmaxf(M, ms[hl * n_parts + pi]);
#pragma unroll 12
      for (int pi = 0; pi < n_parts; ++pi) {
        const float a = __ldcg(accp + pi * pstride);
        const float m = ms[hl * n_parts + pi];
        const float wt = (m == neg_inf()) ? 0.f : exp2f((m - M) * LOG2E);
        L = fmaf(wt, ls[hl * n_parts + pi], L);
        if (pi < n_rot) rot = fmaf(wt, a, rot); else stdv = fmaf(wt, a, stdv);
      }
    }
  }
  // inverse (= forward) normalised Hadamard of the rotated-space sum over the 128 channels of a
  // head (four warps): the butterflies inside a warp by shuffle, the last two through shared memory
  float v = rot;
  if (n_rot > 0) {
    if (active) {
#pragma unroll
      for (int hh = 1; hh < 32; hh <<= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, v, hh);
        v = (d & hh) ? other - v : v + other;
      }
    }
    for (int hh = 32; hh < HD; hh <<= 1) {
      if (active) sm[tid] = v;
      __syncthreads();
      if (active) {
        const float other = sm[tid ^ hh];
        v = (d & hh) ? other - v : v + other;
      }
      __syncthreads();
    }
    v = v / SQRT_HD;
  }
  const float o = v + stdv;
  if (p.push.world > 0) {
    // Sequence-split decode: this CTA holds the rank's final record of four query heads.  It goes
    // straight into slot epoch % 2 of EVERY rank's exchange buffer (plain peer stores over
    // NVLink), then -- after a system-scope fence by every storing thread -- the epoch number is
    // published in every rank's flag word for (this rank, this KV head).  The merge kernel of
    // each rank waits for those flags.
    const int slot = (int)(p.push.epoch & 1u);
    const size_t flag_bytes = peer_flag_bytes(p.push.world, p.sh.nkv);
    const size_t slot_floats = peer_slot_floats(p.push.world, p.sh.nkv);
    if (active) {
      for (int r = 0; r < p.push.world; ++r) {
        float* rec = reinterpret_cast<float*>(p.push.bufs[r] + flag_bytes) + slot * slot_floats +
                     ((size_t)p.push.rank * n_q + h) * PART;
        if (d == 0) { rec[0] = M; rec[1] = L; rec[2] = 0.f; rec[3] = 0.f; }
        rec[4 + d] = o;
      }
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.push.world) {
      volatile unsigned int* flag = reinterpret_cast<volatile unsigned int*>(p.push.bufs[tid]) +
                                    ((size_t)slot * p.push.world + p.push.rank) * p.sh.nkv + kv;
      *flag = p.push.epoch;
    }
    if (p.push.merged_out) {
      // ... and finishes the step itself: wait -- bounded by the global timer -- for every rank's
      // records of this KV head in the own buffer, merge them in rank order, write the attention
      // output.  (Eight CTAs of the launch do this, one per KV head, while the others have retired.)
      if (tid == 0) last_s = 0;                        // reused as "gave up"
      __syncthreads();
      if (tid < p.push.world) {
        volatile unsigned int* flag = reinterpret_cast<volatile unsigned int*>(p.push.bufs[p.push.rank]) +
                                      ((size_t)slot * p.push.world + tid) * p.sh.nkv + kv;
        if (!wait_epoch(flag, p.push.epoch, p.push.wait_ns)) last_s = 1;
        __threadfence_system();
      }
      __syncthreads();
      if (last_s) {
        if (tid == 0 && p.push.status) atomicExch(p.push.status, 1);
      } else if (active) {
        reinterpret_cast<__half*>(p.push.merged_out)[(size_t)h * HD + d] =
            merge_rank_records(p.push.bufs[p.push.rank], p.push.world, p.sh.nkv, slot, h, d);
      }
    }
    if (!sq.out) return;
  }
  if (!active) return;
  if (p.sh.partial_out) {
    float* rec = reinterpret_cast<float*>(sq.out) + (size_t)h * PART;
    if (d == 0) { rec[0] = M; rec[1] = L; rec[2] = 0.f; rec[3] = 0.f; }
    rec[4 + d] = o;
  } else {
    reinterpret_cast<__half*>(sq.out)[(size_t)h * HD + d] = __float2half_rn(o / L);
  }
}

}  // namespace shard
