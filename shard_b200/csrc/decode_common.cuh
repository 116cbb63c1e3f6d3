// Pieces shared by the decode kernels: launch plan, per-CTA query staging, the
// warp-per-token path for fp16 / streamed rows, and the CTA-level merge that emits one
// (max, sum-exp, acc[128]) record per query head.
#pragma once

#include "common.cuh"

namespace shard {

constexpr int STREAM_TOK_PER_CTA = 32;

struct DecodeParams {
  ShardSeq one;
  const ShardSeq* table;
  ShardDecodeShape sh;
  const float* inv_freq;
  const float* codebook;
  float* ws;
  int* status;          // device word set non-zero when a bounded wait gave up
  int* tickets;         // [batch][nkv] arrival counters of the fused combine (zero between calls)
  int n_chunks;         // CTAs (per KV head) that walk the compressed middle
  int tiles_per_chunk;
  int tiles_rem;        // pipelined kernel: the first tiles_rem chunks walk one tile more
  int n_fp16_ctas;      // 1 if there are sink / window rows
  int n_stream_ctas;
  int n_parts;          // n_chunks + n_fp16_ctas + n_stream_ctas
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
// K/V vector of its KV head into that row (warp 0: K, warp 1: V).  The caller synchronises
// the CTA afterwards; the rows are then read back with L2-coherent loads.
__device__ __forceinline__ void append_new_token(const ShardSeq& sq, const ShardDecodeShape& sh, int kv,
                                                 const float* __restrict__ cbs, int warp, int lane) {
  if (warp >= 2) return;
  const bool is_v = warp == 1;
  const size_t row = (size_t)(sh.n_stream - 1) * sh.nkv + kv;
  const __half* src = reinterpret_cast<const __half*>(is_v ? sq.new_v : sq.new_k) + kv * HD;
  uint8_t* idx_out = (is_v ? sq.st_v_idx : sq.st_k_idx) + row * HD;
  __half* norm_out = reinterpret_cast<__half*>(is_v ? sq.st_v_norm : sq.st_k_norm) + row;
  quantize_vec_warp(src, sq.signs, cbs, idx_out, norm_out, lane);
}

// fp16 rows (sink + window) or streamed rows [u_lo, u_hi): one warp per token, lane owns
// channels 4*lane..+3.  `qr` is the query as given (fp32 copy in shared memory), `cbs` the
// stream codebook in shared memory (streamed rows only).
template <int NWARPS>
__device__ __forceinline__ void process_rows(SoftmaxState& st, const ShardSeq& sq, const ShardDecodeShape& sh,
                                             int kv, bool is_fp16, int u_lo, int u_hi,
                                             const float* __restrict__ qr, const float* __restrict__ cbs,
                                             int warp, int lane) {
  float4 sg = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!is_fp16) sg = *reinterpret_cast<const float4*>(sq.signs + 4 * lane);
  float4 qv[GQA];
#pragma unroll
  for (int h = 0; h < GQA; ++h) qv[h] = *reinterpret_cast<const float4*>(qr + h * HD + 4 * lane);
  for (int u = u_lo + warp; u < u_hi; u += NWARPS) {
    float kx[4], vx[4];
    if (is_fp16) {
      const bool in_sink = u < sh.n_sink;
      const int r = in_sink ? u : u - sh.n_sink;
      const int rows = in_sink ? sh.n_sink : sh.n_win;
      const __half* kb = reinterpret_cast<const __half*>(in_sink ? sq.sink_k : sq.win_k);
      const __half* vb = reinterpret_cast<const __half*>(in_sink ? sq.sink_v : sq.win_v);
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
      const size_t row = (size_t)u * sh.nkv + kv;
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

// Merge the per-warp softmax states of a CTA (lane owns channels 4*lane..+3, m/l are
// warp-uniform) and write one record per head.  `scratch` needs NWARPS*4*130 floats and
// must not be in use; the caller has synchronised the CTA before the call.
template <int NWARPS>
__device__ __forceinline__ void emit_partial(const SoftmaxState& st, float* __restrict__ scratch,
                                             float* __restrict__ rec_base, int tid, int warp, int lane) {
  float* mw = scratch;
  float* lw = mw + NWARPS * GQA;
  float* aw = lw + NWARPS * GQA;
  if (lane == 0) {
#pragma unroll
    for (int h = 0; h < GQA; ++h) { mw[warp * GQA + h] = st.m[h]; lw[warp * GQA + h] = st.l[h]; }
  }
#pragma unroll
  for (int h = 0; h < GQA; ++h)
    *reinterpret_cast<float4*>(aw + (warp * GQA + h) * HD + 4 * lane) =
        make_float4(st.acc[h][0], st.acc[h][1], st.acc[h][2], st.acc[h][3]);
  __syncthreads();
  if (tid < HD) {
    const int d = tid;
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
}

// Fused combine.  Every CTA of one (sequence, KV head) calls this after its record is written.
// Each takes a ticket; the CTA that draws the last one sees all records of that KV head
// (release/acquire through the fences around the ticket), merges them for the head's four
// query heads exactly as decode_combine_kernel does (same order, same operations), and puts
// the counter back to zero for the next call.  `sm` needs GQA*HD floats that are free;
// NTHREADS >= GQA*HD.  Thread tid handles head tid/128, channel tid%128.
template <int NTHREADS>
__device__ __forceinline__ void ticket_combine(const DecodeParams& p, const ShardSeq& sq, int kv, int b,
                                               float* sm_raw, int tid) {
  volatile float* sm = sm_raw;   // exchanged between threads: every access must reach shared memory
  static_assert(NTHREADS >= GQA * HD, "one thread per (head, channel)");
  __shared__ int last_s;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* ctr = p.tickets + b * p.sh.nkv + kv;
    const int last = atomicAdd(ctr, 1) == p.n_parts - 1;
    if (last) atomicExch(ctr, 0);
    last_s = last;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  const bool active = tid < GQA * HD;
  const int n_q = p.sh.n_q, n_parts = p.n_parts, n_rot = p.n_chunks;
  const int h = kv * GQA + ((tid >> 7) & (GQA - 1)), d = tid & (HD - 1);
  const float* base = p.ws + ((size_t)b * n_parts * n_q + h) * PART;
  const size_t pstride = (size_t)n_q * PART;
  float M = neg_inf(), L = 0.f, rot = 0.f, stdv = 0.f;
  if (active) {
#pragma unroll 8
    for (int pi = 0; pi < n_parts; ++pi) M = fmaxf(M, __ldcg(base + pi * pstride));
#pragma unroll 8
    for (int pi = 0; pi < n_parts; ++pi) {
      const float* rec = base + pi * pstride;
      const float m = __ldcg(rec);
      const float l = __ldcg(rec + 1);
      const float a = __ldcg(rec + 4 + d);
      const float wt = (m == neg_inf()) ? 0.f : exp2f((m - M) * LOG2E);
      L = fmaf(wt, l, L);
      if (pi < n_rot) rot = fmaf(wt, a, rot); else stdv = fmaf(wt, a, stdv);
    }
  }
  float v = rot;
  if (n_rot > 0) {
    for (int hh = 1; hh < HD; hh <<= 1) {
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
  if (!active) return;
  const float o = v + stdv;
  if (p.sh.partial_out) {
    float* rec = reinterpret_cast<float*>(sq.out) + (size_t)h * PART;
    if (d == 0) { rec[0] = M; rec[1] = L; rec[2] = 0.f; rec[3] = 0.f; }
    rec[4 + d] = o;
  } else {
    reinterpret_cast<__half*>(sq.out)[(size_t)h * HD + d] = __float2half_rn(o / L);
  }
}

}  // namespace shard
