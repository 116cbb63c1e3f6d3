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
  float4 qv[GQA];
#pragma unroll
  for (int h = 0; h < GQA; ++h) qv[h] = *reinterpret_cast<const float4*>(qr + h * HD + 4 * lane);
  auto attend = [&](const float (&kx)[4], const float (&vx)[4]) {
    float s[GQA];
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      float d = qv[h].x * kx[0];
      d = fmaf(qv[h].y, kx[1], d);
      d = fmaf(qv[h].z, kx[2], d);
      s[h] = fmaf(qv[h].w, kx[3], d);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int h = 0; h < GQA; ++h) s[h] += __shfl_xor_sync(0xffffffffu, s[h], o);   // four reductions side by side
    }
#pragma unroll
    for (int h = 0; h < GQA; ++h) s[h] *= INV_SQRT_HD;
    row_update(st, s, vx);
  };
  // ---- fp16 rows: sink, window, fp16 decode buffer ---------------------------------------------
  int u = u_first;
  for (; u < n_fp; u += u_step) {
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
    const float kx[4] = {k01.x, k01.y, k23.x, k23.y}, vx[4] = {v01.x, v01.y, v23.x, v23.y};
    attend(kx, vx);
  }
  // ---- streamed rows (u is this warp's first row behind the fp16 rows) ---------------------------
  if (u >= n_rows) return;
  const float4 sg = *reinterpret_cast<const float4*>(sq.signs + 4 * lane);
  const float sgn[4] = {sg.x, sg.y, sg.z, sg.w};
  // L2-coherent loads: a row may have been written by this CTA a moment ago (fused append).  The
  // next row's codes and norms are fetched while the current row is worked on.
  auto fetch = [&](int ur, uint32_t& kc, uint32_t& vc, unsigned short& kn16, unsigned short& vn16) {
    const size_t row = (size_t)(ur - n_fp) * sh.nkv + kv;
    kn16 = __ldcg(reinterpret_cast<const unsigned short*>(sq.st_k_norm) + row);
    vn16 = __ldcg(reinterpret_cast<const unsigned short*>(sq.st_v_norm) + row);
    kc = __ldcg(reinterpret_cast<const unsigned int*>(sq.st_k_idx + row * HD + 4 * lane));
    vc = __ldcg(reinterpret_cast<const unsigned int*>(sq.st_v_idx + row * HD + 4 * lane));
  };
  uint32_t kc_next = 0u, vc_next = 0u;
  unsigned short kn_next = 0, vn_next = 0;
  fetch(u, kc_next, vc_next, kn_next, vn_next);
  for (; u < n_rows; u += u_step) {
    const uint32_t kc = kc_next, vc = vc_next;
    const float kn = __half2float(__ushort_as_half(kn_next)), vn = __half2float(__ushort_as_half(vn_next));
    if (u + u_step < n_rows) fetch(u + u_step, kc_next, vc_next, kn_next, vn_next);
    // fp16 value of channels 4*lane..+3 exactly as the reference's dequantize_per_token + norm
    // scaling produce it
    float xk[4], xv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xk[i] = cbs[(kc >> (8 * i)) & 0xff];
      xv[i] = cbs[(vc >> (8 * i)) & 0xff];
    }
    fwht128_lane4(xk, lane);
    fwht128_lane4(xv, lane);
    float kx[4], vx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half ku = __float2half_rn(__fmul_rn(__fdiv_rn(xk[i], SQRT_HD), sgn[i]));
      const __half vu = __float2half_rn(__fmul_rn(__fdiv_rn(xv[i], SQRT_HD), sgn[i]));
      kx[i] = __half2float(__float2half_rn(__fmul_rn(__half2float(ku), kn)));
      vx[i] = __half2float(__float2half_rn(__fmul_rn(__half2float(vu), vn)));
    }
    attend(kx, vx);
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
// query heads, and puts the counter back to zero for the next call.  The result does not depend
// on which CTA is last: the parts are always summed in the same order.  `sm` needs 3072 floats
// (or GQA*HD + 2*GQA*n_parts + 8 for more than 64 parts) that are free; NTHREADS >= 512.
//
// The merging CTA is the critical path of the whole launch and runs this code once, out of a
// cold instruction cache: it is kept short.  Warp w < 16 takes query head w % 4 and the parts
// p = w / 4 (mod 4), lane = channels 4*lane .. 4*lane+3: one 16-byte load per part and lane, all of
// a warp's loads in flight together; lane j also fetches (max, sum-exp) of parts j and j + 32, from
// which the warp derives the weights and hands them round by shuffle.  The four partial sums of a
// head meet in shared memory; warp h < 4 adds them in order, runs the inverse Hadamard over the
// 128 channels (two butterflies inside the thread, five by shuffle) and writes the output.
template <int NTHREADS>
__device__ __forceinline__ void ticket_combine(const DecodeParams& p, const ShardSeq& sq, int kv, int b,
                                               float* sm_raw, int tid, bool released = false) {
  volatile float* sm = sm_raw;   // exchanged between threads: every access must reach shared memory
  static_assert(NTHREADS >= GQA * HD, "16 merging warps");
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
  const int n_q = p.sh.n_q, n_parts = p.n_parts, n_rot = p.n_chunks;
  const int w = tid >> 5, lane = tid & 31;
  const float* base0 = p.ws + ((size_t)b * n_parts * n_q + (size_t)kv * GQA) * PART;
  const size_t pstride = (size_t)n_q * PART;
  const bool fin = tid < GQA * 32;                    // warp hl < 4 finishes query head hl
  float M = neg_inf(), L = 0.f;                       // of head w % 4 (the same in every lane)
  float o4[4] = {0.f, 0.f, 0.f, 0.f};                 // channels 4*lane .. 4*lane+3 of head w (fin threads)
  if (n_parts <= 64) {
    float rot4[4] = {0.f, 0.f, 0.f, 0.f}, std4[4] = {0.f, 0.f, 0.f, 0.f};
    if (w < 16) {
      const int hl = w & 3, sub = w >> 2;
      const float* rec0 = base0 + hl * PART;
      constexpr int KB = 5;                            // loads of a batch (18 parts: one batch)
      float4 a[KB];
#pragma unroll
      for (int k = 0; k < KB; ++k) {
        const int pi = sub + 4 * k;
        a[k] = pi < n_parts ? __ldcg(reinterpret_cast<const float4*>(rec0 + pi * pstride + 4) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float mj[2], lj[2], wj[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int pj = lane + 32 * k;
        mj[k] = pj < n_parts ? __ldcg(rec0 + pj * pstride) : neg_inf();
        lj[k] = pj < n_parts ? __ldcg(rec0 + pj * pstride + 1) : 0.f;
      }
      M = warp_max(fmaxf(mj[0], mj[1]));
#pragma unroll
      for (int k = 0; k < 2; ++k) wj[k] = (mj[k] == neg_inf()) ? 0.f : exp2f((mj[k] - M) * LOG2E);
      L = warp_sum(fmaf(wj[0], lj[0], wj[1] * lj[1]));
      for (int k0 = 0; sub + 4 * k0 < n_parts; k0 += KB) {
        if (k0 > 0) {
#pragma unroll
          for (int k = 0; k < KB; ++k) {
            const int pi = sub + 4 * (k0 + k);
            a[k] = pi < n_parts ? __ldcg(reinterpret_cast<const float4*>(rec0 + pi * pstride + 4) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int k = 0; k < KB; ++k) {
          const int pi = sub + 4 * (k0 + k);          // the same in every lane of the warp
          const float wt = __shfl_sync(0xffffffffu, (pi & 32) ? wj[1] : wj[0], pi & 31);
          if (pi < n_parts) {
            float* dst = pi < n_rot ? rot4 : std4;
            dst[0] = fmaf(wt, a[k].x, dst[0]); dst[1] = fmaf(wt, a[k].y, dst[1]);
            dst[2] = fmaf(wt, a[k].z, dst[2]); dst[3] = fmaf(wt, a[k].w, dst[3]);
          }
        }
      }
      if (sub > 0) {
        float4* part4 = reinterpret_cast<float4*>(sm_raw) + ((sub - 1) * GQA + hl) * 64 + lane;
        part4[0] = make_float4(rot4[0], rot4[1], rot4[2], rot4[3]);
        part4[32] = make_float4(std4[0], std4[1], std4[2], std4[3]);
      }
    }
    __syncthreads();
    if (fin) {
#pragma unroll
      for (int sub = 1; sub < 4; ++sub) {
        const float4* part4 = reinterpret_cast<const float4*>(sm_raw) + ((sub - 1) * GQA + w) * 64 + lane;
        const float4 r = part4[0], t = part4[32];
        rot4[0] += r.x; rot4[1] += r.y; rot4[2] += r.z; rot4[3] += r.w;
        std4[0] += t.x; std4[1] += t.y; std4[2] += t.z; std4[3] += t.w;
      }
      if (n_rot > 0) {
        // inverse (= forward) normalised Hadamard over the 128 channels of the head; channel
        // d = 4*lane + c: the butterflies of distance 1 and 2 inside the thread, the others by shuffle
        { const float x0 = rot4[0] + rot4[1], x1 = rot4[0] - rot4[1], x2 = rot4[2] + rot4[3], x3 = rot4[2] - rot4[3];
          rot4[0] = x0 + x2; rot4[1] = x1 + x3; rot4[2] = x0 - x2; rot4[3] = x1 - x3; }
#pragma unroll
        for (int hh = 1; hh < 32; hh <<= 1) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float other = __shfl_xor_sync(0xffffffffu, rot4[c], hh);
            rot4[c] = (lane & hh) ? other - rot4[c] : rot4[c] + other;
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) rot4[c] = rot4[c] / SQRT_HD;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) o4[c] = rot4[c] + std4[c];
    }
  } else {
    // many parts: thread = (head tid / 128, channel tid % 128), (max, sum-exp) of every part of the
    // four heads staged in shared memory, the result handed to the finishing threads through it
    const bool active = tid < GQA * HD;
    const int hl = (tid >> 7) & (GQA - 1), d = tid & (HD - 1);
    volatile float* ms = sm + GQA * HD + 8;             // [GQA][n_parts]
    volatile float* ls = ms + GQA * n_parts;            // [GQA][n_parts]
    for (int idx = tid; idx < GQA * n_parts; idx += NTHREADS) {
      const int hh = idx / n_parts, pi = idx - hh * n_parts;
      const float* rec = base0 + pi * pstride + hh * PART;
      ms[idx] = __ldcg(rec);
      ls[idx] = __ldcg(rec + 1);
    }
    __syncthreads();
    float Mh = neg_inf(), Lh = 0.f, rot = 0.f, stdv = 0.f;
    if (active) {
      for (int pi = 0; pi < n_parts; ++pi) Mh = fmaxf(Mh, ms[hl * n_parts + pi]);
      const float* accp = base0 + hl * PART + 4 + d;
#pragma unroll 4
      for (int pi = 0; pi < n_parts; ++pi) {
        const float a = __ldcg(accp + pi * pstride);
        const float m = ms[hl * n_parts + pi];
        const float wt = (m == neg_inf()) ? 0.f : exp2f((m - Mh) * LOG2E);
        Lh = fmaf(wt, ls[hl * n_parts + pi], Lh);
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
    if (active) {
      sm[tid] = v + stdv;
      if (d == 0) { sm[GQA * HD + hl] = Mh; sm[GQA * HD + GQA + hl] = Lh; }
    }
    __syncthreads();
    if (fin) {
#pragma unroll
      for (int c = 0; c < 4; ++c) o4[c] = sm[w * HD + 4 * lane + c];
      M = sm[GQA * HD + w];
      L = sm[GQA * HD + GQA + w];
    }
  }
  const int h = kv * GQA + w;                          // query head of a finishing thread
  const float4 o = make_float4(o4[0], o4[1], o4[2], o4[3]), ml = make_float4(M, L, 0.f, 0.f);
  if (p.push.world > 0) {
    // Sequence-split decode: this CTA holds the rank's final record of four query heads.  It goes
    // straight into slot epoch % 2 of EVERY rank's exchange buffer (plain peer stores over
    // NVLink), then -- after a system-scope fence by every storing thread -- the epoch number is
    // published in every rank's flag word for (this rank, this KV head).  The merge kernel of
    // each rank waits for those flags.
    const int slot = (int)(p.push.epoch & 1u);
    const size_t flag_bytes = peer_flag_bytes(p.push.world, p.sh.nkv);
    const size_t slot_floats = peer_slot_floats(p.push.world, p.sh.nkv);
    if (fin) {
      for (int r = 0; r < p.push.world; ++r) {
        float4* rec = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.push.bufs[r] + flag_bytes) + slot * slot_floats +
                                                ((size_t)p.push.rank * n_q + h) * PART);
        if (lane == 0) rec[0] = ml;
        rec[1 + lane] = o;
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
      } else if (tid < GQA * HD) {
        const int hq = kv * GQA + (tid >> 7), d = tid & (HD - 1);
        reinterpret_cast<__half*>(p.push.merged_out)[(size_t)hq * HD + d] =
            merge_rank_records(p.push.bufs[p.push.rank], p.push.world, p.sh.nkv, slot, hq, d);
      }
    }
    if (!sq.out) return;
  }
  if (!fin) return;
  if (p.sh.partial_out) {
    float4* rec = reinterpret_cast<float4*>(reinterpret_cast<float*>(sq.out) + (size_t)h * PART);
    if (lane == 0) rec[0] = ml;
    rec[1 + lane] = o;
  } else {
    const __half2 lo = __floats2half2_rn(o4[0] / L, o4[1] / L), hi = __floats2half2_rn(o4[2] / L, o4[3] / L);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    reinterpret_cast<uint2*>(reinterpret_cast<__half*>(sq.out) + (size_t)h * HD)[lane] = pk;
  }
}

}  // namespace shard
