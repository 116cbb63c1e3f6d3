// Fused decode attention over a compressed KV cache (one query token).
//
//   score(h, t) = q_h . RoPE_{pos_t}( W coef_t + mean )        compressed middle
//   score(h, t) = q_h . k_t                                     fp16 sink / window / stream
//   out_h       = softmax_t(score / sqrt(128)) . V_t
//
// Kernels in this file
//   phase_table_kernel    cos/sin(fp32(pos_t - pos_q) * inv_freq) in fp16, shared by all layers
//   decode_prepare_kernel folds the coefficient scale into the PCA basis, appends the
//                         mean as one more contraction column and stores the result in
//                         mma fragment order
//   decode_partial_kernel split-KV pass: every CTA attends to a chunk of tokens for one
//                         KV head (4 query heads) and emits (max, sum-exp, acc[128])
//   decode_combine_kernel log-sum-exp combine of the partials, one inverse Hadamard on
//                         the summed rotated-space part, final normalisation
//
// The middle segment never materialises K: a warp reconstructs the un-rotated keys of
// 16 tokens for one KV head as a [16 x R] x [R x 128] tensor-core product straight from
// the packed int4 coefficients (nibbles are expanded to fp16 in registers), rotates
// them by the relative phase, and dots them with the un-rotated query.
#include <cstdlib>
#include <mutex>

#include "decode_common.cuh"

namespace shard {

constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = 4;
constexpr int TILE_TOK = 16;           // tokens per warp tile of the mma.sync kernel
constexpr int MMA_CTA_SLOTS = 148 * 3; // resident CTAs of the mma.sync kernel on a B200
constexpr int TC_TILE_TOK = 128;       // tokens per tile of the tcgen05 kernel
constexpr int PIPE_CTA_SLOTS = 148;    // the pipelined kernel keeps one CTA per SM
constexpr int WS_STATUS_BYTES = 16;    // status word + padding at the very front of the scratch
// header = status word, then one arrival counter per (sequence, KV head), rounded to 16 bytes
static inline size_t ws_header_bytes(int batch, int nkv) {
  return WS_STATUS_BYTES + (((size_t)batch * nkv * sizeof(int) + 15) & ~(size_t)15);
}

// implemented in decode_pipe.cu
size_t pipe_wprep_bytes(int nkv, int rank);
int launch_prepare_pipe(const void* basis, const void* cscale, const void* mean, int nkv, int rank, void* out,
                        cudaStream_t st);
int launch_partial_pipe(const DecodeParams& p, dim3 grid, cudaStream_t st);

__host__ __device__ inline size_t pipe_blob_bytes(int nkv, int rank) {
  return (size_t)nkv * (((rank + 16 + 63) / 64) * 16384);
}

struct DecodePlan {
  int n_chunks, tiles_per_chunk, tiles_rem, n_fp16_ctas, n_stream_ctas, n_parts;
};

// Which kernel walks the compressed middle: the pipelined tcgen05 kernel (default), or the
// earlier mma.sync kernel kept for A/B timing (environment SHARD_B200_DECODE=mma).
enum DecodeMode { MODE_PIPE = 0, MODE_MMA = 2 };
static DecodeMode decode_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("SHARD_B200_DECODE");
    mode = (e && e[0] == 'm') ? MODE_MMA : MODE_PIPE;
  }
  return (DecodeMode)mode;
}

static DecodePlan make_plan(const ShardDecodeShape& sh, int batch) {
  DecodePlan pl{};
  const DecodeMode mode = decode_mode();
  const int tile_tok = (mode == MODE_MMA) ? TILE_TOK : TC_TILE_TOK;
  const int n_tok = sh.tok_end - sh.tok_begin;
  const int n_tiles = (n_tok + tile_tok - 1) / tile_tok;
  const int groups = sh.nkv * batch;
  if (n_tiles > 0 && mode == MODE_PIPE) {
    // one CTA per SM: spread the tiles of every (sequence, KV head) evenly over its CTAs
    int chunks = (groups >= PIPE_CTA_SLOTS) ? (n_tiles + 15) / 16 : PIPE_CTA_SLOTS / groups;
    if (chunks > n_tiles) chunks = n_tiles;
    if (chunks < 1) chunks = 1;
    pl.n_chunks = chunks;
    pl.tiles_per_chunk = n_tiles / chunks;
    pl.tiles_rem = n_tiles % chunks;
  } else if (n_tiles > 0) {
    int tpc;
    if (groups >= MMA_CTA_SLOTS / 2) {
      tpc = 64;
    } else {
      const int chunks = MMA_CTA_SLOTS / groups;
      tpc = (n_tiles + chunks - 1) / chunks;
      if (tpc < DEC_WARPS) tpc = DEC_WARPS;
    }
    pl.tiles_per_chunk = tpc;
    pl.n_chunks = (n_tiles + tpc - 1) / tpc;
  }
  pl.n_fp16_ctas = (sh.n_sink + sh.n_win) > 0 ? 1 : 0;
  pl.n_stream_ctas = (sh.n_stream + STREAM_TOK_PER_CTA - 1) / STREAM_TOK_PER_CTA;
  pl.n_parts = pl.n_chunks + pl.n_fp16_ctas + pl.n_stream_ctas;
  return pl;
}

// ---------------------------------------------------------------------------
// phase table
// ---------------------------------------------------------------------------
// row t of the table: 64 fp16 cosines (pairs 0..63) followed by 64 fp16 sines
__global__ void __launch_bounds__(256) phase_table_kernel(int delta0, int n, const float* __restrict__ inv_freq,
                                                          __half* __restrict__ out) {
  const size_t total = (size_t)n * HD2;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx >> 6), i = (int)(idx & 63);
    const float phase = __fmul_rn((float)(delta0 + t), inv_freq[i]);
    float sn, cs;
    sincosf(phase, &sn, &cs);
    out[(size_t)t * HD + i] = __float2half_rn(cs);
    out[(size_t)t * HD + HD2 + i] = __float2half_rn(sn);
  }
}

// ---------------------------------------------------------------------------
// prepared weights, fragment order: wprep[kv][ks][nt][lane] = (b0, b1)
//
// Contraction slots are permuted so that a lane can build its A fragments from
// one contiguous R/8-byte piece of the packed coefficient row: lane quad index
// qd owns ranks [R/4*qd, R/4*(qd+1)); 32-bit word w of that piece feeds k-steps
// 2w and 2w+1.  For k-step ks = 2w+s the fragment slots map to
//   slot 2qd   -> r = R/4*qd + 8w + 2s        slot 2qd+1 -> r + 4
//   slot 2qd+8 -> r + 1                       slot 2qd+9 -> r + 5
// The last k-step carries the mean: slot 0 holds mean[row], A supplies 1.0 there.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) decode_prepare_kernel(const __half* __restrict__ basis,
                                                             const __half* __restrict__ cscale,
                                                             const __half* __restrict__ mean, int nkv, int rank,
                                                             uint2* __restrict__ out) {
  const int KD = rank / 16, KS = KD + 1;
  const int total = nkv * KS * 16 * 32;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int lane = idx & 31;
  const int nt = (idx >> 5) & 15;
  const int ks = (idx >> 9) % KS;
  const int kv = (idx >> 9) / KS;
  const int g = lane >> 2, qd = lane & 3;
  const int row = kv * HD + nt * 8 + g;
  __half v[4];
  if (ks < KD) {
    const int w = ks >> 1, s = ks & 1;
    const int r = (rank / 4) * qd + 8 * w + 2 * s;
    const int rr[4] = {r, r + 4, r + 1, r + 5};
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __hmul(basis[(size_t)row * rank + rr[i]], cscale[rr[i]]);
  } else {
    v[0] = (qd == 0) ? mean[row] : __float2half(0.f);
    v[1] = v[2] = v[3] = __float2half(0.f);
  }
  uint2 o;
  o.x = (uint32_t)__half_as_ushort(v[0]) | ((uint32_t)__half_as_ushort(v[1]) << 16);
  o.y = (uint32_t)__half_as_ushort(v[2]) | ((uint32_t)__half_as_ushort(v[3]) << 16);
  out[idx] = o;
}

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// two nibbles (bits 0-3 and 16-19 of y) -> half2 of (nibble - 8)
__device__ __forceinline__ uint32_t nib2half2(uint32_t y) {
  const uint32_t biased = (y & 0x000F000Fu) | 0x64006400u;  // 1024 + nibble
  const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&biased), __half2half2(__ushort_as_half(0x6408)));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// ---------------------------------------------------------------------------
// split-KV pass
// ---------------------------------------------------------------------------
template <int NW>  // 32-bit words of packed coefficients per lane and row = rank / 32
__global__ void __launch_bounds__(DEC_THREADS, 3) decode_partial_kernel(const __grid_constant__ DecodeParams p) {
  constexpr int R = NW * 32;
  constexpr int KD = R / 16;
  constexpr int W_BYTES = (KD + 1) * 16 * 32 * 8;

  extern __shared__ __align__(16) unsigned char smem[];
  uint2* wfrag = reinterpret_cast<uint2*>(smem);                          // W_BYTES (aliased later)
  float* qn = reinterpret_cast<float*>(smem + W_BYTES);                   // [4][128] un-rotated query
  float* qr = qn + GQA * HD;                                              // [4][128] query as given
  uint2* cbv = reinterpret_cast<uint2*>(qr + GQA * HD);                   // [256] V codebook (4 x fp16)
  float* cbs = reinterpret_cast<float*>(cbv + 256);                       // [256] stream codebook
  float4* p_s = reinterpret_cast<float4*>(cbs + 256);                     // [4 warps][16 tokens]
  uint8_t* codes_s = reinterpret_cast<uint8_t*>(p_s + DEC_WARPS * TILE_TOK);  // [4 warps][512]

  const ShardSeq& sq = p.table ? p.table[blockIdx.z] : p.one;
  const ShardDecodeShape& sh = p.sh;
  const int kv = blockIdx.y;
  const int part = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_mid = part < p.n_chunks;
  const bool is_fp16 = !is_mid && part < p.n_chunks + p.n_fp16_ctas;

  // ---- stage per-CTA constants -------------------------------------------
  if (is_mid) {
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(sq.k_wprep) +
                                                      pipe_blob_bytes(sh.nkv, R) + (size_t)kv * W_BYTES);
    uint4* dst = reinterpret_cast<uint4*>(smem);
    for (int i = tid; i < W_BYTES / 16; i += DEC_THREADS) dst[i] = src[i];
    const uint2* cb_src = reinterpret_cast<const uint2*>(sq.v_centroids);
    for (int i = tid; i < 256; i += DEC_THREADS) cbv[i] = cb_src[i];
  } else if (!is_fp16) {
    for (int i = tid; i < 256; i += DEC_THREADS) cbs[i] = p.codebook[i];
  }
  stage_query(sq, kv, sh.pos_q, p.inv_freq, tid, qn, qr);
  __syncthreads();

  SoftmaxState st;
  softmax_init(st);

  if (is_mid) {
    // ---- compressed middle: 16-token tiles, tensor-core K reconstruction -----
    const int g = lane >> 2, qd = lane & 3;
    const int n_tok = sh.tok_end - sh.tok_begin;
    const int n_tiles = (n_tok + TILE_TOK - 1) / TILE_TOK;
    const int tile_lo = part * p.tiles_per_chunk;
    const int tile_hi = min(tile_lo + p.tiles_per_chunk, n_tiles);
    const __half2* phase_tab = reinterpret_cast<const __half2*>(sq.phase);
    const uint8_t* vidx = sq.v_indices + (size_t)kv * sh.n_comp * VQ_GROUPS;
    float4* my_p = p_s + warp * TILE_TOK;
    uint8_t* my_codes = codes_s + warp * (TILE_TOK * VQ_GROUPS);

    for (int tile = tile_lo + warp; tile < tile_hi; tile += DEC_WARPS) {
      const int t0 = sh.tok_begin + tile * TILE_TOK;
      const int tA = t0 + g, tB = t0 + g + 8;
      const bool okA = tA < sh.tok_end, okB = tB < sh.tok_end;
      const int tAc = okA ? tA : sh.tok_end - 1, tBc = okB ? tB : sh.tok_end - 1;

      // V codes of the tile -> shared (16 tokens x 32 bytes, one 16-byte piece per lane)
      {
        const int tv = min(t0 + (lane >> 1), sh.tok_end - 1);
        const uint4 c = *reinterpret_cast<const uint4*>(vidx + (size_t)tv * VQ_GROUPS + 16 * (lane & 1));
        __syncwarp();
        *reinterpret_cast<uint4*>(my_codes + lane * 16) = c;
      }

      // packed coefficients of this lane's two rows
      uint32_t xa[NW], xb[NW];
      {
        const uint32_t* ra = reinterpret_cast<const uint32_t*>(sq.k_coeffs + (size_t)tAc * (R / 2) + (R / 8) * qd);
        const uint32_t* rb = reinterpret_cast<const uint32_t*>(sq.k_coeffs + (size_t)tBc * (R / 2) + (R / 8) * qd);
#pragma unroll
        for (int w = 0; w < NW; ++w) { xa[w] = ra[w]; xb[w] = rb[w]; }
      }

      float acc[16][4];
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }

#pragma unroll
      for (int w = 0; w < NW; ++w) {
#pragma unroll
        for (int s2 = 0; s2 < 2; ++s2) {
          const int ks = 2 * w + s2;
          const uint32_t a0 = nib2half2(xa[w] >> (8 * s2)), a2 = nib2half2(xa[w] >> (8 * s2 + 4));
          const uint32_t a1 = nib2half2(xb[w] >> (8 * s2)), a3 = nib2half2(xb[w] >> (8 * s2 + 4));
          const uint2* wf = wfrag + ks * 512 + lane;
#pragma unroll
          for (int nt = 0; nt < 16; ++nt) {
            const uint2 b = wf[nt * 32];
            mma16816(acc[nt], a0, a1, a2, a3, b.x, b.y);
          }
        }
      }
      {  // mean column: A = 1.0 in slot 0
        const uint32_t one = (qd == 0) ? 0x00003C00u : 0u;
        const uint2* wf = wfrag + KD * 512 + lane;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
          const uint2 b = wf[nt * 32];
          mma16816(acc[nt], one, one, 0u, 0u, b.x, b.y);
        }
      }

      // rotate by the relative phase and dot with the un-rotated query
      float sA[GQA] = {0.f, 0.f, 0.f, 0.f}, sB[GQA] = {0.f, 0.f, 0.f, 0.f};
      const __half2* phA = phase_tab + (size_t)(tAc - sh.tok_begin) * HD2 + qd;   // cos pairs; sines 32 further
      const __half2* phB = phase_tab + (size_t)(tBc - sh.tok_begin) * HD2 + qd;
#pragma unroll
      for (int ntp = 0; ntp < 8; ++ntp) {
        const float2 cosA = __half22float2(phA[4 * ntp]), sinA = __half22float2(phA[32 + 4 * ntp]);
        const float2 cosB = __half22float2(phB[4 * ntp]), sinB = __half22float2(phB[32 + 4 * ntp]);
        float2 qa[GQA], qb[GQA];
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          qa[h] = *reinterpret_cast<const float2*>(qn + h * HD + 8 * ntp + 2 * qd);
          qb[h] = *reinterpret_cast<const float2*>(qn + h * HD + 64 + 8 * ntp + 2 * qd);
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float2 csA = e ? make_float2(cosA.y, sinA.y) : make_float2(cosA.x, sinA.x);
          const float2 csB = e ? make_float2(cosB.y, sinB.y) : make_float2(cosB.x, sinB.x);
          const float cA = acc[ntp][e], dA = acc[ntp + 8][e];
          const float cB = acc[ntp][2 + e], dB = acc[ntp + 8][2 + e];
          const float crA = cA * csA.x - dA * csA.y, drA = dA * csA.x + cA * csA.y;
          const float crB = cB * csB.x - dB * csB.y, drB = dB * csB.x + cB * csB.y;
#pragma unroll
          for (int h = 0; h < GQA; ++h) {
            const float a = e ? qa[h].y : qa[h].x, b = e ? qb[h].y : qb[h].x;
            sA[h] = fmaf(a, crA, fmaf(b, drA, sA[h]));
            sB[h] = fmaf(a, crB, fmaf(b, drB, sB[h]));
          }
        }
      }
#pragma unroll
      for (int h = 0; h < GQA; ++h) {
        sA[h] += __shfl_xor_sync(0xffffffffu, sA[h], 1);
        sB[h] += __shfl_xor_sync(0xffffffffu, sB[h], 1);
        sA[h] += __shfl_xor_sync(0xffffffffu, sA[h], 2);
        sB[h] += __shfl_xor_sync(0xffffffffu, sB[h], 2);
        sA[h] = okA ? sA[h] * INV_SQRT_HD : neg_inf();
        sB[h] = okB ? sB[h] * INV_SQRT_HD : neg_inf();
      }

      // online softmax over the tile
      float pA[GQA], pB[GQA], alpha[GQA];
#pragma unroll
      for (int h = 0; h < GQA; ++h) {
        float tm = fmaxf(sA[h], sB[h]);
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 4));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 16));
        const float mn = fmaxf(st.m[h], tm);  // finite: every tile has at least one valid token
        alpha[h] = (st.m[h] == neg_inf()) ? 0.f : exp2f((st.m[h] - mn) * LOG2E);
        pA[h] = okA ? exp2f((sA[h] - mn) * LOG2E) : 0.f;
        pB[h] = okB ? exp2f((sB[h] - mn) * LOG2E) : 0.f;
        st.m[h] = mn;
        st.l[h] = st.l[h] * alpha[h] + pA[h] + pB[h];  // lane-local; reduced over g at the end
#pragma unroll
        for (int c = 0; c < 4; ++c) st.acc[h][c] *= alpha[h];
      }
      if (qd == 0) {
        my_p[g] = make_float4(pA[0], pA[1], pA[2], pA[3]);
        my_p[g + 8] = make_float4(pB[0], pB[1], pB[2], pB[3]);
      }
      __syncwarp();

      // P.V in the rotated domain: lane owns VQ group `lane` (channels 4*lane..+3)
#pragma unroll 4
      for (int tt = 0; tt < TILE_TOK; ++tt) {
        const float4 pw = my_p[tt];
        const uint2 ent = cbv[my_codes[tt * VQ_GROUPS + lane]];
        const float2 v01 = __half22float2(*reinterpret_cast<const __half2*>(&ent.x));
        const float2 v23 = __half22float2(*reinterpret_cast<const __half2*>(&ent.y));
        const float pv[GQA] = {pw.x, pw.y, pw.z, pw.w};
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          st.acc[h][0] = fmaf(pv[h], v01.x, st.acc[h][0]);
          st.acc[h][1] = fmaf(pv[h], v01.y, st.acc[h][1]);
          st.acc[h][2] = fmaf(pv[h], v23.x, st.acc[h][2]);
          st.acc[h][3] = fmaf(pv[h], v23.y, st.acc[h][3]);
        }
      }
      __syncwarp();
    }
    // lane-local l -> warp total (quad lanes hold identical copies: reduce over g only)
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 4);
      st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 8);
      st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 16);
    }
    // per-channel scale of the rotated V
    const uint2 chraw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(sq.v_ch) + kv * HD + 4 * lane);
    const float2 ch01 = __half22float2(*reinterpret_cast<const __half2*>(&chraw.x));
    const float2 ch23 = __half22float2(*reinterpret_cast<const __half2*>(&chraw.y));
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      st.acc[h][0] *= ch01.x; st.acc[h][1] *= ch01.y; st.acc[h][2] *= ch23.x; st.acc[h][3] *= ch23.y;
    }
  } else {
    int u_lo = 0, u_hi = sh.n_sink + sh.n_win;
    if (!is_fp16) {
      u_lo = (part - p.n_chunks - p.n_fp16_ctas) * STREAM_TOK_PER_CTA;
      u_hi = min(u_lo + STREAM_TOK_PER_CTA, sh.n_stream);
    }
    process_rows<DEC_WARPS>(st, sq, sh, kv, is_fp16, u_lo, u_hi, qr, cbs, warp, lane);
  }

  // ---- merge the 4 warps and emit this CTA's partial -------------------------
  __syncthreads();  // all reads of the W fragments are done; reuse that space
  float* rec_base = p.ws + (((size_t)blockIdx.z * p.n_parts + part) * sh.n_q + (size_t)kv * GQA) * PART;
  emit_partial<DEC_WARPS>(st, reinterpret_cast<float*>(smem), rec_base, tid, warp, lane);
}

// ---------------------------------------------------------------------------
// combine: one CTA per (query head, sequence); thread d owns output channel d
// parts [0, n_rot) carry rotated-space accumulators, the rest standard space
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(HD) decode_combine_kernel(const float* __restrict__ ws, int n_parts, int n_rot,
                                                            int n_q, int partial_out, void* const* out_table,
                                                            void* out_single) {
  __shared__ float sm[HD];
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const float* base = ws + ((size_t)b * n_parts * n_q + h) * PART;
  const size_t pstride = (size_t)n_q * PART;
  float M = neg_inf();
  for (int pi = 0; pi < n_parts; ++pi) M = fmaxf(M, base[pi * pstride]);
  float L = 0.f, rot = 0.f, stdv = 0.f;
  for (int pi = 0; pi < n_parts; ++pi) {
    const float* rec = base + pi * pstride;
    const float m = rec[0];
    const float wt = (m == neg_inf()) ? 0.f : exp2f((m - M) * LOG2E);
    L = fmaf(wt, rec[1], L);
    const float a = rec[4 + d];
    if (pi < n_rot) rot = fmaf(wt, a, rot); else stdv = fmaf(wt, a, stdv);
  }
  // inverse (= forward) normalised Hadamard of the rotated-space sum
  float v = rot;
  if (n_rot > 0) {
    for (int hh = 1; hh < HD; hh <<= 1) {
      sm[d] = v;
      __syncthreads();
      const float other = sm[d ^ hh];
      v = (d & hh) ? other - v : v + other;
      __syncthreads();
    }
    v = v / SQRT_HD;
  }
  const float o = v + stdv;
  void* out = out_table ? out_table[b] : out_single;
  if (partial_out) {
    float* rec = reinterpret_cast<float*>(out) + (size_t)h * PART;
    if (d == 0) { rec[0] = M; rec[1] = L; rec[2] = 0.f; rec[3] = 0.f; }
    rec[4 + d] = o;
  } else {
    reinterpret_cast<__half*>(out)[(size_t)h * HD + d] = __float2half_rn(o / L);
  }
}

// tiny helper for batched launches: gather the out pointers of a device ShardSeq table
__global__ void gather_out_ptrs_kernel(const ShardSeq* table, int batch, void** out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < batch) out[i] = table[i].out;
}

template <int NW>
static int launch_partial(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  constexpr int W_BYTES = (NW * 2 + 1) * 16 * 32 * 8;
  constexpr int SMEM = W_BYTES + 2 * GQA * HD * 4 + 256 * 8 + 256 * 4 + DEC_WARPS * TILE_TOK * 16 +
                       DEC_WARPS * TILE_TOK * VQ_GROUPS;
  static_assert(SMEM >= (2 * DEC_WARPS * GQA + DEC_WARPS * GQA * HD) * 4, "merge area must fit");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_partial_kernel<NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  decode_partial_kernel<NW><<<grid, DEC_THREADS, SMEM, st>>>(p);
  return 0;
}

}  // namespace shard

using namespace shard;

extern "C" int shard_b200_phase_table(int32_t compress_start, int32_t pos_q, int32_t n_comp, const float* inv_freq,
                                      void* out, void* stream) {
  if (!inv_freq || !out || n_comp < 0) return SHARD_E_ARG;
  if (n_comp == 0) return SHARD_OK;
  const size_t total = (size_t)n_comp * HD2;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  phase_table_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(compress_start - pos_q, n_comp, inv_freq,
                                                                (__half*)out);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

// blob = [tcgen05 operand layout: nkv x W atoms (mean folded in)] [mma.sync fragment layout]
static size_t mma_wprep_bytes(int nkv, int rank) { return (size_t)nkv * (rank / 16 + 1) * 16 * 32 * 8; }

extern "C" size_t shard_b200_wprep_bytes(int32_t nkv, int32_t rank) {
  if (nkv < 1 || rank < 32 || rank > 192 || (rank % 32)) return 0;
  return pipe_wprep_bytes(nkv, rank) + mma_wprep_bytes(nkv, rank);
}

extern "C" int shard_b200_decode_prepare(const void* basis_f16, const void* coeff_scale, const void* mean_f16,
                                         int32_t nkv, int32_t rank, void* wprep_out, void* stream) {
  if (!basis_f16 || !coeff_scale || !mean_f16 || !wprep_out) return SHARD_E_ARG;
  if (nkv < 1 || rank < 32 || rank > 192 || (rank % 32)) return SHARD_E_ARG;
  if ((uintptr_t)wprep_out & 15) return SHARD_E_ALIGN;
  int prc = launch_prepare_pipe(basis_f16, coeff_scale, mean_f16, nkv, rank, wprep_out, (cudaStream_t)stream);
  if (prc) return prc;
  const int total = nkv * (rank / 16 + 1) * 16 * 32;
  decode_prepare_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      (const __half*)basis_f16, (const __half*)coeff_scale, (const __half*)mean_f16, nkv, rank,
      (uint2*)((unsigned char*)wprep_out + pipe_wprep_bytes(nkv, rank)));
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

static int check_shape(const ShardDecodeShape* sh) {
  if (!sh) return SHARD_E_ARG;
  if (sh->nkv < 1 || sh->n_q != sh->nkv * GQA) return SHARD_E_ARG;
  if (sh->rank < 32 || sh->rank > 192 || (sh->rank % 32)) return SHARD_E_ARG;
  if (sh->n_comp < 0 || sh->tok_begin < 0 || sh->tok_end < sh->tok_begin || sh->tok_end > sh->n_comp)
    return SHARD_E_ARG;
  if (sh->n_sink < 0 || sh->n_win < 0 || sh->n_stream < 0) return SHARD_E_ARG;
  if ((sh->tok_end - sh->tok_begin) + sh->n_sink + sh->n_win + sh->n_stream <= 0) return SHARD_E_ARG;
  return SHARD_OK;
}

// scratch layout: header (status word, arrival counters; zero between calls),
// [batch][n_parts][n_q][132] fp32 partial records, then (batch > 1) `batch` out pointers
static size_t ws_bytes(const ShardDecodeShape& sh, int batch) {
  const DecodePlan pl = make_plan(sh, batch);
  size_t b = ws_header_bytes(batch, sh.nkv) + (size_t)batch * pl.n_parts * sh.n_q * PART * sizeof(float);
  if (batch > 1) b += (size_t)batch * sizeof(void*);
  return b;
}

extern "C" size_t shard_b200_decode_workspace_bytes(const ShardDecodeShape* shape_host, int32_t batch) {
  if (batch < 1 || check_shape(shape_host) != SHARD_OK) return 0;
  return ws_bytes(*shape_host, batch);
}

extern "C" int shard_b200_decode_attn(const ShardSeq* seqs, int32_t batch, const ShardDecodeShape* shape_host,
                                      const float* inv_freq, const float* codebook, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  if (!seqs || batch < 1 || !inv_freq || !workspace) return SHARD_E_ARG;
  int rc = check_shape(shape_host);
  if (rc != SHARD_OK) return rc;
  const ShardDecodeShape& sh = *shape_host;
  if (sh.n_stream > 0 && !codebook) return SHARD_E_ARG;
  if (sh.append && (sh.n_stream < 1 || (batch == 1 && (!seqs->new_k || !seqs->new_v)))) return SHARD_E_ARG;
  if ((uintptr_t)workspace & 15) return SHARD_E_ALIGN;
  if (workspace_bytes < ws_bytes(sh, batch)) return SHARD_E_WORKSPACE;
  const DecodePlan pl = make_plan(sh, batch);
  cudaStream_t st = (cudaStream_t)stream;

  DecodeParams p{};
  if (batch == 1) {
    p.one = *seqs;
    p.table = nullptr;
    const ShardSeq& s = p.one;
    if (!s.q || !s.out) return SHARD_E_ARG;
    if (sh.tok_end > sh.tok_begin &&
        (!s.k_coeffs || !s.k_wprep || !s.v_indices || !s.v_centroids || !s.v_ch || !s.phase))
      return SHARD_E_ARG;
    if (sh.n_sink > 0 && (!s.sink_k || !s.sink_v)) return SHARD_E_ARG;
    if (sh.n_win > 0 && (!s.win_k || !s.win_v)) return SHARD_E_ARG;
    if (sh.n_stream > 0 && (!s.st_k_idx || !s.st_v_idx || !s.st_k_norm || !s.st_v_norm || !s.signs))
      return SHARD_E_ARG;
    if (((uintptr_t)s.k_coeffs & 3) || ((uintptr_t)s.k_wprep & 15) || ((uintptr_t)s.v_indices & 15) ||
        ((uintptr_t)s.v_centroids & 7) || ((uintptr_t)s.phase & 7) || ((uintptr_t)s.sink_k & 7) ||
        ((uintptr_t)s.sink_v & 7) || ((uintptr_t)s.win_k & 7) || ((uintptr_t)s.win_v & 7) ||
        ((uintptr_t)s.st_k_idx & 3) || ((uintptr_t)s.st_v_idx & 3) || ((uintptr_t)s.signs & 15) ||
        ((uintptr_t)s.v_ch & 7))
      return SHARD_E_ALIGN;
  } else {
    p.table = seqs;
  }
  const size_t header = ws_header_bytes(batch, sh.nkv);
  p.sh = sh;
  p.inv_freq = inv_freq;
  p.codebook = codebook;
  p.ws = (float*)((unsigned char*)workspace + header);
  p.status = (int*)workspace;
  p.tickets = (int*)((unsigned char*)workspace + WS_STATUS_BYTES);
  p.n_chunks = pl.n_chunks;
  p.tiles_per_chunk = pl.tiles_per_chunk;
  p.tiles_rem = pl.tiles_rem;
  p.n_fp16_ctas = pl.n_fp16_ctas;
  p.n_stream_ctas = pl.n_stream_ctas;
  p.n_parts = pl.n_parts;

  dim3 grid(pl.n_parts, sh.nkv, batch);
  if (decode_mode() == MODE_PIPE) {
    // one launch: the append (if asked for), the split-KV pass and the combine
    if (batch == 1 && ((uintptr_t)p.one.k_coeffs & 15)) return SHARD_E_ALIGN;
    rc = launch_partial_pipe(p, grid, st);
    if (rc) return rc;
    SHARD_CHECK_LAUNCH();
    return SHARD_OK;
  } else {
    if (sh.append) {
      rc = shard_b200_stream_quantize(seqs, batch, sh.nkv, sh.n_stream - 1, codebook, stream);
      if (rc) return rc;
    }
    switch (sh.rank / 32) {
      case 1: rc = launch_partial<1>(p, grid, st); break;
      case 2: rc = launch_partial<2>(p, grid, st); break;
      case 3: rc = launch_partial<3>(p, grid, st); break;
      case 4: rc = launch_partial<4>(p, grid, st); break;
      case 5: rc = launch_partial<5>(p, grid, st); break;
      default: rc = launch_partial<6>(p, grid, st); break;
    }
  }
  if (rc) return rc;
  SHARD_CHECK_LAUNCH();

  void** out_table = nullptr;
  if (batch > 1) {
    out_table = reinterpret_cast<void**>(reinterpret_cast<unsigned char*>(workspace) + header +
                                         (size_t)batch * pl.n_parts * sh.n_q * PART * sizeof(float));
    gather_out_ptrs_kernel<<<(batch + 127) / 128, 128, 0, st>>>(seqs, batch, out_table);
  }
  decode_combine_kernel<<<dim3(sh.n_q, batch), HD, 0, st>>>(p.ws, pl.n_parts, pl.n_chunks, sh.n_q, sh.partial_out,
                                                            out_table, batch == 1 ? p.one.out : nullptr);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" int shard_b200_lse_merge(const float* parts, int32_t n_parts, int32_t n_q, void* out_f16, void* stream) {
  if (!parts || !out_f16 || n_parts < 1 || n_q < 1) return SHARD_E_ARG;
  decode_combine_kernel<<<dim3(n_q, 1), HD, 0, (cudaStream_t)stream>>>(parts, n_parts, 0, n_q, 0, nullptr, out_f16);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

// ---------------------------------------------------------------------------
// Decode entry point for callers that cannot allocate device memory
// ---------------------------------------------------------------------------
// The split-KV pass needs a few hundred KB of scratch for its per-chunk partial records.
// The regular entry point takes that scratch from the caller.  Some callers have no way
// to provide it: an inference server that fixes its whole device-memory plan at start-up
// and forbids any later cudaMalloc (so a request can never fail or fragment memory half
// way through), or a host application that only hands this library its tensors and
// exposes no allocator at all.  For them the library carries one fixed scratch area
// inside its own device image.  It costs SHARD_B200_STATIC_SCRATCH_BYTES on every GPU
// that loads the library, for as long as the process lives.
static __device__ __align__(256) unsigned char g_static_scratch[SHARD_B200_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};   // device address of the array, per device
std::mutex g_static_scratch_mutex;

// `g_static_scratch` names a host-side handle here, not device memory: the address a kernel
// can use has to be asked from the runtime, once per device, with that device current.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return SHARD_E_ARG;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_addr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return SHARD_OK;
}
}  // namespace

extern "C" int shard_b200_decode_attn_noalloc(const ShardSeq* seq_host, const ShardDecodeShape* shape_host,
                                              const float* inv_freq, const float* codebook, void* stream) {
  if (!seq_host || !inv_freq) return SHARD_E_ARG;
  int rc = check_shape(shape_host);
  if (rc != SHARD_OK) return rc;
  const size_t need = ws_bytes(*shape_host, 1);
  if (need > (size_t)SHARD_B200_STATIC_SCRATCH_BYTES) return SHARD_E_TOO_LARGE;
  void* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch);
  if (rc != SHARD_OK) return rc;
  // The array still holds whatever the previous call left there.  Only the header (status
  // word and arrival counters) has to start at zero; every partial record is rewritten
  // before it is read.
  cudaError_t e = cudaMemsetAsync(scratch, 0, ws_header_bytes(1, shape_host->nkv), (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return shard_b200_decode_attn(seq_host, 1, shape_host, inv_freq, codebook, scratch,
                                (size_t)SHARD_B200_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int shard_b200_abi_version(void) { return 1; }

extern "C" const char* shard_b200_status_string(int status) {
  switch (status) {
    case SHARD_OK: return "ok";
    case SHARD_E_ARG: return "invalid argument (null pointer, bad size or unsupported geometry)";
    case SHARD_E_WORKSPACE: return "workspace too small";
    case SHARD_E_ALIGN: return "pointer not aligned as documented";
    case SHARD_E_TOO_LARGE: return "request needs more scratch than the library's built-in 2 MiB area";
    default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
  }
}
