// Split-KV decode pass on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// One CTA (256 threads, 2 resident per SM) owns one KV head and walks 128-token tiles
// of the compressed middle segment.  Per tile:
//
//   1. unpack   packed int4 coefficients -> fp16 A tile [128 tok x R] in shared memory
//               (K-major core-matrix layout, no swizzle)
//   2. MMA1     K_n[128 tok x 128 dims] = A . W^T  (tcgen05.mma, fp32 accumulators in TMEM;
//               W = basis * coefficient-scale for this KV head, resident in shared memory)
//   3. rotate   each thread owns one token row: TMEM -> registers, + mean, pack to half2,
//               rotate by the relative phase, write K~ (fp16) back to TMEM
//      gather   the same threads expand the token's 32 VQ codes to a [128 tok x 128 ch]
//               fp16 V tile in shared memory (MN-major core-matrix layout; it reuses the
//               A tile's space, which MMA1 has finished reading)
//   4. MMA2     S[128 tok x 16] = K~ . Q^T  (A operand from TMEM, 4 query heads padded to 16)
//   5. softmax  per warp (32 tokens) online softmax; P goes to shared memory as a
//               [16 x 128 tok] operand whose row 4*warp+head holds that warp's weights, so the
//               four warps keep independent running maxima without a CTA-wide reduction
//   6. MMA3     O[128 ch x 16] = V^T . P^T; thread d rescales and accumulates its channel in
//               registers: acc[n] = acc[n] * alpha[n] + O[d][n]
//
// Every wait on an mbarrier is bounded (4096 attempts of <= 10 us): then the CTA raises an abort flag,
// finishes its barriers, frees its tensor memory and reports through the status word.
#include "decode_common.cuh"
#include "tcgen05.cuh"

namespace shard {

constexpr int TC_THREADS = 256;
constexpr int TC_WARPS = 8;
constexpr int TC_TILE = 128;
constexpr int TC_TMEM_COLS = 256;
constexpr int TC_COL_KN = 0;      // [0,128)   fp32 un-rotated keys of the tile (c parts [0,64), d parts [64,128))
constexpr int TC_COL_KR = 0;      // [0,64)    fp16x2 rotated keys, written in place over the c parts
constexpr int TC_COL_S = 64;      // [64,80)   scores, 4 used (over the consumed d parts)
constexpr int TC_COL_O = 80;      // [80,96)   P.V of the tile
constexpr int TC_COL_A = 128;     // [128,224) fp16x2 coefficients of the tile (A operand of MMA1), R/2 columns

// shared-memory carve-up (bytes)
constexpr int TC_V_BYTES = 16 * 2048;
__host__ __device__ constexpr int tc_w_bytes(int nw) { return ((nw + 1) / 2) * 16384; }   // 64-rank atoms of 128 rows x 128 B
constexpr int TC_Q_BYTES = 4096, TC_P_BYTES = 4096, TC_CB_BYTES = 2048, TC_MEAN_BYTES = 512;
constexpr int TC_MISC_BYTES = 1024 + 1024;  // state, barriers + slack for 1 KB alignment  // q copies for row CTAs live elsewhere; see below
__host__ __device__ constexpr int tc_smem_bytes(int nw) {
  return tc_w_bytes(nw) + TC_V_BYTES + TC_Q_BYTES + TC_P_BYTES + TC_CB_BYTES + TC_MEAN_BYTES + TC_MISC_BYTES;
}

#ifdef SHARD_TC_DEBUG
// development aid (never part of the shipped library): stage dumps of CTA (0,0,0), first tile
__device__ float* g_tc_debug = nullptr;
#ifdef SHARD_TC_DUMP
#define TC_DEBUG_ON (g_tc_debug != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tile == tile_lo)
#else
#define TC_DEBUG_ON false
#endif
// per-CTA phase accounting: thread 0 accumulates clock deltas; slot 0 = absolute start, slot 101 = end
#define TC_STAMP(slot)                                                                              \
  do {                                                                                              \
    if (g_tc_debug != nullptr && tid == 0) {                                                        \
      const long long now__ = clock64();                                                            \
      long long* rec__ = reinterpret_cast<long long*>(g_tc_debug + 36000) +                         \
                         32 * (blockIdx.x + gridDim.x * blockIdx.y);                                \
      const int s__ = (slot);                                                                       \
      if (s__ == 0) { rec__[0] = now__; rec__[30] = now__; unsigned sm__; asm("mov.u32 %0, %%smid;" : "=r"(sm__)); rec__[29] = sm__; } \
      else if (s__ == 101) { rec__[28] = now__ - rec__[0]; }                                        \
      else if (s__ >= 2 && s__ < 100) { rec__[1 + ((s__ - 2) & 7)] += now__ - rec__[30]; rec__[30] = now__; } \
      else if (s__ == 1) { rec__[20] = now__ - rec__[30]; rec__[30] = now__; }                      \
      else if (s__ == 100) { rec__[21] += now__ - rec__[30]; rec__[30] = now__; }                   \
    }                                                                                               \
  } while (0)
#else
#define TC_STAMP(slot) do {} while (0)
#endif

// ---------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------
template <int NW>  // rank / 32
__global__ void __launch_bounds__(TC_THREADS, 2) decode_partial_tc_kernel(const __grid_constant__ DecodeParams p) {
  constexpr int R = NW * 32;
  constexpr int KC = R / 8;          // 16-byte chunks per coefficient row (= 32-bit words of nibbles)
  constexpr int KSTEPS = R / 16;     // MMA1 k-steps
  constexpr int W_BYTES = tc_w_bytes(NW);

  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzle atoms need 1 KB alignment
  unsigned char* w_s = smem;                                   // W  [128 x R] fp16, K-major core matrices
  unsigned char* av_s = w_s + W_BYTES;                          // V  [128 tok x 128 ch] fp16, MN-major
  unsigned char* q_s = av_s + TC_V_BYTES;                         // Q  [16 x 128] fp16 (rows 0-3 used)
  unsigned char* p_s = q_s + TC_Q_BYTES;                        // P  [16 x 128 tok] fp16
  uint2* cbv = reinterpret_cast<uint2*>(p_s + TC_P_BYTES);      // V codebook, 256 x (4 x fp16)
  float* mean_s = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(cbv) + TC_CB_BYTES);  // [128]
  float* misc = mean_s + 128;
  float* alpha_s = misc;                                        // [16]
  float* m_s = misc + 16;                                       // [16]
  float* l_s = misc + 32;                                       // [16]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 48);
  volatile int* abort_s = reinterpret_cast<volatile int*>(misc + 49);
  uint64_t* bars = reinterpret_cast<uint64_t*>(misc + 52);      // 3 mbarriers (8-byte aligned)

  const ShardSeq& sq = p.table ? p.table[blockIdx.z] : p.one;
  const ShardDecodeShape& sh = p.sh;
  const int kv = blockIdx.y;
  const int part = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* rec_base = p.ws + (((size_t)blockIdx.z * p.n_parts + part) * sh.n_q + (size_t)kv * GQA) * PART;

  if (part >= p.n_chunks) {
    // ---- sink + window rows, or streamed rows: warp-per-token path ------------------
    float* qn = reinterpret_cast<float*>(smem);                 // [4][128]
    float* qr = qn + GQA * HD;
    float* cbs = qr + GQA * HD;                                 // [256]
    float* scratch = cbs + 256;
    const bool is_fp16 = part < p.n_chunks + p.n_fp16_ctas;
    if (!is_fp16) for (int i = tid; i < 256; i += TC_THREADS) cbs[i] = p.codebook[i];
    if (tid < HD) stage_query(sq, kv, sh.pos_q, p.inv_freq, tid, qn, qr);
    __syncthreads();
    int u_lo = 0, u_hi = sh.n_sink + sh.n_win;
    if (!is_fp16) {
      u_lo = (part - p.n_chunks - p.n_fp16_ctas) * STREAM_TOK_PER_CTA;
      u_hi = min(u_lo + STREAM_TOK_PER_CTA, sh.n_stream);
    }
    SoftmaxState st;
    softmax_init(st);
    process_rows<TC_WARPS>(st, sq, sh, kv, is_fp16, u_lo, u_hi, qr, cbs, warp, lane);
    __syncthreads();
    emit_partial<TC_WARPS>(st, scratch, rec_base, tid, warp, lane);
    return;
  }

  // ---- compressed middle ----------------------------------------------------------------
  TC_STAMP(0);
  const int wg = warp >> 2;              // which half of the per-token work this warp does
  const int quad = warp & 3;             // TMEM lane quadrant = tokens / channels 32*quad ..
  const int m = quad * 32 + lane;        // token row (steps 1-5) or output channel (step 6)
  const uint32_t av_u = smem_u32(av_s), w_u = smem_u32(w_s), q_u = smem_u32(q_s), p_u = smem_u32(p_s);
  const uint32_t bar1 = smem_u32(&bars[0]), bar2 = smem_u32(&bars[1]), bar3 = smem_u32(&bars[2]);

  // one-time setup: W, codebook, mean, Q operand, zeroed P, barriers, tensor memory
  {
    const unsigned char* blob = reinterpret_cast<const unsigned char*>(sq.k_wprep) + (size_t)kv * (W_BYTES + TC_MEAN_BYTES);
    const uint4* src = reinterpret_cast<const uint4*>(blob);
    uint4* dst = reinterpret_cast<uint4*>(w_s);
    for (int i = tid; i < W_BYTES / 16; i += TC_THREADS) dst[i] = src[i];
    if (tid < 128) mean_s[tid] = reinterpret_cast<const float*>(blob + W_BYTES)[tid];
    const uint2* cb_src = reinterpret_cast<const uint2*>(sq.v_centroids);
    cbv[tid] = cb_src[tid];
    uint4* z = reinterpret_cast<uint4*>(q_s);
    for (int i = tid; i < (TC_Q_BYTES + TC_P_BYTES) / 16; i += TC_THREADS) z[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) {
      mbar_init(bar1, 1); mbar_init(bar2, 1); mbar_init(bar3, 1);
      *abort_s = 0;
    }
  }
  __syncthreads();
  if (tid < HD) {
    // un-rotated query of the 4 heads -> Q operand rows 0..3, element k at
    // (k/8)*256 + (n/8)*128 + (n%8)*16 + (k%8)*2
    float qn4[GQA];
    {
      const int d = tid, i = d & 63;
      // contraction position of K~ element (pair i, c or d part): column 32*(i/32) + 16*((i/16)&1) +
      // (i%16)/2 (+8 for the d part), two elements per column
      const int kk = 2 * (32 * (i >> 5) + 16 * ((i >> 4) & 1) + ((i & 15) >> 1) + (d >= 64 ? 8 : 0)) + (i & 1);
      const float phase = __fmul_rn((float)sh.pos_q, p.inv_freq[i]);
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
        *reinterpret_cast<__half*>(q_s + (kk >> 6) * 2048 + sw128_off(h, (kk >> 3) & 7) + (kk & 7) * 2) = un;
        qn4[h] = 0.f;
      }
      (void)qn4;
    }
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), TC_TMEM_COLS);
    tmem_relinquish();
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);

  // operand descriptors of k-step 0; later k-steps add a byte offset (>> 4) to the address field
  const uint64_t wdesc1 = smem_desc_sw128(w_u, 16, 1024);
  const uint64_t qdesc = smem_desc_sw128(q_u, 16, 1024), pdesc = smem_desc_sw128(p_u, 16, 1024);
  const uint64_t vdesc = smem_desc_sw128(av_u, 16384, 1024);
  const uint32_t leader = (lane == 0) ? 1u : 0u;
  constexpr uint32_t IDESC1 = umma_idesc(128, 128, false, false);
  constexpr uint32_t IDESC2 = umma_idesc(128, 16, false, false);
  constexpr uint32_t IDESC3 = umma_idesc(128, 16, true, false);

  const int n_tok = sh.tok_end - sh.tok_begin;
  const int n_tiles = (n_tok + TC_TILE - 1) / TC_TILE;
  const int tile_lo = part * p.tiles_per_chunk;
  const int tile_hi = min(tile_lo + p.tiles_per_chunk, n_tiles);
  const uint32_t* phase_tab = reinterpret_cast<const uint32_t*>(sq.phase);   // row = 32 cos words + 32 sin words
  const uint8_t* vidx = sq.v_indices + (size_t)kv * sh.n_comp * VQ_GROUPS;

  float acc[8];                       // channel m, operand columns n = 8*wg .. 8*wg+7
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  float run_m[GQA], run_l[GQA];       // softmax state of this warp's 32 tokens (wg == 0 warps)
#pragma unroll
  for (int h = 0; h < GQA; ++h) { run_m[h] = neg_inf(); run_l[h] = 0.f; }

  // coefficient words and VQ codes of the first tile; later tiles are prefetched one ahead
  uint2 xpre[NW];
  uint4 codes_pre = make_uint4(0u, 0u, 0u, 0u);
  if (tile_lo < tile_hi) {
    const int tokp = min(sh.tok_begin + tile_lo * TC_TILE + m, sh.tok_end - 1);
    const uint2* row = reinterpret_cast<const uint2*>(sq.k_coeffs + (size_t)tokp * (R / 2)) + wg * NW;
#pragma unroll
    for (int i = 0; i < NW; ++i) xpre[i] = row[i];
    codes_pre = *reinterpret_cast<const uint4*>(vidx + (size_t)tokp * VQ_GROUPS + 16 * wg);
  }

  TC_STAMP(1);
  uint32_t parity = 0;
  for (int tile = tile_lo; tile < tile_hi; ++tile, parity ^= 1u) {
    __syncthreads();
    if (*abort_s) break;
    TC_STAMP(2 + 8 * (tile - tile_lo) + 0);
    const int t0 = sh.tok_begin + tile * TC_TILE;
    const int tok = min(t0 + m, sh.tok_end - 1);
    const bool valid = (t0 + m) < sh.tok_end;

    // ---- 1. unpack this token's coefficient words [wg*KC/2, (wg+1)*KC/2) into tensor memory:
    //         word c -> columns 4c..4c+3 of the A operand, ranks (8c+0,8c+4) (8c+1,8c+5) ... ------
#pragma unroll
    for (int i = 0; i < NW; i += 2) {
      uint32_t o[16];
#pragma unroll
      for (int ii = 0; ii < 2; ++ii) {
        const uint2 x = (i + ii < NW) ? xpre[i + ii] : make_uint2(0x88888888u, 0x88888888u);
        const uint32_t wv[2] = {x.x, x.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          o[8 * ii + 4 * e + 0] = nib2half2_tc(wv[e]);
          o[8 * ii + 4 * e + 1] = nib2half2_tc(wv[e] >> 4);
          o[8 * ii + 4 * e + 2] = nib2half2_tc(wv[e] >> 8);
          o[8 * ii + 4 * e + 3] = nib2half2_tc(wv[e] >> 12);
        }
      }
      if (i + 1 < NW) {
        tmem_st_x16(lane_addr + TC_COL_A + 4 * (wg * (KC / 2) + 2 * i), o);
      } else {
        uint32_t o8[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o8[k] = o[k];
        tmem_st_x8(lane_addr + TC_COL_A + 4 * (wg * (KC / 2) + 2 * i), o8);
      }
    }
    tmem_wait_st();
    const uint4 codes = codes_pre;
    tc_fence_before();
    __syncthreads();
    TC_STAMP(2 + 8 * (tile - tile_lo) + 1);

    // ---- 2. MMA1 ---------------------------------------------------------------------------
    if (warp == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        umma_ts(tmem_base + TC_COL_KN, tmem_base + TC_COL_A + 8 * ks,
                wdesc1 + (uint64_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), IDESC1, ks > 0 ? 1u : 0u, leader);
      }
      umma_commit(bar1, leader);
    }
    // while the tensor core works: phase row of this token (pairs 32*wg .. +31) and the next
    // tile's coefficient words / codes
    uint32_t cos2[16], sin2[16];
    {
      const uint4* prow = reinterpret_cast<const uint4*>(phase_tab + (size_t)(tok - sh.tok_begin) * 64);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 c = prow[wg * 4 + i], sn = prow[8 + wg * 4 + i];
        cos2[4 * i] = c.x; cos2[4 * i + 1] = c.y; cos2[4 * i + 2] = c.z; cos2[4 * i + 3] = c.w;
        sin2[4 * i] = sn.x; sin2[4 * i + 1] = sn.y; sin2[4 * i + 2] = sn.z; sin2[4 * i + 3] = sn.w;
      }
    }
    if (tile + 1 < tile_hi) {
      const int tokp = min(t0 + TC_TILE + m, sh.tok_end - 1);
      const uint2* row = reinterpret_cast<const uint2*>(sq.k_coeffs + (size_t)tokp * (R / 2)) + wg * NW;
#pragma unroll
      for (int i = 0; i < NW; ++i) xpre[i] = row[i];
      codes_pre = *reinterpret_cast<const uint4*>(vidx + (size_t)tokp * VQ_GROUPS + 16 * wg);
    }
    TC_STAMP(2 + 8 * (tile - tile_lo) + 2);
    mbar_wait(bar1, parity, abort_s);
    tc_fence_after();
    TC_STAMP(2 + 8 * (tile - tile_lo) + 3);

    // ---- 3. rotate (pairs 32*wg..+31 of token m, 16 at a time) and gather V -----------------
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t cr[16], dr[16];
      tmem_ld_x16(lane_addr + TC_COL_KN + 32 * wg + 16 * half, cr);
      tmem_ld_x16(lane_addr + TC_COL_KN + 64 + 32 * wg + 16 * half, dr);
      tmem_wait_ld();
#ifdef SHARD_TC_DEBUG
      if (TC_DEBUG_ON) {
        for (int j = 0; j < 16; ++j) {
          g_tc_debug[m * 128 + 32 * wg + 16 * half + j] = __uint_as_float(cr[j]);
          g_tc_debug[m * 128 + 64 + 32 * wg + 16 * half + j] = __uint_as_float(dr[j]);
        }
      }
#endif
      uint32_t oc[8], od[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int pj = 8 * half + j;                    // pair-of-pairs index within this thread's 16
        const float2 mc = *reinterpret_cast<const float2*>(mean_s + 32 * wg + 2 * pj);
        const float2 md = *reinterpret_cast<const float2*>(mean_s + 64 + 32 * wg + 2 * pj);
        const __half2 c2 = __floats2half2_rn(__uint_as_float(cr[2 * j]) + mc.x, __uint_as_float(cr[2 * j + 1]) + mc.y);
        const __half2 d2 = __floats2half2_rn(__uint_as_float(dr[2 * j]) + md.x, __uint_as_float(dr[2 * j + 1]) + md.y);
        const __half2 cs = as_half2(cos2[pj]), sn = as_half2(sin2[pj]);
        oc[j] = as_u32(__hfma2(c2, cs, __hneg2(__hmul2(d2, sn))));   // c cos - d sin
        od[j] = as_u32(__hfma2(d2, cs, __hmul2(c2, sn)));            // d cos + c sin
      }
#ifdef SHARD_TC_DEBUG
      if (TC_DEBUG_ON) {
        for (int j = 0; j < 8; ++j) {
          const float2 a = __half22float2(as_half2(oc[j])), b = __half22float2(as_half2(od[j]));
          const int i0 = 32 * wg + 16 * half + 2 * j;
          g_tc_debug[16384 + m * 128 + i0] = a.x;
          g_tc_debug[16384 + m * 128 + i0 + 1] = a.y;
          g_tc_debug[16384 + m * 128 + 64 + i0] = b.x;
          g_tc_debug[16384 + m * 128 + 64 + i0 + 1] = b.y;
        }
      }
#endif
      // in place: the 16 columns this half just consumed from the c parts take 8 columns of
      // c' (pairs 2 per column) followed by 8 columns of d'
      tmem_st_x8(lane_addr + TC_COL_KR + 32 * wg + 16 * half, oc);
      tmem_st_x8(lane_addr + TC_COL_KR + 32 * wg + 16 * half + 8, od);
    }
    {
      // V tile (MN-major, 128-byte swizzle): two 64-channel halves of 16 KB; token row m is 128 bytes
      const uint32_t cw[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t two = cw[j >> 1] >> (16 * (j & 1));
        const uint2 e0 = cbv[two & 0xff], e1 = cbv[(two >> 8) & 0xff];
        *reinterpret_cast<uint4*>(av_s + wg * 16384 + sw128_off(m, j)) = make_uint4(e0.x, e0.y, e1.x, e1.y);
      }
      tmem_wait_st();
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    TC_STAMP(2 + 8 * (tile - tile_lo) + 4);

    // ---- 4. MMA2: scores -------------------------------------------------------------------
    if (warp == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_ts(tmem_base + TC_COL_S, tmem_base + TC_COL_KR + 8 * ks,
                qdesc + (uint64_t)(((ks >> 2) * 2048 + (ks & 3) * 32) >> 4), IDESC2, ks > 0 ? 1u : 0u, leader);
      umma_commit(bar2, leader);
    }

    // ---- 5. per-warp online softmax (first warp group) --------------------------------------
    if (wg == 0) {
      mbar_wait(bar2, parity, abort_s);
      tc_fence_after();
      uint32_t sraw[4];
      tmem_ld_x4(lane_addr + TC_COL_S, sraw);
      tmem_wait_ld();
#ifdef SHARD_TC_DEBUG
      if (TC_DEBUG_ON) for (int h = 0; h < 4; ++h) g_tc_debug[32768 + m * 4 + h] = __uint_as_float(sraw[h]);
#endif
#pragma unroll
      for (int h = 0; h < GQA; ++h) {
        const float s = valid ? __uint_as_float(sraw[h]) * INV_SQRT_HD : neg_inf();
        const float tm = warp_max(s);
        const float mn = fmaxf(run_m[h], tm);
        const float al = (run_m[h] == neg_inf()) ? 0.f : exp2f((run_m[h] - mn) * LOG2E);
        const float pr = valid ? exp2f((s - mn) * LOG2E) : 0.f;
        run_m[h] = mn;
        run_l[h] = run_l[h] * al + pr;
        const int n = 4 * quad + h;
        *reinterpret_cast<__half*>(p_s + (m >> 6) * 2048 + sw128_off(n, (m >> 3) & 7) + (m & 7) * 2) =
            __float2half_rn(pr);
        if (lane == 0) alpha_s[n] = al;
      }
      fence_proxy_async();
      tc_fence_before();
    }
    __syncthreads();
    TC_STAMP(2 + 8 * (tile - tile_lo) + 5);

    // ---- 6. MMA3: P.V of the tile, then rescale-and-accumulate in registers -----------------
    if (warp == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_ss(tmem_base + TC_COL_O, vdesc + (uint64_t)((ks * 2048) >> 4),
                pdesc + (uint64_t)(((ks >> 2) * 2048 + (ks & 3) * 32) >> 4), IDESC3, ks > 0 ? 1u : 0u, leader);
      umma_commit(bar3, leader);
    }
    mbar_wait(bar3, parity, abort_s);
    tc_fence_after();
    TC_STAMP(2 + 8 * (tile - tile_lo) + 6);
    {
      uint32_t o[8];
      tmem_ld_x8(lane_addr + TC_COL_O + 8 * wg, o);
      tmem_wait_ld();
#ifdef SHARD_TC_DEBUG
      if (TC_DEBUG_ON) for (int j = 0; j < 8; ++j) g_tc_debug[33280 + m * 16 + 8 * wg + j] = __uint_as_float(o[j]);
#endif
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(acc[j], alpha_s[8 * wg + j], __uint_as_float(o[j]));
    }
    tc_fence_before();
    TC_STAMP(2 + 8 * (tile - tile_lo) + 7);
  }
  TC_STAMP(100);

  // ---- epilogue: merge the four token-warps' states per head and emit the record -------------
  __syncthreads();
  if (wg == 0) {
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      const float l = warp_sum(run_l[h]);
      if (lane == 0) { m_s[4 * quad + h] = run_m[h]; l_s[4 * quad + h] = l; }
    }
  }
  float* acc_s = reinterpret_cast<float*>(av_s);                // [16][128]
#pragma unroll
  for (int j = 0; j < 8; ++j) acc_s[(8 * wg + j) * HD + m] = acc[j];
  __syncthreads();
  {
    const float ch = __half2float(reinterpret_cast<const __half*>(sq.v_ch)[kv * HD + m]);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int h = 2 * wg + hh;
      float M = neg_inf();
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, m_s[4 * w + h]);
      float L = 0.f, a = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mv = m_s[4 * w + h];
        const float wt = (mv == neg_inf()) ? 0.f : exp2f((mv - M) * LOG2E);
        L = fmaf(wt, l_s[4 * w + h], L);
        a = fmaf(wt, acc_s[(4 * w + h) * HD + m], a);
      }
      float* rec = rec_base + h * PART;
      if (m == 0) { rec[0] = M; rec[1] = L; rec[2] = 0.f; rec[3] = 0.f; }
      rec[4 + m] = a * ch;
    }
  }
  if (tid == 0 && *abort_s && p.status) atomicExch(p.status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, TC_TMEM_COLS);
  TC_STAMP(101);
}

// prepared weights for this kernel: per KV head, W = basis * coefficient scale as fp16 in the
// K-major core-matrix layout (rank position kk = 8c + p holds rank r = 8c + perm[p], the
// order in which the unpack step emits the nibbles of word c), followed by the mean as fp32.
__global__ void __launch_bounds__(256) decode_prepare_tc_kernel(const __half* __restrict__ basis,
                                                                const __half* __restrict__ cscale,
                                                                const __half* __restrict__ mean, int nkv, int rank,
                                                                unsigned char* __restrict__ out) {
  const int w_bytes = ((rank + 63) / 64) * 16384;
  const int per_kv = w_bytes + TC_MEAN_BYTES;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int total = nkv * HD * rank;
  if (idx < total) {
    const int kk = idx % rank;
    const int j = (idx / rank) % HD;
    const int kv = idx / (rank * HD);
    const int c = kk >> 3, pp = kk & 7;
    const int perm = ((pp & 1) << 2) | (pp >> 1);                // 0,4,1,5,2,6,3,7
    const int r = 8 * c + perm;
    const __half v = __hmul(basis[(size_t)(kv * HD + j) * rank + r], cscale[r]);
    *reinterpret_cast<__half*>(out + (size_t)kv * per_kv + (c >> 3) * 16384 + (j >> 3) * 1024 + (j & 7) * 128 +
                               (((c & 7) ^ (j & 7)) << 4) + pp * 2) = v;
  }
  if (idx < nkv * HD) {
    const int kv = idx / HD, j = idx % HD;
    reinterpret_cast<float*>(out + (size_t)kv * per_kv + w_bytes)[j] = __half2float(mean[idx]);
  }
}

#ifdef SHARD_TC_DEBUG
extern "C" int shard_b200_debug_set(float* buf) {
  return (int)cudaMemcpyToSymbol(g_tc_debug, &buf, sizeof(buf));
}
#endif

size_t tc_wprep_bytes(int nkv, int rank) { return (size_t)nkv * (((rank + 63) / 64) * 16384 + TC_MEAN_BYTES); }

int launch_prepare_tc(const void* basis, const void* cscale, const void* mean, int nkv, int rank, void* out,
                      cudaStream_t st) {
  const int total = nkv * HD * rank;
  decode_prepare_tc_kernel<<<(total + 255) / 256, 256, 0, st>>>((const __half*)basis, (const __half*)cscale,
                                                                 (const __half*)mean, nkv, rank, (unsigned char*)out);
  return 0;
}

template <int NW>
static int launch_tc_one(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  constexpr int SMEM = tc_smem_bytes(NW);
  static_assert(SMEM >= (2 * GQA * HD + 256 + TC_WARPS * GQA * 130) * 4, "row path scratch must fit");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_partial_tc_kernel<NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  decode_partial_tc_kernel<NW><<<grid, TC_THREADS, SMEM, st>>>(p);
  return 0;
}

int launch_partial_tc(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  switch (p.sh.rank / 32) {
    case 1: return launch_tc_one<1>(p, grid, st);
    case 2: return launch_tc_one<2>(p, grid, st);
    case 3: return launch_tc_one<3>(p, grid, st);
    case 4: return launch_tc_one<4>(p, grid, st);
    case 5: return launch_tc_one<5>(p, grid, st);
    default: return launch_tc_one<6>(p, grid, st);
  }
}

}  // namespace shard
