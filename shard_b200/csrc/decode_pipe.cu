// One decode step of one layer in one launch: split-KV pass over the compressed middle
// (tcgen05 + tensor memory + bulk copy engine, warp-specialised, three tiles in flight per SM),
// the fp16 / streamed rows, the stream append and the combine.
//
// One CTA per SM (16 warps) owns one KV head and a run of 128-token tiles of the middle segment.
//
//   copy engine         the weights W once; per tile the packed int4 coefficient rows (two buffers,
//                       two tiles ahead) and the V codes (one buffer per consumer group) land in
//                       shared memory and are announced on mbarriers -- no load instruction touches
//                       the cache data
//   unpack warps (4)    coefficient rows -> fp16 A operand in tensor memory (one A slot, handed back
//                       by MMA1 in thirds so that the next tile's unpack overlaps its later k-steps);
//                       in their slack at the end: this CTA's share of the fp16 sink / window rows
//                       and the streamed rows (dequantised on the fly), transformed into the rotated
//                       space of the middle's accumulator and handed to the epilogue
//   consumer groups (3 x 4 warps; group g owns V / P slot g and tiles g, g+3, ...), thread = token
//                       row; one thread per group issues all tensor-core work of the group:
//                       MMA1  K_n[128 tok x 128] = A . W^T           (A from TMEM, W in smem; the last
//                             k-step adds the mean), for the tile two ahead
//                       K_n -> half2 -> rotate by the relative phase -> K~ written in place
//                       MMA2  S[128 tok x 16]    = K~ . Q^T          (A = K~ from TMEM)
//                       meanwhile the token's 32 VQ codes are expanded into the group's V tile
//                       per-warp online softmax with a lazily moving reference point -> P
//                       MMA3  O[128 ch x 16]    += V^T . P^T         (V, P in smem; accumulates in
//                             tensor memory, rescaled only when a reference point moved)
//   append              in the CTA that owns the newest streamed row two warps of the last consumer
//                       group quantise the new token while its other two stage the query
//   epilogue            the 12 token-warps' states and the rows' state merge into ONE record per CTA
//   combine             the last CTA of a (sequence, KV head) to finish merges all records
//
// Launched with programmatic stream serialization: the set-up, the first tiles' unpack,
// reconstruction products, rotation and V expansion use only tensors that no decode call writes
// (and the phase table, complete before a launch can start) and run before griddepcontrol.wait.
//
// Tensor memory: two key stages of 128 columns (tile t uses stage t % 2: un-rotated keys in fp32,
// overwritten in place by K~ as fp16x2 in columns 0-63 of the stage), the A operand at [256, 360),
// and per consumer group 16 columns of scores and 16 of P.V accumulator from column 360 on.
// Every hand-over is an mbarrier whose waiters see each of its phases; every wait is bounded and
// raises the CTA's abort flag when it gives up, after which all roles drain, bulk copies in flight
// are waited for, tensor memory is freed and the status word is set.
#include <atomic>
#include <cstdlib>

#include "decode_common.cuh"
#include "tcgen05.cuh"

namespace shard {

constexpr int PP_STAGES = 3;
constexpr int PP_CONS_WARPS = 12;
constexpr int PP_UNPACK_WARP0 = 12;
constexpr int PP_WARPS = 16;
constexpr int PP_THREADS = PP_WARPS * 32;
constexpr int PP_TMEM_COLS = 512;
// tensor memory: two key stages of 128 columns, the A operand slot (R/2 coefficient columns + 8
// constant columns 1, 0, ...), and per consumer group 16 columns of scores + 16 of P.V accumulator
constexpr int PP_COL_A = 256;
constexpr int PP_COL_SO = 360;
constexpr float PP_LAZY_LOG2 = 8.f;   // a softmax reference point moves only when exceeded by more than 2^8
constexpr int PP_V_BYTES = 32768, PP_P_BYTES = 4096, PP_Q_BYTES = 4096;
constexpr int PP_CB_COPIES = 4;       // interleaved copies of the V codebook: lane l reads copy l % 4, entry e of copy c at 4e + c
constexpr int PP_CB_BYTES = 2048 * PP_CB_COPIES;
constexpr int PP_ROWQ_BYTES = (GQA * HD + 256) * 4;   // queries as given + stream codebook, for the row path
constexpr int PP_MISC_BYTES = 1024 + 1024;   // state + barriers, and slack for 1 KB alignment

// W holds R + 16 contraction positions (the last 16 carry the mean), in 64-position atoms of 16 KB
__host__ __device__ constexpr int pp_w_bytes(int nw) { return ((32 * nw + 16 + 63) / 64) * 16384; }
// staging filled by the bulk copy engine: two tiles of packed coefficients (128 rows x R/2 bytes)
// and one tile of V codes (128 rows x 32 bytes) per consumer group
// (at least 5312 bytes each, so that the pair can double as the 8.3 KB row-merge scratch plus the
// 2.1 KB record of the rows)
__host__ __device__ constexpr int pp_c_bytes(int nw) { return 128 * 16 * nw < 5312 ? 5312 : 128 * 16 * nw; }
constexpr int PP_VC_BYTES = 128 * VQ_GROUPS;
__host__ __device__ constexpr int pp_smem_bytes(int nw) {
  return pp_w_bytes(nw) + PP_STAGES * (PP_V_BYTES + PP_P_BYTES) + PP_Q_BYTES + PP_CB_BYTES + PP_ROWQ_BYTES +
         2 * pp_c_bytes(nw) + PP_STAGES * PP_VC_BYTES + PP_MISC_BYTES;
}

// single-thread forms (the caller is one elected thread)
__device__ __forceinline__ void umma_ss_1t(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_ts_1t(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit_1t(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Plain barrier among a subset of the CTA's warps (id 1..15, `count` threads).
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// The same barrier, also ORing a flag over the participants.  The roles use it to agree on giving
// up: a warp whose bounded wait failed never leaves its siblings alone at a barrier -- everybody
// reaches the barrier, learns the combined flag and leaves the tile loop together.
__device__ __forceinline__ bool named_bar_or(int id, int count, bool flag) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %3, 0;\n\t"
      "bar.red.or.pred p, %1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out) : "r"(id), "r"(count), "r"((uint32_t)flag) : "memory");
  return out != 0;
}


// A launch without a middle segment (a cache that holds fp16 and streamed rows only): every CTA
// attends to its share of the rows (row u belongs to CTA u % gridDim.x, one warp per row), the CTA
// that owns the newest streamed row quantises it first, the last CTA of a KV head combines.
constexpr int ROWS_THREADS = 512;
constexpr int ROWS_SMEM_BYTES = (2 * GQA * HD + 256 + (ROWS_THREADS / 32) * GQA * 130) * 4;
__global__ void __launch_bounds__(ROWS_THREADS, 1) decode_rows_only_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(128) unsigned char smem_rows[];
  const ShardSeq& sq = p.table ? p.table[blockIdx.z] : p.one;
  const ShardDecodeShape& sh = p.sh;
  const int kv = blockIdx.y, part = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rows = sh.n_sink + sh.n_win + sh.n_dec + sh.n_stream;
  const bool append_here = sh.append && p.n_row_parts > 0 && (n_rows - 1) % p.n_row_parts == part;
  float* rec_rows = p.ws + (((size_t)blockIdx.z * p.n_parts + part) * sh.n_q + (size_t)kv * GQA) * PART;
  griddep_launch();
  griddep_wait();
  float* qn = reinterpret_cast<float*>(smem_rows);
  float* qr = qn + GQA * HD;
  float* cbs = qr + GQA * HD;
  float* scratch = cbs + 256;
  if (sh.n_stream > 0) for (int i = tid; i < 256; i += ROWS_THREADS) cbs[i] = p.codebook[i];
  if (tid < HD) stage_query(sq, kv, sh.pos_q, p.inv_freq, tid, qn, qr);
  __syncthreads();
  if (append_here) {
    if (warp < 2) append_new_token(sq, sh, kv, cbs, warp == 1, lane);
    __syncthreads();
  }
  SoftmaxState st;
  softmax_init(st);
  process_rows(st, sq, sh, kv, part + p.n_row_parts * warp, p.n_row_parts * (ROWS_THREADS / 32), qr, cbs, lane);
  partial_store<ROWS_THREADS / 32>(st, scratch, warp, lane);
  __syncthreads();
  if (tid < HD) partial_merge<ROWS_THREADS / 32>(scratch, rec_rows, tid);
  ticket_combine<ROWS_THREADS>(p, sq, kv, blockIdx.z, scratch, tid);
}

template <int NW>  // rank / 32
__global__ void __launch_bounds__(PP_THREADS, 1) decode_partial_pipe_kernel(const __grid_constant__ DecodeParams p) {
  constexpr int R = NW * 32;
  constexpr int KSTEPS = R / 16 + 1;   // + one step whose A columns are (1, 0, ...) and whose W slice is the mean
  constexpr int W_BYTES = pp_w_bytes(NW);
  constexpr int W_ATOMS = W_BYTES / 16384;
  constexpr int NSUB = (NW + 1) / 2;   // thirds of the A slot: 4 k-steps (64 ranks) each

  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* w_s = smem;
  unsigned char* v_s = w_s + W_BYTES;                              // [3] V tiles, MN-major, 128B swizzle
  unsigned char* p_s = v_s + PP_STAGES * PP_V_BYTES;               // [3] P operands [16 x 128 tok]
  unsigned char* q_s = p_s + PP_STAGES * PP_P_BYTES;               // Q operand [16 x 128]
  uint2* cbv = reinterpret_cast<uint2*>(q_s + PP_Q_BYTES);         // V codebook
  float* qr_s = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(cbv) + PP_CB_BYTES);   // queries as given [4][128]
  float* cbs_s = qr_s + GQA * HD;                                  // stream codebook [256]
  unsigned char* c_s = reinterpret_cast<unsigned char*>(cbs_s + 256);         // [2] coefficient tiles
  float* rows_rec_s = reinterpret_cast<float*>(c_s) + 4 * GQA * 130;   // record of this CTA's rows (valid once the coefficient buffers are free)
  unsigned char* vc_s = c_s + 2 * pp_c_bytes(NW);                  // [3] V code tiles
  float* misc = reinterpret_cast<float*>(vc_s + PP_STAGES * PP_VC_BYTES);
  float* alpha_s = misc;                                           // [3][16]
  float* m_s = misc + 48;                                          // [3][16]
  float* l_s = misc + 96;                                          // [3][16]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 144);
  volatile int* abort_s = reinterpret_cast<volatile int*>(misc + 145);
  volatile int* c_cnt = reinterpret_cast<volatile int*>(misc + 146);   // [2] coefficient tiles requested per buffer
  volatile int* mma1_next = reinterpret_cast<volatile int*>(misc + 208);   // next tile whose MMA1 is to be issued
  uint64_t* bars = reinterpret_cast<uint64_t*>(misc + 148);        // 29 mbarriers

  const ShardSeq& sq = p.table ? p.table[blockIdx.z] : p.one;
  const ShardDecodeShape& sh = p.sh;
  const int kv = blockIdx.y;
  const int part = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* rec_base = p.ws + (((size_t)blockIdx.z * p.n_parts + part) * sh.n_q + (size_t)kv * GQA) * PART;

  const int n_rows = sh.n_sink + sh.n_win + sh.n_dec + sh.n_stream;
  // the CTA that owns the newest streamed row quantises it before anybody reads the stream
  const bool append_here = sh.append && p.n_row_parts > 0 && (n_rows - 1) % p.n_row_parts == part;

  griddep_launch();

  // barrier addresses
  const uint32_t bar0 = smem_u32(bars);
  auto KN_FULL = [&](int g) { return bar0 + 8u * (uint32_t)g; };          // MMA1 of group g's next tile done
  auto S_FULL = [&](int g) { return bar0 + 8u * (uint32_t)(3 + g); };     // MMA2 done
  auto O_DONE = [&](int g) { return bar0 + 8u * (uint32_t)(6 + g); };     // MMA3 done (V tile, P and O of the group are free / final)
  auto A_EMPTY = [&](int j) { return bar0 + 8u * (uint32_t)(12 + j); };   // MMA1 has read third j of the A slot
  auto A_FULL = [&](int j) { return bar0 + 8u * (uint32_t)(25 + j); };    // third j of the next tile's A operand is in place
  auto W_FULL = [&](int a) { return bar0 + 8u * (uint32_t)(15 + a); };    // atom a (64 contraction positions) of the weights has landed
  auto C_FULL = [&](int b) { return bar0 + 8u * (uint32_t)(19 + b); };    // coefficient tile has landed
  auto V_FULL = [&](int g) { return bar0 + 8u * (uint32_t)(21 + g); };    // V code tile has landed
  const uint32_t APPEND_DONE = bar0 + 8u * 24u;                           // the newest streamed row has been written
  const uint32_t Q_READY = bar0 + 8u * 28u;                               // the query operand and the fp32 queries are staged

  // tiles of this chunk: evenly spread, the first `tiles_rem` chunks get one more
  const int tile_lo = part * p.tiles_per_chunk + min(part, p.tiles_rem);
  const int n_my = p.tiles_per_chunk + (part < p.tiles_rem ? 1 : 0);
  // bulk copies of tile `it` of this chunk: its packed coefficient rows into buffer it % 2, its
  // V codes into the buffer of consumer group it % 3.  The last tile of the segment may be
  // short; the rows behind it keep whatever the buffer held (any byte pattern decodes to finite
  // values, and those rows get zero weight).
  auto issue_coef = [&](int it) {
    const int t0 = sh.tok_begin + (tile_lo + it) * 128;
    const uint32_t bytes = (uint32_t)min(128, sh.tok_end - t0) * (uint32_t)(R / 2);
    mbar_expect_tx(C_FULL(it & 1), bytes);
    bulk_g2s(smem_u32(c_s + (it & 1) * pp_c_bytes(NW)), sq.k_coeffs + (size_t)t0 * (R / 2), bytes, C_FULL(it & 1));
  };
  auto issue_vcodes = [&](int it) {
    const int t0 = sh.tok_begin + (tile_lo + it) * 128, g = it % PP_STAGES;
    const uint32_t bytes = (uint32_t)min(128, sh.tok_end - t0) * (uint32_t)VQ_GROUPS;
    mbar_expect_tx(V_FULL(g), bytes);
    bulk_g2s(smem_u32(vc_s + g * PP_VC_BYTES), sq.v_indices + ((size_t)kv * sh.n_comp + t0) * VQ_GROUPS, bytes,
             V_FULL(g));
  };

  // ---- one-time set-up, first part: tensor memory, mbarriers, the first bulk copies ---------------
  if (warp == PP_UNPACK_WARP0) {
    tmem_alloc(smem_u32(tmem_slot), PP_TMEM_COLS);
    tmem_relinquish();
  }
  if (tid == 0) {
    // first the barriers of the bulk copies, so that the copy engine starts as early as possible:
    // the first coefficient tile, the weights atom by atom (the first k-steps only need the first
    // atom), the second coefficient tile and the first V code tile of every consumer group
    mbar_init(C_FULL(0), 1); mbar_init(C_FULL(1), 1);
    for (int a = 0; a < W_ATOMS; ++a) mbar_init(W_FULL(a), 1);
    for (int g = 0; g < PP_STAGES; ++g) mbar_init(V_FULL(g), 1);
    c_cnt[0] = n_my > 0 ? 1 : 0; c_cnt[1] = n_my > 1 ? 1 : 0;
    fence_mbar_init();
    if (n_my > 0) issue_coef(0);
    for (int a = 0; a < W_ATOMS; ++a) {
      mbar_expect_tx(W_FULL(a), 16384u);
      bulk_g2s(smem_u32(w_s + a * 16384), reinterpret_cast<const unsigned char*>(sq.k_wprep) + (size_t)kv * W_BYTES + a * 16384,
               16384u, W_FULL(a));
    }
    if (n_my > 1) issue_coef(1);
    for (int j = 0; j < min(PP_STAGES, n_my); ++j) issue_vcodes(j);
  } else if (tid == 32) {
    for (int s = 0; s < PP_STAGES; ++s) {
      mbar_init(KN_FULL(s), 1); mbar_init(S_FULL(s), 1); mbar_init(O_DONE(s), 1); mbar_init(A_EMPTY(s), 1);
    }
    *mma1_next = 0;
    for (int j = 0; j < 3; ++j) mbar_init(A_FULL(j), 4);
    mbar_init(APPEND_DONE, 2);
    mbar_init(Q_READY, 2);
    *abort_s = 0;
    fence_mbar_init();
  }
  // (one CTA barrier for what everybody needs: tensor memory, the mbarriers, the copies in flight)
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  float run_m[GQA], run_l[GQA];
#pragma unroll
  for (int h = 0; h < GQA; ++h) { run_m[h] = neg_inf(); run_l[h] = 0.f; }

  if (warp < PP_CONS_WARPS) {
    // =============================== consumer groups ======================================
    const int g = warp >> 2, quad = warp & 3, m = quad * 32 + lane;
    // Second part of the set-up, by the consumer warps alone -- the unpack warps are already at
    // work on the first tile: the codebooks into shared memory, zeros where they have to stay.
    if (tid < 256) {
      const uint2 e = reinterpret_cast<const uint2*>(sq.v_centroids)[tid];
#pragma unroll
      for (int c = 0; c < PP_CB_COPIES; ++c) cbv[PP_CB_COPIES * tid + c] = e;
    } else if (sh.n_stream > 0) {
      for (int i = tid - 256; i < 256; i += 128) cbs_s[i] = p.codebook[i];
    }
    {
      // P rows that a token's warp does not own stay zero for the whole kernel, and so do rows 4..15
      // of the Q operand (it follows the P operands in memory)
      uint4* z = reinterpret_cast<uint4*>(p_s);
      for (int i = tid; i < (PP_STAGES * PP_P_BYTES + PP_Q_BYTES) / 16; i += PP_CONS_WARPS * 32) z[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async();
    named_bar_sync(5, PP_CONS_WARPS * 32);
    // the MMA-issuing threads of the CTA (one per consumer group + the unpack side's) sit on four
    // different warp schedulers: group g issues from its warp g + 1, the unpack side from warp 12
    const int issuer_quad = g + 1;
    const uint32_t SO_g = tmem_base + (uint32_t)(PP_COL_SO + 32 * g);      // scores at +0, P.V accumulator at +16
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    constexpr uint32_t IDESC2 = umma_idesc(128, 16, false, false);
    constexpr uint32_t IDESC3 = umma_idesc(128, 16, true, false);
    const uint64_t qdesc = smem_desc_sw128(smem_u32(q_s), 16, 1024);
    const uint64_t vdesc = smem_desc_sw128(smem_u32(v_s + g * PP_V_BYTES), 16384, 1024);
    const uint64_t pdesc = smem_desc_sw128(smem_u32(p_s + g * PP_P_BYTES), 16, 1024);
    unsigned char* v_g = v_s + g * PP_V_BYTES;
    unsigned char* p_g = p_s + g * PP_P_BYTES;
    float* alpha_g = alpha_s + 16 * g;
    const uint4* phase_tab = reinterpret_cast<const uint4*>(sq.phase);
    const unsigned char* vc_g = vc_s + g * PP_VC_BYTES;
    int vc_issued = g < n_my ? 1 : 0;        // V code tiles requested for this group so far
    const bool issuer = quad == issuer_quad && lane == 0;
    // MMA1 of tile t: K_n[128 tok x 128] = A . W^T into key stage t % 2, issued third by third of the A
    // slot as the unpack warps fill it, each third handed back as soon as its k-steps have run.
    // Issued by a consumer group's issuing thread: tiles 0 and 1 at the start, tile t >= 2 by the
    // thread that has just issued the scores product of tile t - 2 out of the same key stage (one
    // thread's tensor-core instructions run in issue order, so the stage is not overwritten early).
    // `mma1_next` keeps the issuing threads in tile order.  A k-step of 128 columns holds its
    // issuing thread for about as long as the previous one runs (about 900 cycles per tile), which
    // is why the issuing thread's warp takes no part in expanding the V codes: its three sibling
    // warps do that for all 128 tokens meanwhile.
    constexpr uint32_t IDESC1 = umma_idesc(128, 128, false, false);
    const uint64_t wdesc = smem_desc_sw128(smem_u32(w_s), 16, 1024);
    auto issue_mma1 = [&](int t) -> bool {
      int spins = 0;
      while (*mma1_next != t) {
        if (++spins > (1 << 20) || *abort_s) { *abort_s = 1; return false; }
        __nanosleep(32);
      }
      const uint32_t T_t = tmem_base + (uint32_t)(128 * (t & 1));
#pragma unroll
      for (int j = 0; j < NSUB; ++j) {
        if (!mbar_wait(A_FULL(j), (uint32_t)(t & 1), abort_s)) return false;
        if (t == 0) {                                             // only the very first MMA1 can be ahead of the weights
          if (!mbar_wait(W_FULL(j), 0u, abort_s)) return false;
          if (j == NSUB - 1 && W_ATOMS > NSUB && !mbar_wait(W_FULL(W_ATOMS - 1), 0u, abort_s)) return false;
        }
        tc_fence_after();
        const int ks_hi = (j == NSUB - 1) ? KSTEPS : 4 * j + 4;
#pragma unroll
        for (int ks = 4 * j; ks < 4 * j + 5; ++ks) {
          if (ks < ks_hi)
            umma_ts_1t(T_t, tmem_base + PP_COL_A + 8 * ks, wdesc + (uint64_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4),
                       IDESC1, ks > 0 ? 1u : 0u);
        }
        umma_commit_1t(A_EMPTY(j));
      }
      umma_commit_1t(KN_FULL(t % PP_STAGES));
      if (t + 2 < n_my) { issue_coef(t + 2); c_cnt[t & 1] = c_cnt[t & 1] + 1; }   // the unpack warps are done with that buffer
      *mma1_next = t + 1;
      return true;
    };
    // gather work of the three non-issuing warps: 512 units of (token row, 8 codes), 96 threads
    const int gq = quad - (quad > issuer_quad ? 1 : 0);        // 0..2 among the gathering warps
    const int gather_first = gq * 32 + lane;
    const uint2* cbv4 = cbv + (lane & (PP_CB_COPIES - 1));   // this lane's copy of the codebook (fewer bank conflicts)

    // 256 units of (token row, 16 codes) over the 96 threads of the three non-issuing warps;
    // consecutive lanes take consecutive rows, so the eight 16-byte stores of a quarter-warp fall
    // into eight different bank groups of the swizzled tile
    auto gather_tile = [&]() {
#pragma unroll 1
      for (int u = gather_first; u < 256; u += 96) {
        const int row = u & 127, hf = u >> 7;              // codes 16*hf .. 16*hf+15 of the row
        const uint4 cq = *reinterpret_cast<const uint4*>(vc_g + row * VQ_GROUPS + 16 * hf);
        const uint32_t cw[4] = {cq.x, cq.y, cq.z, cq.w};
        unsigned char* dst = v_g + hf * 16384;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const uint32_t two = cw[jj >> 1] >> (16 * (jj & 1));
          const uint2 e0 = cbv4[4 * (two & 0xff)], e1 = cbv4[4 * ((two >> 8) & 0xff)];
          *reinterpret_cast<uint4*>(dst + sw128_off(row, jj)) = make_uint4(e0.x, e0.y, e1.x, e1.y);
        }
      }
    };

    bool bad = false;
    if (issuer && g < 2 && g < n_my) bad |= !issue_mma1(g);
    __syncwarp();
    // the V codes of the group's first tile are cache data as well: expanded while waiting
    if (g < n_my && quad != issuer_quad) {
      bad |= !mbar_wait(V_FULL(g), 0u, abort_s);
      gather_tile();
    }
    // Up to here only tensors that no decode call ever writes were touched (weights, coefficients,
    // V codes, codebooks): the set-up, the first two tiles' unpack and reconstruction products run
    // while the launch before this one is still finishing.  The query, the new token, the stream
    // rows, the scratch and the output may come from, or still be in use by, that launch: every
    // role waits for it before it touches them.  (The phase table is complete before any CTA of this
    // launch starts: the kernel that writes it never releases its dependents early.  So the first
    // two groups also rotate their first tile before they wait.)
    // The last consumer group -- whose first tile is the furthest away -- has two jobs here: its
    // first two warps stage the query (the cos / sin of the query position do not depend on the
    // launch before), and in the CTA that owns the newest streamed row its other two quantise the
    // new token into it meanwhile (bit-identical to stream_quantize_kernel).  The row is read near
    // the end of the kernel by the unpack warps, which wait on APPEND_DONE first.
    const bool stages_q = g == PP_STAGES - 1 && quad < 2;
    __half c16 = __float2half_rn(1.f), s16 = __float2half_rn(0.f);
    if (stages_q) {
      const float phase = __fmul_rn((float)sh.pos_q, p.inv_freq[tid - 256]);
      float sn, cs;
      sincosf(phase, &sn, &cs);
      c16 = __float2half_rn(cs); s16 = __float2half_rn(sn);
    }
    if (g == PP_STAGES - 1) griddep_wait();
    if (stages_q) {
      // un-rotated query (fp16 arithmetic as the reference) -> Q operand rows 0..3 (rows 4..15 stay
      // zero); element of pair i (c or d part) sits at the contraction position of the in-place K~
      // layout: column 8*(i/8) + (i%8)/2 (+4 for the d part), two elements per column.  This thread
      // takes pair i: dimensions i and i + 64.
      const int i = tid - 256;
      const __half* qg = reinterpret_cast<const __half*>(sq.q) + (size_t)kv * GQA * HD;
      __half x_lo[GQA], x_hi[GQA];
#pragma unroll
      for (int h = 0; h < GQA; ++h) { x_lo[h] = qg[h * HD + i]; x_hi[h] = qg[h * HD + i + 64]; }
#pragma unroll
      for (int part2 = 0; part2 < 2; ++part2) {
        const int d = i + 64 * part2;
        const int kk = 2 * (8 * (i >> 3) + ((i & 7) >> 1) + (part2 ? 4 : 0)) + (i & 1);
        unsigned char* qcol = q_s + (kk >> 6) * 2048 + (kk & 7) * 2;
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          const __half x = part2 ? x_hi[h] : x_lo[h];
          const __half rot = part2 ? x_lo[h] : __hneg(x_hi[h]);
          const __half un = __hsub(__hmul(x, c16), __hmul(rot, s16));
          *reinterpret_cast<__half*>(qcol + sw128_off(h, (kk >> 3) & 7)) = un;
          qr_s[h * HD + d] = __half2float(x);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(Q_READY);
    } else if (append_here && g == PP_STAGES - 1) {
      append_new_token(sq, sh, kv, cbs_s, quad == 3, lane);
      __syncwarp();
      if (lane == 0) mbar_arrive(APPEND_DONE);
    }
    int use = 0;
    for (int it = g; it < n_my; it += PP_STAGES, ++use) {
      const uint32_t par = (uint32_t)(use & 1);
      const uint32_t T_s = tmem_base + (uint32_t)(128 * (it & 1));   // key stage of this tile
      const uint32_t lane_T = T_s + lane_off;
      const int t0 = sh.tok_begin + (tile_lo + it) * 128;
      const int tok = min(t0 + m, sh.tok_end - 1);
      const bool valid = (t0 + m) < sh.tok_end;
      // cos/sin of the row: plane c of the token's block of 32 holds 8 pairs for each of its tokens,
      // so a warp reads 512 contiguous bytes per plane; kept three chunks ahead of use
      const int tl = tok - sh.tok_begin;
      const uint4* prow = phase_tab + (size_t)(tl >> 5) * 512 + (tl & 31);
      uint4 pc[8], ps[8];
      pc[0] = prow[0 * 32]; ps[0] = prow[8 * 32];
      pc[1] = prow[1 * 32]; ps[1] = prow[9 * 32];
      pc[2] = prow[2 * 32]; ps[2] = prow[10 * 32];

      bad |= !mbar_wait(KN_FULL(g), par, abort_s);
      tc_fence_after();

      // ---- rotate: 8 chunks of 8 pairs; K~ goes back in place --------------------------------
      // chunk ch reads c columns [8ch, 8ch+8) and d columns [64+8ch, ...) and writes 4 columns of c'
      // and 4 of d' (two pairs per column) over the 8 c columns it has just consumed
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        uint32_t cr[8], dr[8];
        tmem_ld_x8(lane_T + 8 * ch, cr);
        tmem_ld_x8(lane_T + 64 + 8 * ch, dr);
        if (ch + 3 < 8) { pc[ch + 3] = prow[(ch + 3) * 32]; ps[ch + 3] = prow[(8 + ch + 3) * 32]; }
        const uint32_t cos2[4] = {pc[ch].x, pc[ch].y, pc[ch].z, pc[ch].w};
        const uint32_t sin2[4] = {ps[ch].x, ps[ch].y, ps[ch].z, ps[ch].w};
        tmem_wait_ld();
        uint32_t oc[4], od[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __half2 c2 = __floats2half2_rn(__uint_as_float(cr[2 * j]), __uint_as_float(cr[2 * j + 1]));
          const __half2 d2 = __floats2half2_rn(__uint_as_float(dr[2 * j]), __uint_as_float(dr[2 * j + 1]));
          const __half2 cs = as_half2(cos2[j]), sn = as_half2(sin2[j]);
          oc[j] = as_u32(__hfma2(c2, cs, __hneg2(__hmul2(d2, sn))));   // c cos - d sin
          od[j] = as_u32(__hfma2(d2, cs, __hmul2(c2, sn)));            // d cos + c sin
        }
        tmem_st_x4(lane_T + 8 * ch, oc);
        tmem_st_x4(lane_T + 8 * ch + 4, od);
      }
      tmem_wait_st();
      tc_fence_before();
      bad = named_bar_or(1 + g, 128, bad || *abort_s);
      if (bad) break;                                   // uniform over the group
      if (use == 0) griddep_wait();                     // (the last group has waited already)
      if (issuer) {
        if (use == 0) bad |= !mbar_wait(Q_READY, 0u, abort_s);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts_1t(SO_g, T_s + 8 * ks, qdesc + (uint64_t)(((ks >> 2) * 2048 + (ks & 3) * 32) >> 4), IDESC2,
                     ks > 0 ? 1u : 0u);
        umma_commit_1t(S_FULL(g));
        if (it + 2 < n_my) bad |= !issue_mma1(it + 2);  // the same key stage, behind the scores product
      }
      __syncwarp();
      // (while the tensor core computes the scores)
      // ---- gather the token's V row (32 codes) into the group's V tile ---------------------------
      // the previous tile's P.V product must have finished reading the V tile and P
      // (the first tile's were expanded before the loop)
      if (use > 0) {
        bad |= !mbar_wait(O_DONE(g), (uint32_t)((use - 1) & 1), abort_s);
        bad |= !mbar_wait(V_FULL(g), par, abort_s);
        if (quad != issuer_quad) gather_tile();
      }

      // ---- softmax over this warp's 32 tokens ---------------------------------------------------
      // The reference point of a (warp, head) only moves when the tile's maximum exceeds it by more
      // than 2^PP_LAZY_LOG2 (weights then stay below that factor, far inside fp16 range): the
      // accumulator in tensor memory is rescaled only in those rare tiles.
      bad |= !mbar_wait(S_FULL(g), par, abort_s);
      tc_fence_after();
      {
        uint32_t sraw[4];
        tmem_ld_x4(SO_g + lane_off, sraw);
        tmem_wait_ld();
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          const float s2 = valid ? __uint_as_float(sraw[h]) * (INV_SQRT_HD * LOG2E) : neg_inf();   // log2 domain
          const float tm = warp_max(s2);
          float al = 1.f;
          if (tm > run_m[h] + PP_LAZY_LOG2) {            // also the first tile with a valid token (run_m = -inf)
            al = (run_m[h] == neg_inf()) ? 0.f : exp2f(run_m[h] - tm);
            run_m[h] = tm;
          }
          const float pr = valid ? exp2f(s2 - run_m[h]) : 0.f;
          run_l[h] = run_l[h] * al + pr;
          const int n = 4 * quad + h;
          *reinterpret_cast<__half*>(p_g + (m >> 6) * 2048 + sw128_off(n, (m >> 3) & 7) + (m & 7) * 2) = __float2half_rn(pr);
          if (lane == 0) alpha_g[n] = al;
        }
      }
      fence_proxy_async();
      tc_fence_before();
      bad = named_bar_or(1 + g, 128, bad || *abort_s);
      if (bad) break;                                   // uniform over the group
      if (use > 0) {
        // rescale channel m of the accumulator where a reference point moved (same decision in
        // every thread of the group: all read the same 16 factors)
        float al[16];
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const float4 a4 = *reinterpret_cast<const float4*>(alpha_g + 4 * j4);
          al[4 * j4] = a4.x; al[4 * j4 + 1] = a4.y; al[4 * j4 + 2] = a4.z; al[4 * j4 + 3] = a4.w;
        }
        bool moved = false;
#pragma unroll
        for (int j = 0; j < 16; ++j) moved |= al[j] != 1.f;
        if (moved) {
          uint32_t o[16];
          tmem_ld_x16(SO_g + 16 + lane_off, o);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * al[j]);
          tmem_st_x16(SO_g + 16 + lane_off, o);
          tmem_wait_st();
          tc_fence_before();
          named_bar_sync(1 + g, 128);
        }
      }
      if (issuer) {
        if (it + PP_STAGES < n_my) { issue_vcodes(it + PP_STAGES); ++vc_issued; }   // every lane has read its codes
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss_1t(SO_g + 16, vdesc + (uint64_t)((ks * 2048) >> 4),
                     pdesc + (uint64_t)(((ks >> 2) * 2048 + (ks & 3) * 32) >> 4), IDESC3, (ks > 0 || use > 0) ? 1u : 0u);
        umma_commit_1t(O_DONE(g));
      }
      __syncwarp();
    }
    griddep_wait();                                     // a group without tiles, or one that gave up early
    // the group's accumulated P.V: channel m, 16 (warp, head) columns
    if (use > 0 && !(bad || *abort_s)) {
      bad |= !mbar_wait(O_DONE(g), (uint32_t)((use - 1) & 1), abort_s);
      tc_fence_after();
      if (!bad) {
        uint32_t o[16];
        tmem_ld_x16(SO_g + 16 + lane_off, o);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = __uint_as_float(o[j]);
      }
    }
    // giving up: do not leave while a copy this thread asked for may still be landing
    if ((bad || *abort_s) && issuer && vc_issued > 0)
      mbar_wait(V_FULL(g), (uint32_t)((vc_issued - 1) & 1), abort_s);
  } else {
    // =============================== unpack warps =========================================
    const int quad = warp - PP_UNPACK_WARP0, m = quad * 32 + lane;
    const uint32_t lane_A = tmem_base + PP_COL_A + ((uint32_t)(quad * 32) << 16);
    {
      // constant part of the A operand: position R is 1.0 (it multiplies the mean slice of W)
      const uint32_t ones[8] = {0x00003C00u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      tmem_st_x8(lane_A + R / 2, ones);
    }
    bool bad = false;
    for (int it = 0; it < n_my && !bad; ++it) {
      bad = !mbar_wait(C_FULL(it & 1), (uint32_t)((it >> 1) & 1), abort_s);
      const uint4* row = reinterpret_cast<const uint4*>(c_s + (it & 1) * pp_c_bytes(NW) + m * (R / 2));
#pragma unroll
      for (int j = 0; j < NSUB; ++j) {
        // third j of the slot is free once the previous tile's MMA1 has run its k-steps over it
        if (it > 0) bad |= !mbar_wait(A_EMPTY(j), (uint32_t)((it - 1) & 1), abort_s);
        bad = __any_sync(0xffffffffu, bad || *abort_s);
        if (bad) break;                                 // uniform over the warp
        tc_fence_after();
#pragma unroll
        for (int i = 2 * j; i < 2 * j + 2 && i < NW; ++i) {
          const uint4 xi = row[i];
          const uint32_t wv[4] = {xi.x, xi.y, xi.z, xi.w};
          uint32_t o[16];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t hi = wv[e] >> 8;
            o[4 * e + 0] = nib2half2_tc(wv[e]);          // ranks 8c+0, 8c+4 of word c = 4i+e
            o[4 * e + 1] = nib2half2_hi(wv[e]);          //       8c+1, 8c+5
            o[4 * e + 2] = nib2half2_tc(hi);             //       8c+2, 8c+6
            o[4 * e + 3] = nib2half2_hi(hi);             //       8c+3, 8c+7
          }
          tmem_st_x16(lane_A + 16 * i, o);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(A_FULL(j));          // this warp's rows of the third are in place
      }
    }
    // The unpack warps run about three tiles ahead of the consumers.  In that slack they take this
    // CTA's share of the fp16 / streamed rows (row u belongs to CTA u % n_row_parts), one warp per
    // row.  The rows get a record of their own: standard V space, while the middle's record is in rotated space.
    // The coefficient staging buffers are free by now and serve as merge scratch.
    bad = named_bar_or(4, 128, bad || *abort_s);
    griddep_wait();
    if (!bad && p.n_row_parts > 0) {
      bad = !mbar_wait(Q_READY, 0u, abort_s);
      if (append_here) bad |= !mbar_wait(APPEND_DONE, 0u, abort_s);
      SoftmaxState st;
      softmax_init(st);
      if (!bad) process_rows(st, sq, sh, kv, part + p.n_row_parts * quad, p.n_row_parts * 4, qr_s, cbs_s, lane);
      float* scratch = reinterpret_cast<float*>(c_s);
      partial_store<4>(st, scratch, quad, lane);
      named_bar_sync(4, 128);
      partial_merge<4>(scratch, rows_rec_s, m);
      // Into the rotated space of the middle's accumulator (normalised Hadamard over the channels of
      // each head; the combine's inverse transform takes it back): the CTA then has one record.
      float v[GQA];
#pragma unroll
      for (int h = 0; h < GQA; ++h) v[h] = rows_rec_s[h * PART + 4 + m];
#pragma unroll
      for (int hh = 1; hh < 32; hh <<= 1) {
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          const float other = __shfl_xor_sync(0xffffffffu, v[h], hh);
          v[h] = (m & hh) ? other - v[h] : v[h] + other;
        }
      }
      for (int hh = 32; hh < HD; hh <<= 1) {
        named_bar_sync(4, 128);
#pragma unroll
        for (int h = 0; h < GQA; ++h) rows_rec_s[h * PART + 4 + m] = v[h];
        named_bar_sync(4, 128);
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          const float other = rows_rec_s[h * PART + 4 + (m ^ hh)];
          v[h] = (m & hh) ? other - v[h] : v[h] + other;
        }
      }
      named_bar_sync(4, 128);
#pragma unroll
      for (int h = 0; h < GQA; ++h) rows_rec_s[h * PART + 4 + m] = v[h] / SQRT_HD;
    } else {
      // no rows for this launch (or gave up): an empty state
#pragma unroll
      for (int h = 0; h < GQA; ++h) {
        if (m == 0) { rows_rec_s[h * PART] = neg_inf(); rows_rec_s[h * PART + 1] = 0.f; }
        rows_rec_s[h * PART + 4 + m] = 0.f;
      }
    }
  }

  // ---- epilogue: merge the 12 token-warps' states per head and emit the record -------------------
  // every consumer group parks its state in its own V tile (its last MMA3 has completed), so one
  // CTA barrier separates the tile loops from the merge
  const float ch_scale = __half2float(reinterpret_cast<const __half*>(sq.v_ch)[kv * HD + (tid & 127)]);
  if (warp < PP_CONS_WARPS) {
    const int g = warp >> 2, quad = warp & 3, m = quad * 32 + lane;
    float* acc_g = reinterpret_cast<float*>(v_s + g * PP_V_BYTES);   // [16][128]
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      const float l = warp_sum(run_l[h]);
      if (lane == 0) { m_s[16 * g + 4 * quad + h] = run_m[h]; l_s[16 * g + 4 * quad + h] = l; }
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) acc_g[j * HD + m] = acc[j];
  }
  __syncthreads();
  {
    // run_m is kept in the log2 domain (score * log2 e); the record carries the natural-log maximum
    const int h = tid >> 7, m = tid & 127;              // 512 threads: one (head, channel) each
    // the rows' state (natural-log reference, already in rotated space and final units)
    const float rows_m = rows_rec_s[h * PART] * LOG2E, rows_l = rows_rec_s[h * PART + 1], rows_a = rows_rec_s[h * PART + 4 + m];
    float M = rows_m;
#pragma unroll
    for (int e = 0; e < 12; ++e) M = fmaxf(M, m_s[16 * (e >> 2) + 4 * (e & 3) + h]);
    float L = 0.f, a = 0.f;
#pragma unroll
    for (int e = 0; e < 12; ++e) {
      const int idx = 16 * (e >> 2) + 4 * (e & 3) + h;
      const float mv = m_s[idx];
      const float wt = (mv == neg_inf()) ? 0.f : exp2f(mv - M);
      L = fmaf(wt, l_s[idx], L);
      a = fmaf(wt, reinterpret_cast<const float*>(v_s + (e >> 2) * PP_V_BYTES)[(4 * (e & 3) + h) * HD + m], a);
    }
    const float wr = (rows_m == neg_inf()) ? 0.f : exp2f(rows_m - M);
    L = fmaf(wr, rows_l, L);
    float* rec = rec_base + h * PART;
    if (m == 0) { rec[0] = M * LN2; rec[1] = L; rec[2] = 0.f; rec[3] = 0.f; }
    rec[4 + m] = fmaf(wr, rows_a, a * ch_scale);
  }
  if (tid == 0 && *abort_s) {
    // gave up somewhere: do not leave while a bulk copy may still be landing in this CTA's memory
    for (int a = 0; a < W_ATOMS; ++a) mbar_wait(W_FULL(a), 0u, abort_s);
    for (int b = 0; b < 2; ++b)
      if (c_cnt[b] > 0) mbar_wait(C_FULL(b), (uint32_t)((c_cnt[b] - 1) & 1), abort_s);
    if (p.status) atomicExch(p.status, 1);
  }
  // one barrier serves the hand-back of tensor memory and the release of this CTA's records
  __threadfence();
  tc_fence_before();
  __syncthreads();
  if (warp == PP_UNPACK_WARP0) tmem_dealloc(tmem_base, PP_TMEM_COLS);
  ticket_combine<PP_THREADS>(p, sq, kv, blockIdx.z, reinterpret_cast<float*>(v_s), tid, true);   // the V tiles are free
}

// Prepared weights: per KV head, W = basis * coefficient scale as fp16 in the K-major, 128-byte
// swizzled operand layout (atoms of 64 contraction positions x 128 rows).  Position kk = 8c + p
// holds rank 8c + perm[p] (the order in which the unpack step emits the nibbles of word c);
// position R holds the mean, positions R+1 .. R+15 are zero.
__global__ void __launch_bounds__(256) decode_prepare_pipe_kernel(const __half* __restrict__ basis,
                                                                  const __half* __restrict__ cscale,
                                                                  const __half* __restrict__ mean, int nkv, int rank,
                                                                  unsigned char* __restrict__ out) {
  const int kpos = rank + 16;
  const int w_bytes = ((kpos + 63) / 64) * 16384;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nkv * HD * kpos) return;
  const int kk = idx % kpos;
  const int j = (idx / kpos) % HD;
  const int kv = idx / (kpos * HD);
  const int c = kk >> 3, pp = kk & 7;
  __half v = __float2half(0.f);
  if (kk < rank) {
    const int perm = ((pp & 1) << 2) | (pp >> 1);                // 0,4,1,5,2,6,3,7
    const int r = 8 * c + perm;
    v = __hmul(basis[(size_t)(kv * HD + j) * rank + r], cscale[r]);
  } else if (kk == rank) {
    v = mean[kv * HD + j];
  }
  *reinterpret_cast<__half*>(out + (size_t)kv * w_bytes + (c >> 3) * 16384 + (j >> 3) * 1024 + (j & 7) * 128 +
                             (((c & 7) ^ (j & 7)) << 4) + pp * 2) = v;
}

size_t pipe_wprep_bytes(int nkv, int rank) { return (size_t)nkv * (((rank + 16 + 63) / 64) * 16384); }

int launch_prepare_pipe(const void* basis, const void* cscale, const void* mean, int nkv, int rank, void* out,
                        cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(out, 0, pipe_wprep_bytes(nkv, rank), st);   // unused tail of the last atom
  if (e != cudaSuccess) return (int)e;
  const int total = nkv * HD * (rank + 16);
  decode_prepare_pipe_kernel<<<(total + 255) / 256, 256, 0, st>>>((const __half*)basis, (const __half*)cscale,
                                                                   (const __half*)mean, nkv, rank, (unsigned char*)out);
  return 0;
}

template <int NW>
static int launch_pipe_one(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  constexpr int SMEM = pp_smem_bytes(NW);
  // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel
  static std::atomic<bool> configured[MAX_DEVICES];
  int dev = -1;
  cudaError_t de = cudaGetDevice(&dev);
  if (de != cudaSuccess) return (int)de;
  if (dev < 0 || dev >= MAX_DEVICES) return SHARD_E_ARG;
  if (!configured[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(decode_partial_pipe_kernel<NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured[dev].store(true, std::memory_order_release);
  }
  // Programmatic dependent launch: this launch's CTAs may move onto SMs and run their set-up
  // (barriers, first bulk copies of tensors that no decode call writes) while the kernel in front
  // of it in the stream is still finishing; griddep_wait in the kernel keeps the order of
  // everything else.  Off for a call with shape.no_overlap, or for all calls with
  // SHARD_B200_PDL=0 in the environment.
  static int use_pdl_env = -1;
  if (use_pdl_env < 0) {
    const char* e = getenv("SHARD_B200_PDL");
    use_pdl_env = (e && e[0] == '0') ? 0 : 1;
  }
  const int use_pdl = use_pdl_env && !p.sh.no_overlap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(PP_THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_partial_pipe_kernel<NW>, p);
  return e == cudaSuccess ? 0 : (int)e;
}

static int launch_rows_only(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  // (38 KB of dynamic shared memory: no opt-in needed)
  static_assert(ROWS_SMEM_BYTES <= 48 * 1024, "fits the default dynamic shared memory");
  decode_rows_only_kernel<<<grid, ROWS_THREADS, ROWS_SMEM_BYTES, st>>>(p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

int launch_partial_pipe(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  if (p.n_chunks == 0) return launch_rows_only(p, grid, st);
  switch (p.sh.rank / 32) {
    case 1: return launch_pipe_one<1>(p, grid, st);
    case 2: return launch_pipe_one<2>(p, grid, st);
    case 3: return launch_pipe_one<3>(p, grid, st);
    case 4: return launch_pipe_one<4>(p, grid, st);
    case 5: return launch_pipe_one<5>(p, grid, st);
    default: return launch_pipe_one<6>(p, grid, st);
  }
}

}  // namespace shard
