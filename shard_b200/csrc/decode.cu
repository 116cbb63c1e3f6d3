// Fused decode attention over a compressed KV cache (one query token): host side of the
// C ABI, the phase-table kernel and the stand-alone log-sum-exp merge.
//
//   score(h, t) = q_h . RoPE_{pos_t}( W coef_t + mean )        compressed middle
//   score(h, t) = q_h . k_t                                     fp16 sink / window / stream
//   out_h       = softmax_t(score / sqrt(128)) . V_t
//
// Kernels
//   phase_table_kernel          cos/sin(fp32(pos_t - pos_q) * inv_freq) in fp16, shared by all layers
//   decode_partial_pipe_kernel  (decode_pipe.cu) one launch per layer-step: optional stream append,
//                               split-KV pass over the middle / fp16 rows / streamed rows, and the
//                               combine, done by the last CTA of each KV head to arrive
//   decode_combine_kernel       the same combine as a kernel of its own, for merging the partial
//                               records of several launches or several GPUs (shard_b200_lse_merge)
#include <cstdlib>
#include <mutex>

#include "decode_common.cuh"

namespace shard {

constexpr int TILE_TOK = 128;          // tokens per tile of the middle segment
constexpr int DEFAULT_CTA_SLOTS = 148;  // SMs of a B200; used only when no device can be asked
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

struct DecodePlan {
  int n_chunks, tiles_per_chunk, tiles_rem, n_row_parts, n_parts, grid_x;
};

// the decode kernel keeps one CTA per SM: one CTA slot per SM of the current device
static int cta_slots() {
  const int n = sm_count();
  return n > 0 ? n : DEFAULT_CTA_SLOTS;
}

static DecodePlan make_plan(const ShardDecodeShape& sh, int batch) {
  DecodePlan pl{};
  const int CTA_SLOTS = cta_slots();
  const int n_tok = sh.tok_end - sh.tok_begin;
  const int n_tiles = (n_tok + TILE_TOK - 1) / TILE_TOK;
  const int groups = sh.nkv * batch;
  if (n_tiles > 0) {
    // one CTA per SM: spread the tiles of every (sequence, KV head) evenly over its CTAs
    int chunks = (groups >= CTA_SLOTS) ? (n_tiles + 15) / 16 : CTA_SLOTS / groups;
    if (chunks > n_tiles) chunks = n_tiles;
    if (chunks < 1) chunks = 1;
    pl.n_chunks = chunks;
    pl.tiles_per_chunk = n_tiles / chunks;
    pl.tiles_rem = n_tiles % chunks;
  }
  // the fp16 / streamed rows ride along in the chunk CTAs (dealt out row by row, handled while a
  // CTA waits for its first tile); only a launch without a middle gets CTAs just for them
  const int n_rows = sh.n_sink + sh.n_win + sh.n_dec + sh.n_stream;
  if (n_rows > 0) {
    pl.n_row_parts = pl.n_chunks;
    if (pl.n_chunks == 0) {
      pl.n_row_parts = (n_rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
      if (pl.n_row_parts > MAX_ROW_CTAS) pl.n_row_parts = MAX_ROW_CTAS;
    }
  }
  // a chunk CTA folds its share of the rows into its one record; only a launch without a middle
  // has records of rows alone
  pl.n_parts = pl.n_chunks > 0 ? pl.n_chunks : pl.n_row_parts;
  pl.grid_x = pl.n_chunks > 0 ? pl.n_chunks : pl.n_row_parts;
  return pl;
}

// ---------------------------------------------------------------------------
// phase table
// ---------------------------------------------------------------------------
// Layout: tokens in blocks of 32; within a block 16 planes of 32 x 16 bytes: plane c < 8 holds
// the cosines of pairs 8c..8c+7 of the block's 32 tokens (one 16-byte group per token), plane
// 8 + c the sines.  A warp whose lanes own 32 consecutive tokens reads a plane as 512
// contiguous bytes.  One thread computes one token's 8 pairs of one plane pair.
__global__ void __launch_bounds__(256) phase_table_kernel(int delta0, int n, const float* __restrict__ inv_freq,
                                                          uint4* __restrict__ out) {
  const int n_blocks = (n + 31) >> 5;
  const int total = n_blocks * 8 * 32;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int r = idx & 31, c = (idx >> 5) & 7, blk = idx >> 8;
    const int t = blk * 32 + r;
    if (t >= n) continue;
    uint32_t cw[4], sw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float sn0, cs0, sn1, cs1;
      sincosf(__fmul_rn((float)(delta0 + t), inv_freq[8 * c + 2 * j]), &sn0, &cs0);
      sincosf(__fmul_rn((float)(delta0 + t), inv_freq[8 * c + 2 * j + 1]), &sn1, &cs1);
      cw[j] = (uint32_t)__half_as_ushort(__float2half_rn(cs0)) | ((uint32_t)__half_as_ushort(__float2half_rn(cs1)) << 16);
      sw[j] = (uint32_t)__half_as_ushort(__float2half_rn(sn0)) | ((uint32_t)__half_as_ushort(__float2half_rn(sn1)) << 16);
    }
    out[((size_t)blk * 16 + c) * 32 + r] = make_uint4(cw[0], cw[1], cw[2], cw[3]);
    out[((size_t)blk * 16 + 8 + c) * 32 + r] = make_uint4(sw[0], sw[1], sw[2], sw[3]);
  }
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

}  // namespace shard

using namespace shard;

extern "C" size_t shard_b200_phase_table_bytes(int32_t n_tok) {
  if (n_tok < 0) return 0;
  return (size_t)((n_tok + 31) / 32) * 32 * HD * sizeof(__half);
}

extern "C" int shard_b200_phase_table(int32_t compress_start, int32_t pos_q, int32_t n_tok, const float* inv_freq,
                                      void* out, void* stream) {
  if (!inv_freq || !out || n_tok < 0) return SHARD_E_ARG;
  if ((uintptr_t)out & 15) return SHARD_E_ALIGN;
  if (n_tok == 0) return SHARD_OK;
  const int total = ((n_tok + 31) / 32) * 256;
  const int blocks = capped_blocks((total + 255) / 256, 8);
  phase_table_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(compress_start - pos_q, n_tok, inv_freq, (uint4*)out);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" size_t shard_b200_wprep_bytes(int32_t nkv, int32_t rank) {
  if (nkv < 1 || rank < 32 || rank > 192 || (rank % 32)) return 0;
  return pipe_wprep_bytes(nkv, rank);
}

extern "C" int shard_b200_decode_prepare(const void* basis_f16, const void* coeff_scale, const void* mean_f16,
                                         int32_t nkv, int32_t rank, void* wprep_out, void* stream) {
  if (!basis_f16 || !coeff_scale || !mean_f16 || !wprep_out) return SHARD_E_ARG;
  if (nkv < 1 || rank < 32 || rank > 192 || (rank % 32)) return SHARD_E_ARG;
  if ((uintptr_t)wprep_out & 15) return SHARD_E_ALIGN;
  int prc = launch_prepare_pipe(basis_f16, coeff_scale, mean_f16, nkv, rank, wprep_out, (cudaStream_t)stream);
  if (prc) return prc;
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

static int check_shape(const ShardDecodeShape* sh) {
  if (!sh) return SHARD_E_ARG;
  if (sh->nkv < 1 || sh->n_q != sh->nkv * GQA) return SHARD_E_ARG;
  if (sh->rank < 32 || sh->rank > 192 || (sh->rank % 32)) return SHARD_E_ARG;
  if (sh->n_comp < 0 || sh->tok_begin < 0 || sh->tok_end < sh->tok_begin || sh->tok_end > sh->n_comp)
    return SHARD_E_ARG;
  if (sh->n_sink < 0 || sh->n_win < 0 || sh->n_stream < 0 || sh->n_dec < 0) return SHARD_E_ARG;
  if (sh->dec_cap != 0 && sh->dec_cap < sh->n_dec) return SHARD_E_ARG;
  if ((sh->tok_end - sh->tok_begin) + sh->n_sink + sh->n_win + sh->n_dec + sh->n_stream <= 0) return SHARD_E_ARG;
  return SHARD_OK;
}

// scratch layout: header (status word, arrival counters; zero between calls), then
// [batch][n_parts][n_q][132] fp32 partial records
static size_t ws_bytes(const ShardDecodeShape& sh, int batch) {
  const DecodePlan pl = make_plan(sh, batch);
  return ws_header_bytes(batch, sh.nkv) + (size_t)batch * pl.n_parts * sh.n_q * PART * sizeof(float);
}

extern "C" size_t shard_b200_decode_workspace_bytes(const ShardDecodeShape* shape_host, int32_t batch) {
  if (batch < 1 || check_shape(shape_host) != SHARD_OK) return 0;
  return ws_bytes(*shape_host, batch);
}

static int decode_attn_impl(const ShardSeq* seqs, int32_t batch, const ShardDecodeShape* shape_host,
                            const float* inv_freq, const float* codebook, void* workspace, size_t workspace_bytes,
                            const PeerPush* push, void* stream) {
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
    if (!s.q || (!s.out && !push)) return SHARD_E_ARG;
    if (sh.tok_end > sh.tok_begin &&
        (!s.k_coeffs || !s.k_wprep || !s.v_indices || !s.v_centroids || !s.v_ch || !s.phase))
      return SHARD_E_ARG;
    if (sh.n_sink > 0 && (!s.sink_k || !s.sink_v)) return SHARD_E_ARG;
    if (sh.n_win > 0 && (!s.win_k || !s.win_v)) return SHARD_E_ARG;
    if (sh.n_dec > 0 && (!s.dec_k || !s.dec_v)) return SHARD_E_ARG;
    if (sh.n_stream > 0 && (!s.st_k_idx || !s.st_v_idx || !s.st_k_norm || !s.st_v_norm || !s.signs))
      return SHARD_E_ARG;
    if (((uintptr_t)s.k_coeffs & 15) || ((uintptr_t)s.k_wprep & 15) || ((uintptr_t)s.v_indices & 15) ||
        ((uintptr_t)s.v_centroids & 7) || ((uintptr_t)s.phase & 15) || ((uintptr_t)s.sink_k & 7) ||
        ((uintptr_t)s.sink_v & 7) || ((uintptr_t)s.win_k & 7) || ((uintptr_t)s.win_v & 7) ||
        ((uintptr_t)s.dec_k & 7) || ((uintptr_t)s.dec_v & 7) ||
        ((uintptr_t)s.st_k_idx & 3) || ((uintptr_t)s.st_v_idx & 3) || ((uintptr_t)s.signs & 15) ||
        ((uintptr_t)s.v_ch & 7))
      return SHARD_E_ALIGN;
  } else {
    if (push) return SHARD_E_ARG;
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
  p.n_row_parts = pl.n_row_parts;
  p.n_parts = pl.n_parts;
  p.n_ctas = pl.grid_x;
  if (push) p.push = *push;

  // one launch: the append (if asked for), the split-KV pass and the combine
  dim3 grid(pl.grid_x, sh.nkv, batch);
  rc = launch_partial_pipe(p, grid, st);
  if (rc) return rc;
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" int shard_b200_decode_attn(const ShardSeq* seqs, int32_t batch, const ShardDecodeShape* shape_host,
                                      const float* inv_freq, const float* codebook, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  return decode_attn_impl(seqs, batch, shape_host, inv_freq, codebook, workspace, workspace_bytes, nullptr, stream);
}

extern "C" int shard_b200_decode_attn_seqsplit(const ShardSeq* seq_host, const ShardDecodeShape* shape_host,
                                               const float* inv_freq, const float* codebook, void* workspace,
                                               size_t workspace_bytes, void* const* bufs_host, int32_t rank,
                                               int32_t world, uint32_t epoch, void* merged_out_f16,
                                               int* status_dev, uint32_t timeout_us, void* stream) {
  if (!bufs_host || world < 1 || world > PEER_MAX_WORLD || rank < 0 || rank >= world || epoch == 0 || !shape_host)
    return SHARD_E_ARG;
  if (!shape_host->partial_out) return SHARD_E_ARG;   // what travels is the unnormalised record
  PeerPush push{};
  for (int r = 0; r < world; ++r) {
    if (!bufs_host[r]) return SHARD_E_ARG;
    push.bufs[r] = reinterpret_cast<unsigned char*>(bufs_host[r]);
  }
  push.rank = rank;
  push.world = world;
  push.epoch = epoch;
  push.merged_out = merged_out_f16;
  push.status = status_dev;
  push.wait_ns = timeout_us ? (unsigned long long)timeout_us * 1000ull : PEER_DEFAULT_WAIT_NS;
  return decode_attn_impl(seq_host, 1, shape_host, inv_freq, codebook, workspace, workspace_bytes, &push, stream);
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
  // The array still holds whatever the previous call left there.  Only the arrival counters
  // have to start at zero; every partial record is rewritten before it is read.  The status
  // word in front of the counters is left alone: a launch that gave up leaves a 1 there, and
  // it stays until shard_b200_decode_status(NULL, ...) has reported it.
  cudaError_t e = cudaMemsetAsync((unsigned char*)scratch + WS_STATUS_BYTES, 0,
                                  ws_header_bytes(1, shape_host->nkv) - WS_STATUS_BYTES, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return shard_b200_decode_attn(seq_host, 1, shape_host, inv_freq, codebook, scratch,
                                (size_t)SHARD_B200_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int shard_b200_decode_status(void* workspace, int32_t* status_host_out, void* stream) {
  if (!status_host_out) return SHARD_E_ARG;
  void* ws = workspace;
  if (!ws) {
    int rc = static_scratch_for_current_device(&ws);
    if (rc != SHARD_OK) return rc;
  }
  cudaStream_t st = (cudaStream_t)stream;
  int32_t word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, ws, sizeof(word), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return (int)e;
  if (word != 0) {
    e = cudaMemsetAsync(ws, 0, sizeof(word), st);   // reported once; the next launch starts clean
    if (e != cudaSuccess) return (int)e;
  }
  *status_host_out = word;
  return SHARD_OK;
}

extern "C" int shard_b200_abi_version(void) { return 3; }

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
