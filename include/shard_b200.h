/*
 * shard_b200 -- C ABI of the B200 (sm_100a) compressed-KV attention kernels.
 *
 * The reference (bhengubv/shard) is pure Python: its device code is eight
 * Triton kernels with PyTorch fallbacks and it has no foreign-function
 * interface of its own.  Each entry point below therefore cites the Python
 * function(s) of the reference whose work it replaces (paths relative to the
 * reference project root).
 *
 * Conventions
 *   - every pointer is a CUDA device pointer unless its name ends in _host;
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream);
 *   - return value: 0 on success, a negative SHARD_E_* code on a rejected
 *     argument, a positive value = cudaError_t of the failed runtime call;
 *   - no entry point allocates or frees device memory; scratch space is passed
 *     in by the caller (see the *_workspace_bytes helpers);
 *   - kernels are asynchronous with respect to the host: they are enqueued on
 *     `stream` and the call returns immediately;
 *   - head_dim is 128 and the codebook has 256 entries of 4 channels
 *     everywhere (Llama-3.1-8B geometry, the reference's defaults).
 */
#ifndef SHARD_B200_H_
#define SHARD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SHARD_OK 0
#define SHARD_E_ARG (-1)       /* null pointer, bad size or unsupported geometry  */
#define SHARD_E_WORKSPACE (-2) /* workspace too small                             */
#define SHARD_E_ALIGN (-3)     /* pointer not aligned as documented               */
#define SHARD_E_TOO_LARGE (-4) /* more scratch needed than the built-in area holds */

#define SHARD_HEAD_DIM 128
#define SHARD_PART_STRIDE 132  /* floats per (part, head) record: m, l, 0, 0, acc[128] */

/* ABI version of this header; bumped on any signature change. */
int shard_b200_abi_version(void);

/* Human-readable text for a status code returned by any entry point. */
const char* shard_b200_status_string(int status);

/*
 * Per-sequence tensor table of one layer's compressed cache: the device view of
 * the dict the reference builds in Cache._build_gpu_format
 * (src/shard/cache.py:406-460) plus the streamed-token buffers of
 * CacheLayer._stream_append (src/shard/cache.py:193-241).
 */
typedef struct ShardSeq {
  const uint8_t* k_coeffs;   /* [n_comp][rank/2]  packed int4 PCA coefficients, 16-byte aligned */
  const void* k_wprep;       /* output of shard_b200_decode_prepare for this layer      */
  const uint8_t* v_indices;  /* [nkv][n_comp][32] VQ codes                              */
  const void* v_centroids;   /* fp16 [256][4]                                           */
  const void* v_ch;          /* fp16 [nkv][128]   per-channel max-abs                   */
  const void* sink_k;        /* fp16 [nkv][n_sink][128] (keys carry RoPE)               */
  const void* sink_v;        /* fp16 [nkv][n_sink][128]                                 */
  const void* win_k;         /* fp16 [nkv][n_win][128]                                  */
  const void* win_v;         /* fp16 [nkv][n_win][128]                                  */
  uint8_t* st_k_idx;         /* [cap][nkv][128]   8-bit Lloyd-Max codes of streamed K   */
  uint8_t* st_v_idx;         /* [cap][nkv][128]                                         */
  void* st_k_norm;           /* fp16 [cap][nkv]                                         */
  void* st_v_norm;           /* fp16 [cap][nkv]                                         */
  const float* signs;        /* [128] +-1, per layer                                    */
  const void* phase;         /* table written by shard_b200_phase_table for [tok_begin, tok_end) */
  const void* q;             /* fp16 [n_q][128]   query, RoPE applied at pos_q          */
  void* out;                 /* fp16 [n_q][128] result, or fp32 [n_q][132] partial      */
  const void* new_k;         /* fp16 [nkv][128]   token to append (stream_quantize)     */
  const void* new_v;         /* fp16 [nkv][128]                                         */
  const void* dec_k;         /* fp16 [nkv][dec_cap or n_dec][128] tokens appended as they are by a */
  const void* dec_v;         /* non-streaming cache (gc["decode_k"], gc["decode_v"])    */
} ShardSeq;

/* Scalars shared by every sequence of a launch. */
typedef struct ShardDecodeShape {
  int32_t n_q;            /* query heads (n_q / nkv must be 4)                           */
  int32_t nkv;            /* KV heads                                                    */
  int32_t rank;           /* PCA rank R: multiple of 32, 32..192                         */
  int32_t n_comp;         /* tokens in the compressed middle segment                     */
  int32_t tok_begin;      /* this call attends to middle tokens [tok_begin, tok_end)     */
  int32_t tok_end;
  int32_t n_sink;         /* fp16 sink tokens (0 to skip; sequence-split ranks > 0)      */
  int32_t n_win;          /* fp16 window tokens                                          */
  int32_t n_stream;       /* streamed tokens to attend to                                */
  int32_t pos_q;          /* position of the query token                                 */
  int32_t partial_out;    /* 0: out = fp16 attention; 1: out = fp32 (m, l, acc) partial  */
  int32_t append;         /* 1: first quantise new_k/new_v into stream row n_stream-1 (fused append) */
  int32_t n_dec;          /* rows of the fp16 decode buffer (dec_k / dec_v)              */
  int32_t no_overlap;     /* 1: plain launch, no early start behind the preceding kernel (see decode_attn) */
  int32_t dec_cap;        /* rows allocated per KV head in dec_k / dec_v (0: exactly n_dec)    */
} ShardDecodeShape;

/*
 * cos/sin of fp32(compress_start + t - pos_q) * inv_freq[i], rounded to fp16, for
 * t in [0, n_tok), i in [0, 64): the table of src/shard/attention.py:76-79.
 * It depends only on positions, so one table serves every layer of a step.
 * out (16-byte aligned, shard_b200_phase_table_bytes(n_tok) bytes) is opaque to the caller:
 * tokens are grouped in blocks of 32, and a block stores 16 planes of 32 x 16 bytes -- plane c < 8
 * the cosines of pairs 8c..8c+7 for each of its tokens, plane 8 + c the sines -- so that a warp
 * owning 32 consecutive tokens reads each plane as one contiguous 512-byte run.
 */
size_t shard_b200_phase_table_bytes(int32_t n_tok);
int shard_b200_phase_table(int32_t compress_start, int32_t pos_q, int32_t n_tok,
                           const float* inv_freq, void* out, void* stream);

/*
 * Size in bytes of the prepared-weight blob for `nkv` KV heads and PCA rank `rank`.
 */
size_t shard_b200_wprep_bytes(int32_t nkv, int32_t rank);

/*
 * Folds k_coeff_scale into k_basis_f16, appends k_mean as one extra contraction
 * column and lays the result out as the 128-byte-swizzled K-major operand that
 * tcgen05.mma reads from shared memory.  Runs once per
 * layer after compression; replaces the per-step operand build of
 * compressed_scores (src/shard/attention.py:34-63).
 * basis_f16: [nkv*128][rank], coeff_scale: [rank], mean_f16: [nkv*128] (all fp16).
 */
int shard_b200_decode_prepare(const void* basis_f16, const void* coeff_scale, const void* mean_f16,
                              int32_t nkv, int32_t rank, void* wprep_out, void* stream);

/*
 * Bytes of scratch shard_b200_decode_attn needs for `batch` sequences of this shape
 * (0 if the shape is rejected).
 */
size_t shard_b200_decode_workspace_bytes(const ShardDecodeShape* shape_host, int32_t batch);

/*
 * Fused decode attention of one query token over
 * [sink | compressed middle | window | fp16 decode buffer | streamed tokens]: replaces
 * fused_attention_compressed (src/shard/attention.py:270-343) with its callees
 * compressed_scores (18-81), int4_matmul (triton_kernels.py:65-88),
 * _v_weighted_sum_compressed (83-121), vq_weighted_sum_all
 * (triton_kernels.py:255-295), hadamard (cache.py:10-19) and
 * CacheLayer._dequant_stream (cache.py:243-279).
 *
 * batch == 1: `seqs` is a HOST pointer to one ShardSeq (copied by value).
 * batch  > 1: `seqs` is a DEVICE pointer to `batch` ShardSeq records describing
 *             independent sequences that share `shape`.
 * inv_freq: [64] fp32.  workspace: at least shard_b200_decode_workspace_bytes(shape, batch)
 * bytes, 16-byte aligned, zero-filled once after it was allocated (see below).
 * The call is one kernel launch: append (if asked for), attention over all four segments
 * and the combine of the split-KV partial results.
 * With shape.partial_out the result is the unnormalised per-head triple
 * (max, sum-exp, acc[128]) in standard V space, ready for shard_b200_lse_merge.
 * With shape.append the call also does the work of shard_b200_stream_quantize for the newest
 * token: new_k/new_v are quantised into stream row n_stream-1 (n_stream counts that token)
 * before the stream is attended to.
 * The head of the workspace (a status word, then one arrival counter per sequence and KV head:
 * 16 + 4*batch*nkv bytes rounded up to 16) must be zero before the first call that uses the
 * workspace; every call leaves it zero again unless a bounded wait inside the kernel gave up,
 * in which case the status word is left at 1 and the output of that call is undefined
 * (read it with shard_b200_decode_status).
 * The kernel is launched with programmatic stream serialization: its CTAs may start while the
 * kernel directly in front of it in the stream is still running, and before waiting for that
 * kernel they read k_wprep, k_coeffs, v_indices, v_centroids, the stream codebook, inv_freq and
 * (batch > 1) the ShardSeq table, and already expand the first tiles of the middle segment from them;
 * they also read the phase table, which therefore has to be complete when the launch starts (it is
 * when shard_b200_phase_table produced it earlier on the same stream: that kernel does not release
 * the launches behind it early).  So the kernel directly in front must not be one that WRITES any of those
 * (shard_b200_decode_prepare, the kernels that produce the codes, a copy into the table): for
 * the first decode call behind such work set shape.no_overlap = 1, which launches the plain way
 * (or set SHARD_B200_PDL=0 in the environment to do so always).  Everything else -- query, new
 * token, stream rows, workspace, output -- is read and written only after the
 * preceding work has completed.
 */
int shard_b200_decode_attn(const ShardSeq* seqs, int32_t batch, const ShardDecodeShape* shape_host,
                           const float* inv_freq, const float* codebook, void* workspace,
                           size_t workspace_bytes, void* stream);

/*
 * Reads the status word a decode launch leaves at the head of its workspace: waits for
 * `stream`, stores the word in *status_host_out (0 = every launch since the last query
 * completed normally, 1 = a bounded wait inside a kernel gave up and that call's output is
 * undefined) and, if it was set, clears it.  workspace == NULL names the built-in scratch of
 * shard_b200_decode_attn_noalloc on the current device.  Meant to be called once per step or
 * per request, not per launch.  No reference counterpart (the reference has no device-side
 * waits).
 */
int shard_b200_decode_status(void* workspace, int32_t* status_host_out, void* stream);

/*
 * Size of the scratch area that lives inside the library's device image and is used by
 * shard_b200_decode_attn_noalloc.  Every GPU that loads the library sets this much memory
 * aside until the process exits.
 */
#define SHARD_B200_STATIC_SCRATCH_BYTES (2u << 20)

/*
 * shard_b200_decode_attn for one sequence, for callers that cannot allocate device memory
 * and so have no workspace to pass: for example a server that freezes its device-memory
 * plan at start-up and forbids cudaMalloc afterwards, or a host program that only lends
 * this library its tensors and offers no allocator.  The scratch comes from a fixed
 * 2 MiB area built into the library; inputs and outputs are still the caller's
 * (`seq_host` is a host pointer to one ShardSeq, exactly as with batch == 1 above).
 * This entry point has no counterpart in the reference.
 *
 *   - Shapes whose split-KV records do not fit in SHARD_B200_STATIC_SCRATCH_BYTES are
 *     refused with SHARD_E_TOO_LARGE and nothing is launched.  With 32 query heads the
 *     area holds 124 records per head; a launch writes at most 36 (18 chunks of the middle
 *     segment, each with one record for the middle and one for its share of the sink /
 *     window / streamed rows), so only very wide head counts are refused.
 *   - No cudaMalloc / cudaFree or other allocating call is made, now or later.
 *   - The first call on a device looks up the device address of the built-in area
 *     (cudaGetSymbolAddress, with that device current) and remembers it; make that
 *     first call before starting any stream capture.
 *   - All calls on a device share the one area, and it keeps the previous call's
 *     contents (the part that must start at zero is cleared on `stream` by each call;
 *     the status word is kept until shard_b200_decode_status(NULL, ...) has reported it).
 *     Two calls whose kernels can overlap on the GPU -- different streams without an
 *     ordering between them -- race on it and give wrong results; serialise them.
 */
int shard_b200_decode_attn_noalloc(const ShardSeq* seq_host, const ShardDecodeShape* shape_host,
                                   const float* inv_freq, const float* codebook, void* stream);

/*
 * Log-sum-exp combine of `n_parts` partials (fp32 [n_parts][n_q][132]) into fp16
 * [n_q][128]: the mixing step of fused_attention_compressed_full
 * (src/shard/attention.py:262-266), here used to merge the per-GPU partials of a
 * sequence-split cache.  Parts are combined in index order.
 */
int shard_b200_lse_merge(const float* parts, int32_t n_parts, int32_t n_q, void* out_f16, void* stream);

/*
 * Sequence-split decode on one multi-GPU node: exchange of the per-rank partial records over
 * NVLink peer memory and their merge, in one kernel per rank and layer-step (no reference
 * counterpart; the mixing formula is fused_attention_compressed_full's,
 * src/shard/attention.py:262-266).
 *
 * Every rank allocates one exchange buffer of shard_b200_peer_buffer_bytes(world, nkv) bytes with
 * shard_b200_peer_alloc (cudaMalloc + zero fill + CUDA IPC export: a set-up call, not for the
 * hot path), hands the 64-byte handle to the other ranks by any means, and opens theirs with
 * shard_b200_peer_open.  shard_b200_seqsplit_merge then takes this rank's fp32 [4*nkv][132]
 * partial (the output of shard_b200_decode_attn with shape.partial_out), stores it into every
 * rank's buffer with plain peer stores, publishes `epoch`, waits -- bounded by `timeout_us`
 * microseconds of the GPU's global timer (0 = 200 000), after which *status_dev is set to 1 and
 * out is left unwritten -- for all ranks' records of the same epoch and merges them in rank order
 * into out_f16 (fp16 [4*nkv][128]), bit-identical on every rank.  `bufs_host` is a HOST array of
 * `world` device pointers (entry `rank` = own buffer); `epoch` starts at 1 and grows by 1 per
 * call, in step on all ranks.
 *
 * Faster forms of the same step: shard_b200_decode_attn_seqsplit is shard_b200_decode_attn for one
 * sequence (shape.partial_out must be 1) whose combining CTAs deliver the record straight into
 * every rank's buffer and publish `epoch` -- the decode launch does the exchange.  With
 * merged_out_f16 set (fp16 [4*nkv][128]) the same CTAs then wait, bounded by `timeout_us` like
 * above (status_dev), for all ranks' records and write the merged attention output: the whole
 * step is ONE launch per rank.  With merged_out_f16 == NULL the wait + merge half is a launch of
 * its own, shard_b200_seqsplit_wait_merge, started so that it is already polling while the decode
 * launch in front of it runs.  seq_host->out may be NULL in both.  Per epoch a rank uses one of the
 * three forms; ranks may differ.
 */
size_t shard_b200_peer_buffer_bytes(int32_t world, int32_t nkv);
int shard_b200_peer_alloc(size_t bytes, void** ptr_out, void* handle_out_64);
int shard_b200_peer_open(const void* handle_64, void** ptr_out);
int shard_b200_peer_close(void* ptr);
int shard_b200_peer_free(void* ptr);
int shard_b200_seqsplit_merge(const float* my_part, void* const* bufs_host, int32_t rank, int32_t world,
                              int32_t nkv, uint32_t epoch, void* out_f16, int* status_dev,
                              uint32_t timeout_us, void* stream);
int shard_b200_decode_attn_seqsplit(const ShardSeq* seq_host, const ShardDecodeShape* shape_host,
                                    const float* inv_freq, const float* codebook, void* workspace,
                                    size_t workspace_bytes, void* const* bufs_host, int32_t rank,
                                    int32_t world, uint32_t epoch, void* merged_out_f16, int* status_dev,
                                    uint32_t timeout_us, void* stream);
int shard_b200_seqsplit_wait_merge(void* const* bufs_host, int32_t rank, int32_t world, int32_t nkv,
                                   uint32_t epoch, void* out_f16, int* status_dev, uint32_t timeout_us,
                                   void* stream);

/*
 * 8-bit Lloyd-Max quantisation of one new K and V token per KV head and append
 * at row `slot` of the stream buffers: CacheLayer._stream_append
 * (src/shard/cache.py:193-241) + quantize_per_token (src/shard/streaming.py:59-72).
 * Uses new_k/new_v, signs and the st_* buffers of each ShardSeq.
 * batch == 1: host pointer to one record; batch > 1: device pointer to a table.
 * codebook: [256] fp32 ascending (Lloyd-Max centroids of N(0, 1/128)).
 */
int shard_b200_stream_quantize(const ShardSeq* seqs, int32_t batch, int32_t nkv, int32_t slot,
                               const float* codebook, void* stream);

/*
 * fp16 K/V [nkv][n_stream][128] of the streamed tokens: CacheLayer._dequant_stream
 * (src/shard/cache.py:243-279) + dequantize_per_token (streaming.py:74-79).  Used by
 * the non-fused read path only.
 */
int shard_b200_stream_dequant(const uint8_t* idx, const void* norm_f16, const float* signs,
                              const float* codebook, int32_t n_stream, int32_t nkv, void* out_f16,
                              void* stream);

/*
 * Undo RoPE on prefill keys and flatten to [n][nkv*128] fp32 (column = kv*128+d):
 * undo_rope (src/shard/rope.py:20-24) as called from Cache._compress_k
 * (src/shard/cache.py:370-372).  k_f16: [nkv][.][128] with `tok_stride` elements
 * between tokens' rows and `head_stride` elements between heads; token t has
 * position pos_start + t.
 */
int shard_b200_undo_rope(const void* k_f16, int64_t head_stride, int64_t tok_stride, int32_t nkv,
                         int32_t n, int32_t pos_start, const float* inv_freq, float* flat_out,
                         void* stream);

/*
 * proj[n][keep] = (flat - mean) @ w: the PCA projection of Cache._compress_k
 * (src/shard/cache.py:392), on the tensor cores with fp32 accuracy (every operand is split into
 * a tf32 head and tail; three tf32 products per k-step accumulate in fp32).
 * flat: [n][dim], mean: [dim], w: [dim][keep] (= int8 basis * fp32 scale), all fp32, 16-byte
 * aligned; dim a multiple of 32, at most 1024; keep even, at most 192.  workspace:
 * shard_b200_k_project_workspace_bytes(dim, keep) bytes, 16-byte aligned (a status word that a
 * bounded wait inside the kernel sets to 1 when it gives up, then the split weights).
 */
size_t shard_b200_k_project_workspace_bytes(int32_t dim, int32_t keep);
int shard_b200_k_project(const float* flat, const float* mean, const float* w, int32_t n, int32_t dim,
                         int32_t keep, float* proj_out, void* workspace, size_t workspace_bytes,
                         void* stream);

/* Scratch bytes for shard_b200_k_quantize_pack. */
size_t shard_b200_k_quantize_workspace_bytes(int32_t n, int32_t keep);

/*
 * int4 codes of the projected keys: quantize_group -> dequantize_group
 * (src/shard/rope.py:95-161) -> re-quantisation to [-7, 7]
 * (src/shard/cache.py:416-419) -> int4_pack (triton_kernels.py:665-682).
 * proj: [n][keep] fp32, alloc_bits: [keep] int32 in {0,2,4,6,8}, keep even.
 * Outputs: coeff_scale fp32 [keep], packed [n*keep/2].
 */
int shard_b200_k_quantize_pack(const float* proj, const int32_t* alloc_bits, int32_t n, int32_t keep,
                               float* coeff_scale_out, uint8_t* packed_out, void* workspace,
                               size_t workspace_bytes, void* stream);

/* Pairs adjacent int8 values in [-7, 7] into nibbles: int4_pack (triton_kernels.py:665-682). */
int shard_b200_int4_pack(const int8_t* q, int64_t n_values, uint8_t* packed_out, void* stream);

/*
 * Hadamard rotation + per-channel max-abs normalisation of prefill values:
 * Cache._compress_v (src/shard/cache.py:398-404) and the first half of vq_encode
 * (cache.py:41-46).  v_f16: [nkv][.][128] with the given strides (elements).
 * Outputs: x fp32 [nkv][n][128] (= rot / ch_max; viewed by the caller as
 * [nkv*n*32][4] sub-vectors) and ch_max fp32 [nkv][128].
 */
int shard_b200_v_hadamard_normalise(const void* v_f16, int64_t head_stride, int64_t tok_stride,
                                    int32_t nkv, int32_t n, float* x_out, float* ch_max_out,
                                    void* stream);

/*
 * Nearest-centroid assignment, first minimum wins: vq_assign
 * (triton_kernels.py:689-746).  x: [n][4] fp32, centroids: [256][4] fp32.
 * Writes idx_u8 [n] and, if non-null, idx_i64 [n] (for the caller's centroid update).
 */
int shard_b200_vq_assign(const float* x, const float* centroids, int64_t n, uint8_t* idx_u8,
                         int64_t* idx_i64, void* stream);

/*
 * One Lloyd iteration's heavy part: the assignment of shard_b200_vq_assign plus, in the same
 * pass, the per-centroid sums (fp32 [256][4]) and counts (fp32 [256]) that the reference gets
 * from two index_add_ calls in kmeans (src/shard/cache.py:29-32).  `sums` and `counts` must be
 * zero on entry; the additions happen in no fixed order (as index_add_ on a GPU).
 */
int shard_b200_vq_assign_accumulate(const float* x, const float* centroids, int64_t n, uint8_t* idx_u8,
                                    float* sums, float* counts, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SHARD_B200_H_ */
