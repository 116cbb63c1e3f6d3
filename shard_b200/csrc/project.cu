// PCA projection of the prefill keys on the tensor cores:
//
//     proj[n][keep] = (flat[n][dim] - mean[dim]) . w[dim][keep]        fp32 in, fp32 out
//
// the one dense contraction of the prefill compressor (Cache._compress_k, the reference's
// `(flat - mean) @ (basis_q * scale)`).  The int4 codes that follow are sensitive to the last
// bits of the result, so the product keeps fp32 accuracy: both operands are split into a tf32
// head and a tf32 tail (x = hi + lo, hi = tf32(x), lo = tf32(x - hi)) and every k-step issues
// three `tcgen05.mma kind::tf32` products -- lo.hi, hi.lo, hi.hi -- into one fp32 accumulator in
// tensor memory.  The dropped lo.lo term and the rounding of the tails are 2^-22 relative to a
// product, the size of fp32's own rounding.
//
// The tensor core adds each k-step to its accumulator with truncation, which over the 384
// k-step products of a 1024-deep contraction would cost a hundred units in the last place.  So the
// accumulator only ever holds a group of four chunks (48 products): two accumulator buffers
// alternate, and while one fills the other is added -- rounded to nearest, on the CUDA cores --
// to the running fp32 sum that eight warps keep in registers.
//
// One CTA computes 128 rows x all `keep` columns (padded to a multiple of 16, at most 192) with a
// two-stage ring over the contraction in chunks of 32 (one 128-byte swizzle row):
//
//   warps 0-3   thread = row: load 32 fp32 of the row, subtract the mean, split, store head and
//               tail into the stage's A tiles (K-major, 128-byte swizzle)
//   warp 4      one thread: bulk copies of the weight chunks and all MMAs.  The weights are split
//               and laid out in their shared-memory image once per call by a small kernel
//               (`k_project_prepare_kernel`), so a chunk of both parts is ONE bulk copy.
//   warps 5-12  thread = (row, half of the columns): promotion of the accumulator buffers, and the
//               store of the result
#include <atomic>

#include "tcgen05.cuh"

namespace shard {

constexpr int PJ_ROWS = 128;          // rows per CTA
constexpr int PJ_KC = 32;             // contraction positions per chunk (128 bytes of fp32)
constexpr int PJ_MAX_N = 192;
constexpr int PJ_STAGES = 2;
constexpr int PJ_THREADS = 13 * 32;     // 4 producer warps, 1 issuing warp, 8 promotion warps
constexpr int PJ_GROUP = 4;               // chunks accumulated in tensor memory between two promotions
constexpr int PJ_A_BYTES = PJ_ROWS * 128;                 // one A tile (head or tail) of a stage

__host__ __device__ inline int pj_pad_n(int keep) { return (keep + 15) & ~15; }
__host__ __device__ inline size_t pj_b_chunk_bytes(int keep) { return (size_t)2 * pj_pad_n(keep) * 128; }
__host__ __device__ inline size_t pj_smem_bytes(int keep) {
  return 1024 + PJ_STAGES * (2 * PJ_A_BYTES + pj_b_chunk_bytes(keep)) + 4096 /* mean */ + 256;
}

__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// Weights -> per chunk of 32 contraction positions the shared-memory image of the B operand:
// [chunk][head | tail][keepP rows x 128 bytes, K-major, 128-byte swizzle]; rows >= keep are zero.
__global__ void __launch_bounds__(256) k_project_prepare_kernel(const float* __restrict__ w, int dim, int keep,
                                                                unsigned char* __restrict__ out) {
  const int keepP = pj_pad_n(keep);
  const size_t total = (size_t)dim * keepP;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int nrow = (int)(idx % keepP), k = (int)(idx / keepP);
    const float x = nrow < keep ? w[(size_t)k * keep + nrow] : 0.f;
    const float hi = tf32_rna(x), lo = tf32_rna(x - hi);
    const int c = k / PJ_KC, kk = k % PJ_KC;
    unsigned char* base = out + (size_t)c * pj_b_chunk_bytes(keep);
    const uint32_t off = sw128_off(nrow, kk >> 2) + (uint32_t)(kk & 3) * 4u;
    *reinterpret_cast<float*>(base + off) = hi;
    *reinterpret_cast<float*>(base + (size_t)keepP * 128 + off) = lo;
  }
}

__device__ __forceinline__ void umma_tf32_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// instruction descriptor for kind::tf32: tf32 operands (format 2), fp32 accumulation, both K-major
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__global__ void __launch_bounds__(PJ_THREADS, 1) k_project_tc_kernel(const float* __restrict__ flat,
                                                                      const float* __restrict__ mean,
                                                                      const unsigned char* __restrict__ wimg, int n,
                                                                      int dim, int keep, float* __restrict__ proj,
                                                                      int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int keepP = pj_pad_n(keep);
  const uint32_t b_bytes = (uint32_t)pj_b_chunk_bytes(keep);
  const uint32_t stage_bytes = 2 * PJ_A_BYTES + b_bytes;
  float* mean_s = reinterpret_cast<float*>(smem + PJ_STAGES * stage_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(mean_s) + 4096);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto FULL = [&](int s) { return bar0 + 8u * (uint32_t)s; };            // A tiles written (4 warps) + weight chunk landed
  auto EMPTY = [&](int s) { return bar0 + 8u * (uint32_t)(2 + s); };     // the stage's MMAs have run
  auto ACC_FULL = [&](int b) { return bar0 + 8u * (uint32_t)(4 + b); };  // a group of chunks has been accumulated in buffer b
  auto ACC_FREE = [&](int b) { return bar0 + 8u * (uint32_t)(6 + b); };  // buffer b has been added to the registers

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = blockIdx.x * PJ_ROWS;
  const int n_chunks = dim / PJ_KC;
  const int n_groups = (n_chunks + PJ_GROUP - 1) / PJ_GROUP;

  if (warp == 4) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
    if (lane == 0) {
      for (int s = 0; s < PJ_STAGES; ++s) {
        mbar_init(FULL(s), 5); mbar_init(EMPTY(s), 1); mbar_init(ACC_FULL(s), 1); mbar_init(ACC_FREE(s), 8);
      }
      *abort_s = 0;
      fence_mbar_init();
    }
  }
  for (int i = tid; i < dim; i += PJ_THREADS) mean_s[i] = mean[i];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    // ---- A producers ---------------------------------------------------------------------------
    const int r = warp * 32 + lane;
    const bool live = row0 + r < n;
    const float* src = flat + (size_t)(row0 + (live ? r : 0)) * dim;
    bool bad = false;
    for (int c = 0; c < n_chunks && !bad; ++c) {
      const int s = c & 1;
      if (c >= PJ_STAGES) bad = !mbar_wait(EMPTY(s), (uint32_t)(((c >> 1) - 1) & 1), abort_s);
      bad = __any_sync(0xffffffffu, bad || *abort_s);
      if (bad) break;
      unsigned char* a_hi = smem + s * stage_bytes;
      unsigned char* a_lo = a_hi + PJ_A_BYTES;
      float4 x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        x[j] = live ? *reinterpret_cast<const float4*>(src + c * PJ_KC + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 mu = *reinterpret_cast<const float4*>(mean_s + c * PJ_KC + 4 * j);
        const float v[4] = {__fsub_rn(x[j].x, mu.x), __fsub_rn(x[j].y, mu.y), __fsub_rn(x[j].z, mu.z),
                            __fsub_rn(x[j].w, mu.w)};
        float hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float t = live ? v[e] : 0.f;
          hi[e] = tf32_rna(t);
          lo[e] = tf32_rna(t - hi[e]);
        }
        const uint32_t off = sw128_off(r, j);
        *reinterpret_cast<float4*>(a_hi + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<float4*>(a_lo + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(FULL(s));
    }
  } else if (warp == 4) {
    // ---- bulk copies of the weight chunks and all MMAs ----------------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_tf32(128, keepP);
      bool ok = true;
      auto issue_b = [&](int c) {
        const int s = c & 1;
        mbar_expect_tx(FULL(s), b_bytes);
        bulk_g2s(smem_u32(smem + s * stage_bytes + 2 * PJ_A_BYTES), wimg + (size_t)c * b_bytes, b_bytes, FULL(s));
      };
      issue_b(0);
      for (int c = 0; c < n_chunks && ok; ++c) {
        const int s = c & 1, grp = c / PJ_GROUP, b = grp & 1;
        if (c + 1 < n_chunks) {
          if (c + 1 >= PJ_STAGES) ok = mbar_wait(EMPTY((c + 1) & 1), (uint32_t)((((c + 1) >> 1) - 1) & 1), abort_s);
          if (!ok) break;
          issue_b(c + 1);
        }
        const bool first = (c % PJ_GROUP) == 0;
        if (first && grp >= 2) ok = mbar_wait(ACC_FREE(b), (uint32_t)(((grp >> 1) - 1) & 1), abort_s);
        ok = ok && mbar_wait(FULL(s), (uint32_t)((c >> 1) & 1), abort_s);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(256 * b);
        const uint32_t a_hi = smem_u32(smem + s * stage_bytes), a_lo = a_hi + PJ_A_BYTES;
        const uint32_t b_hi = a_hi + 2 * PJ_A_BYTES, b_lo = b_hi + (uint32_t)keepP * 128u;
        const uint64_t dah = smem_desc_sw128(a_hi, 16, 1024), dal = smem_desc_sw128(a_lo, 16, 1024);
        const uint64_t dbh = smem_desc_sw128(b_hi, 16, 1024), dbl = smem_desc_sw128(b_lo, 16, 1024);
#pragma unroll
        for (int ks = 0; ks < PJ_KC / 8; ++ks) {
          const uint64_t adv = (uint64_t)((ks * 32) >> 4);
          umma_tf32_ss(acc, dal + adv, dbh + adv, idesc, (!first || ks > 0) ? 1u : 0u);   // the small terms first
          umma_tf32_ss(acc, dah + adv, dbl + adv, idesc, 1u);
          umma_tf32_ss(acc, dah + adv, dbh + adv, idesc, 1u);
        }
        umma_commit(EMPTY(s));
        if ((c % PJ_GROUP) == PJ_GROUP - 1 || c == n_chunks - 1) umma_commit(ACC_FULL(b));
      }
      if (!ok) *abort_s = 1;
    }
    __syncwarp();
  } else {
    // ---- promotion: the accumulator of every group of chunks is added, rounded to nearest, to an
    // fp32 sum in registers; thread = (row, half of the columns) ---------------------------------
    const int pw = warp - 5, quad = warp & 3, half = pw >> 2;
    const int r = quad * 32 + lane;
    const bool live = row0 + r < n;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int col0 = half * (PJ_MAX_N / 2);
    float sum[PJ_MAX_N / 2];
#pragma unroll
    for (int j = 0; j < PJ_MAX_N / 2; ++j) sum[j] = 0.f;
    bool bad = false;
    for (int grp = 0; grp < n_groups; ++grp) {
      const int b = grp & 1;
      bad = !mbar_wait(ACC_FULL(b), (uint32_t)((grp >> 1) & 1), abort_s);
      bad = __any_sync(0xffffffffu, bad || *abort_s);
      if (bad) break;
      tc_fence_after();
#pragma unroll
      for (int i = 0; i < PJ_MAX_N / 32; ++i) {
        if (col0 + 16 * i < keepP) {                    // uniform over the CTA
          uint32_t o[16];
          tmem_ld_x16(tmem_base + (uint32_t)(256 * b + col0 + 16 * i) + lane_off, o);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) sum[16 * i + j] = __fadd_rn(sum[16 * i + j], __uint_as_float(o[j]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ACC_FREE(b));
    }
    if (!bad && live) {
      float* dst = proj + (size_t)(row0 + r) * keep + col0;
#pragma unroll
      for (int j = 0; j < PJ_MAX_N / 2; j += 2)
        if (col0 + j < keep)                          // keep is even: pairs are stored together
          *reinterpret_cast<float2*>(dst + j) = make_float2(sum[j], sum[j + 1]);
    }
  }
  if (tid == 0 && *abort_s && status) atomicExch(status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, 512);
}

}  // namespace shard

using namespace shard;

extern "C" size_t shard_b200_k_project_workspace_bytes(int32_t dim, int32_t keep) {
  if (dim < PJ_KC || (dim % PJ_KC) || keep < 2 || keep > PJ_MAX_N || (keep & 1)) return 0;
  return 16 + (size_t)(dim / PJ_KC) * pj_b_chunk_bytes(keep);
}

extern "C" int shard_b200_k_project(const float* flat, const float* mean, const float* w, int32_t n, int32_t dim,
                                    int32_t keep, float* proj_out, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  if (!flat || !mean || !w || !proj_out || !workspace || n < 0) return SHARD_E_ARG;
  const size_t need = shard_b200_k_project_workspace_bytes(dim, keep);
  if (need == 0 || dim > 1024) return SHARD_E_ARG;
  if (workspace_bytes < need) return SHARD_E_WORKSPACE;
  if ((((uintptr_t)flat | (uintptr_t)mean | (uintptr_t)workspace) & 15) || ((uintptr_t)proj_out & 7)) return SHARD_E_ALIGN;
  if (n == 0) return SHARD_OK;
  cudaStream_t st = (cudaStream_t)stream;
  int* status = (int*)workspace;                       // bounded-wait status word, then the weight image
  unsigned char* wimg = (unsigned char*)workspace + 16;
  cudaError_t e = cudaMemsetAsync(status, 0, 16, st);
  if (e != cudaSuccess) return (int)e;
  k_project_prepare_kernel<<<capped_blocks(((long long)dim * pj_pad_n(keep) + 255) / 256, 8), 256, 0, st>>>(w, dim, keep, wimg);
  const size_t smem = pj_smem_bytes(keep);
  static std::atomic<bool> configured[MAX_DEVICES];
  int dev = -1;
  e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return SHARD_E_ARG;
  if (!configured[dev].load(std::memory_order_acquire)) {
    e = cudaFuncSetAttribute(k_project_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pj_smem_bytes(PJ_MAX_N));
    if (e != cudaSuccess) return (int)e;
    configured[dev].store(true, std::memory_order_release);
  }
  k_project_tc_kernel<<<(n + PJ_ROWS - 1) / PJ_ROWS, PJ_THREADS, smem, st>>>(flat, mean, wimg, n, dim, keep, proj_out, status);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}
