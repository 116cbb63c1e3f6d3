// Prefill compressor kernels: RoPE removal, the two-stage int4
// quantiser with nibble packing, Hadamard + per-channel normalisation of V and
// nearest-centroid VQ assignment.
//
// Every stage that ends in an integer code uses explicitly rounded fp32
// operations (__fmul_rn/__fadd_rn/__fdiv_rn, rintf) in the order the reference's
// PyTorch code performs them, so that the codes are bit-identical for identical
// fp32 inputs.  Reductions that decide codes (min, max, max-abs) are
// order-independent.
#include "common.cuh"

namespace shard {

// ---------------------------------------------------------------------------
// undo RoPE: flat[t][kv*128+d] = k*cos - rotate_half(k)*sin, fp32
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) undo_rope_kernel(const __half* __restrict__ k, int64_t head_stride,
                                                        int64_t tok_stride, int nkv, int n, int pos_start,
                                                        const float* __restrict__ inv_freq,
                                                        float* __restrict__ flat) {
  // one block per token; thread (kv_sub, i) covers pair i of several heads
  const int t = blockIdx.x;
  const int i = threadIdx.x & 63;
  const float phase = __fmul_rn((float)(pos_start + t), inv_freq[i]);
  float sn, cs;
  sincosf(phase, &sn, &cs);
  for (int kv = threadIdx.x >> 6; kv < nkv; kv += 2) {
    const __half* row = k + kv * head_stride + (int64_t)t * tok_stride;
    const float lo = __half2float(row[i]);
    const float hi = __half2float(row[i + 64]);
    float* o = flat + (size_t)t * nkv * HD + kv * HD;
    // d < 64: k[d]*cos - (-k[d+64])*sin ; d >= 64: k[d]*cos - k[d-64]*sin
    o[i] = __fadd_rn(__fmul_rn(lo, cs), __fmul_rn(hi, sn));
    o[i + 64] = __fsub_rn(__fmul_rn(hi, cs), __fmul_rn(lo, sn));
  }
}

// ---------------------------------------------------------------------------
// K quantiser
// ---------------------------------------------------------------------------
// Monotone map float -> uint32 so that unsigned atomicMin/atomicMax order floats.
__device__ __forceinline__ uint32_t f2ord(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ord2f(uint32_t o) {
  return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}

// ws layout (uint32): [0,keep) ordered min, [keep,2keep) ordered max, [2keep,3keep) max|xhat| bits
__global__ void kq_init_kernel(uint32_t* ws, int keep) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j < keep) { ws[j] = 0xffffffffu; ws[keep + j] = 0u; ws[2 * keep + j] = 0u; }
}

constexpr int KQ_ROWS = 64;  // rows per block

__global__ void __launch_bounds__(256) kq_minmax_kernel(const float* __restrict__ proj, int n, int keep,
                                                        uint32_t* __restrict__ ws) {
  const int r0 = blockIdx.x * KQ_ROWS;
  for (int j = threadIdx.x; j < keep; j += blockDim.x) {
    float lo = __int_as_float(0x7f800000), hi = neg_inf();
    const int r1 = min(r0 + KQ_ROWS, n);
    for (int r = r0; r < r1; ++r) {
      const float v = proj[(size_t)r * keep + j];
      lo = fminf(lo, v); hi = fmaxf(hi, v);
    }
    atomicMin(ws + j, f2ord(lo));
    atomicMax(ws + keep + j, f2ord(hi));
  }
}

__device__ __forceinline__ float kq_xhat(float x, float lo, float rng, float levels) {
  float unit = __fdiv_rn(__fsub_rn(x, lo), rng);
  unit = fminf(fmaxf(unit, 0.f), 1.f);
  float code = rintf(__fmul_rn(unit, levels));
  code = fminf(fmaxf(code, 0.f), levels);
  return __fadd_rn(__fmul_rn(__fdiv_rn(code, levels), rng), lo);
}

__global__ void __launch_bounds__(256) kq_absmax_kernel(const float* __restrict__ proj,
                                                        const int32_t* __restrict__ alloc, int n, int keep,
                                                        uint32_t* __restrict__ ws) {
  const int r0 = blockIdx.x * KQ_ROWS;
  for (int j = threadIdx.x; j < keep; j += blockDim.x) {
    const int bits = alloc[j];
    if (bits == 0) continue;
    const float lo = ord2f(ws[j]);
    const float rng = fmaxf(__fsub_rn(ord2f(ws[keep + j]), lo), 1e-6f);
    const float levels = (float)((1 << bits) - 1);
    float am = 0.f;
    const int r1 = min(r0 + KQ_ROWS, n);
    for (int r = r0; r < r1; ++r) am = fmaxf(am, fabsf(kq_xhat(proj[(size_t)r * keep + j], lo, rng, levels)));
    atomicMax(ws + 2 * keep + j, __float_as_uint(am));  // non-negative floats order as integers
  }
}

__global__ void kq_scale_kernel(const uint32_t* __restrict__ ws, int keep, float* __restrict__ coeff_scale) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j < keep) coeff_scale[j] = __fdiv_rn(fmaxf(__uint_as_float(ws[2 * keep + j]), 1e-6f), 7.0f);
}

__global__ void __launch_bounds__(256) kq_pack_kernel(const float* __restrict__ proj,
                                                      const int32_t* __restrict__ alloc, int n, int keep,
                                                      const uint32_t* __restrict__ ws,
                                                      const float* __restrict__ coeff_scale,
                                                      uint8_t* __restrict__ packed) {
  const int half = keep >> 1;
  const size_t total = (size_t)n * half;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / half;
    const int j = (int)(i - r * half) * 2;
    const float2 x = *reinterpret_cast<const float2*>(proj + r * keep + j);
    int q[2];
    const float xv[2] = {x.x, x.y};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int bits = alloc[j + e];
      float xh = 0.f;
      if (bits) {
        const float lo = ord2f(ws[j + e]);
        const float rng = fmaxf(__fsub_rn(ord2f(ws[keep + j + e]), lo), 1e-6f);
        xh = kq_xhat(xv[e], lo, rng, (float)((1 << bits) - 1));
      }
      float v = rintf(__fdiv_rn(xh, coeff_scale[j + e]));
      v = fminf(fmaxf(v, -7.f), 7.f);
      q[e] = (int)v;
    }
    packed[i] = (uint8_t)(((q[0] + 8) & 15) | (((q[1] + 8) & 15) << 4));
  }
}

__global__ void int4_pack_kernel(const int8_t* __restrict__ q, int64_t n_values, uint8_t* __restrict__ packed) {
  const int64_t n_bytes = (n_values + 1) >> 1;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_bytes;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int lo = q[2 * i];
    const int hi = (2 * i + 1 < n_values) ? q[2 * i + 1] : 0;
    packed[i] = (uint8_t)(((lo + 8) & 15) | (((hi + 8) & 15) << 4));
  }
}

// ---------------------------------------------------------------------------
// V: Hadamard + per-channel max-abs normalisation
// ---------------------------------------------------------------------------
// pass 1: x = H128(v) / sqrt(128); ch_max = max_t |x|   (uint atomicMax on non-negative floats)
__global__ void __launch_bounds__(256) v_rotate_kernel(const __half* __restrict__ v, int64_t head_stride,
                                                       int64_t tok_stride, int nkv, int n,
                                                       float* __restrict__ x, uint32_t* __restrict__ ch_max) {
  const int lane = threadIdx.x & 31;
  const int kv = blockIdx.y;
  float am[4] = {0.f, 0.f, 0.f, 0.f};
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < n; t += gridDim.x * (blockDim.x >> 5)) {
    const uint2 raw = *reinterpret_cast<const uint2*>(v + kv * head_stride + (int64_t)t * tok_stride + 4 * lane);
    const __half2 h01 = *reinterpret_cast<const __half2*>(&raw.x);
    const __half2 h23 = *reinterpret_cast<const __half2*>(&raw.y);
    float y[4] = {__low2float(h01), __high2float(h01), __low2float(h23), __high2float(h23)};
    fwht128_lane4(y, lane);
#pragma unroll
    for (int i = 0; i < 4; ++i) { y[i] = __fdiv_rn(y[i], SQRT_HD); am[i] = fmaxf(am[i], fabsf(y[i])); }
    *reinterpret_cast<float4*>(x + ((size_t)kv * n + t) * HD + 4 * lane) = make_float4(y[0], y[1], y[2], y[3]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) atomicMax(ch_max + kv * HD + 4 * lane + i, __float_as_uint(am[i]));
}

__global__ void v_clamp_kernel(float* ch_max, int count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) ch_max[i] = fmaxf(ch_max[i], 1e-8f);
}

// pass 2: x /= ch_max
__global__ void __launch_bounds__(256) v_normalise_kernel(float* __restrict__ x, const float* __restrict__ ch_max,
                                                          int nkv, int n) {
  const size_t total4 = (size_t)nkv * n * (HD / 4);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4;
       i += (size_t)gridDim.x * blockDim.x) {
    const int d4 = (int)(i & 31);
    const int kv = (int)(i / ((size_t)n * 32));
    float4 y = reinterpret_cast<float4*>(x)[i];
    const float4 c = *reinterpret_cast<const float4*>(ch_max + kv * HD + 4 * d4);
    y.x = __fdiv_rn(y.x, c.x); y.y = __fdiv_rn(y.y, c.y); y.z = __fdiv_rn(y.z, c.z); y.w = __fdiv_rn(y.w, c.w);
    reinterpret_cast<float4*>(x)[i] = y;
  }
}

// ---------------------------------------------------------------------------
// VQ assign: argmin_k ((x0-c0)^2 + (x1-c1)^2) + (x2-c2)^2) + (x3-c3)^2, first minimum
// ---------------------------------------------------------------------------
// With ACCUMULATE the kernel also does the k-means statistics of the same pass: per-centroid sums
// and counts are collected in shared memory (atomics) and added to `sums` / `counts` once per CTA,
// replacing two index_add_ passes over all points.  The order of those additions is not fixed,
// exactly as with index_add_ on a GPU.
template <bool ACCUMULATE>
__global__ void __launch_bounds__(256) vq_assign_kernel(const float4* __restrict__ x,
                                                        const float4* __restrict__ centroids, int64_t n,
                                                        uint8_t* __restrict__ idx_u8, int64_t* __restrict__ idx_i64,
                                                        float* __restrict__ sums, float* __restrict__ counts) {
  __shared__ float4 cb[256];
  __shared__ float acc_s[ACCUMULATE ? 256 * 5 : 1];
  cb[threadIdx.x] = centroids[threadIdx.x];
  if (ACCUMULATE)
    for (int i = threadIdx.x; i < 256 * 5; i += 256) acc_s[i] = 0.f;
  __syncthreads();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 p = x[i];
    float best = __int_as_float(0x7f800000);
    int arg = 0;
#pragma unroll 8
    for (int k = 0; k < 256; ++k) {
      const float4 c = cb[k];
      const float d0 = __fsub_rn(p.x, c.x), d1 = __fsub_rn(p.y, c.y);
      const float d2 = __fsub_rn(p.z, c.z), d3 = __fsub_rn(p.w, c.w);
      float dist = __fadd_rn(__fmul_rn(d0, d0), __fmul_rn(d1, d1));
      dist = __fadd_rn(dist, __fmul_rn(d2, d2));
      dist = __fadd_rn(dist, __fmul_rn(d3, d3));
      if (dist < best) { best = dist; arg = k; }
    }
    idx_u8[i] = (uint8_t)arg;
    if (idx_i64) idx_i64[i] = arg;
    if (ACCUMULATE) {
      atomicAdd(&acc_s[arg * 5 + 0], p.x);
      atomicAdd(&acc_s[arg * 5 + 1], p.y);
      atomicAdd(&acc_s[arg * 5 + 2], p.z);
      atomicAdd(&acc_s[arg * 5 + 3], p.w);
      atomicAdd(&acc_s[arg * 5 + 4], 1.f);
    }
  }
  if (ACCUMULATE) {
    __syncthreads();
    const int k = threadIdx.x;
    if (acc_s[k * 5 + 4] > 0.f) {
#pragma unroll
      for (int c = 0; c < 4; ++c) atomicAdd(&sums[k * 4 + c], acc_s[k * 5 + c]);
      atomicAdd(&counts[k], acc_s[k * 5 + 4]);
    }
  }
}

}  // namespace shard

using namespace shard;

extern "C" int shard_b200_undo_rope(const void* k_f16, int64_t head_stride, int64_t tok_stride, int32_t nkv,
                                    int32_t n, int32_t pos_start, const float* inv_freq, float* flat_out,
                                    void* stream) {
  if (!k_f16 || !inv_freq || !flat_out || nkv < 1 || n < 0) return SHARD_E_ARG;
  if (n == 0) return SHARD_OK;
  undo_rope_kernel<<<n, 128, 0, (cudaStream_t)stream>>>((const __half*)k_f16, head_stride, tok_stride, nkv, n,
                                                         pos_start, inv_freq, flat_out);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" size_t shard_b200_k_quantize_workspace_bytes(int32_t n, int32_t keep) {
  (void)n;
  return (size_t)3 * (keep > 0 ? keep : 0) * sizeof(uint32_t);
}

extern "C" int shard_b200_k_quantize_pack(const float* proj, const int32_t* alloc_bits, int32_t n, int32_t keep,
                                          float* coeff_scale_out, uint8_t* packed_out, void* workspace,
                                          size_t workspace_bytes, void* stream) {
  if (!proj || !alloc_bits || !coeff_scale_out || !packed_out || !workspace || n < 1 || keep < 2 || (keep & 1))
    return SHARD_E_ARG;
  if (workspace_bytes < shard_b200_k_quantize_workspace_bytes(n, keep)) return SHARD_E_WORKSPACE;
  if ((uintptr_t)proj & 7) return SHARD_E_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t* ws = (uint32_t*)workspace;
  const int row_blocks = (n + KQ_ROWS - 1) / KQ_ROWS;
  kq_init_kernel<<<(keep + 255) / 256, 256, 0, st>>>(ws, keep);
  kq_minmax_kernel<<<row_blocks, 256, 0, st>>>(proj, n, keep, ws);
  kq_absmax_kernel<<<row_blocks, 256, 0, st>>>(proj, alloc_bits, n, keep, ws);
  kq_scale_kernel<<<(keep + 255) / 256, 256, 0, st>>>(ws, keep, coeff_scale_out);
  const size_t total = (size_t)n * (keep / 2);
  const int blocks = capped_blocks((long long)((total + 255) / 256), 16);
  kq_pack_kernel<<<blocks, 256, 0, st>>>(proj, alloc_bits, n, keep, ws, coeff_scale_out, packed_out);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" int shard_b200_int4_pack(const int8_t* q, int64_t n_values, uint8_t* packed_out, void* stream) {
  if (!q || !packed_out || n_values < 0) return SHARD_E_ARG;
  if (n_values == 0) return SHARD_OK;
  const int64_t n_bytes = (n_values + 1) / 2;
  const int blocks = capped_blocks((n_bytes + 255) / 256, 16);
  int4_pack_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(q, n_values, packed_out);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" int shard_b200_v_hadamard_normalise(const void* v_f16, int64_t head_stride, int64_t tok_stride,
                                               int32_t nkv, int32_t n, float* x_out, float* ch_max_out,
                                               void* stream) {
  if (!v_f16 || !x_out || !ch_max_out || nkv < 1 || n < 1) return SHARD_E_ARG;
  if (((uintptr_t)v_f16 & 7) || (head_stride & 3) || (tok_stride & 3) || ((uintptr_t)x_out & 15))
    return SHARD_E_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(ch_max_out, 0, (size_t)nkv * HD * sizeof(float), st);
  if (e != cudaSuccess) return (int)e;
  const int bx = capped_blocks((n + 7) / 8, 2);
  v_rotate_kernel<<<dim3(bx, nkv), 256, 0, st>>>((const __half*)v_f16, head_stride, tok_stride, nkv, n, x_out,
                                                 (uint32_t*)ch_max_out);
  v_clamp_kernel<<<(nkv * HD + 255) / 256, 256, 0, st>>>(ch_max_out, nkv * HD);
  const size_t total4 = (size_t)nkv * n * 32;
  const int blocks = capped_blocks((long long)((total4 + 255) / 256), 16);
  v_normalise_kernel<<<blocks, 256, 0, st>>>(x_out, ch_max_out, nkv, n);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" int shard_b200_vq_assign(const float* x, const float* centroids, int64_t n, uint8_t* idx_u8,
                                    int64_t* idx_i64, void* stream) {
  if (!x || !centroids || !idx_u8 || n < 0) return SHARD_E_ARG;
  if (((uintptr_t)x | (uintptr_t)centroids) & 15) return SHARD_E_ALIGN;
  if (n == 0) return SHARD_OK;
  const int64_t want = (n + 255) / 256;
  const int blocks = capped_blocks(want, 8);
  vq_assign_kernel<false><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float4*)x, (const float4*)centroids, n,
                                                                     idx_u8, idx_i64, nullptr, nullptr);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" int shard_b200_vq_assign_accumulate(const float* x, const float* centroids, int64_t n, uint8_t* idx_u8,
                                               float* sums, float* counts, void* stream) {
  if (!x || !centroids || !idx_u8 || !sums || !counts || n < 0) return SHARD_E_ARG;
  if (((uintptr_t)x | (uintptr_t)centroids) & 15) return SHARD_E_ALIGN;
  if (n == 0) return SHARD_OK;
  const int64_t want = (n + 255) / 256;
  const int blocks = capped_blocks(want, 8);
  vq_assign_kernel<true><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float4*)x, (const float4*)centroids, n,
                                                                    idx_u8, nullptr, sums, counts);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}
