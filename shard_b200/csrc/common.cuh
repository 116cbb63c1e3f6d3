// Shared device helpers for the shard_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/shard_b200.h"

#define SHARD_CHECK_LAUNCH()                         \
  do {                                               \
    cudaError_t e__ = cudaGetLastError();            \
    if (e__ != cudaSuccess) return (int)e__;         \
  } while (0)

namespace shard {

constexpr int MAX_DEVICES = 64;   // per-device host-side state (SM counts, kernel attributes, ...)

// Number of SMs of the current device, asked from the runtime once per device.  Grids of the
// persistent / one-wave kernels are sized from it.  Returns 0 if the query fails.
inline int sm_count() {
  static int cached[MAX_DEVICES] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 0;
  int n = cached[dev];               // a racing first call writes the same value twice
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return n;
}
// grid size for a grid-stride kernel: enough blocks for `want`, at most `per_sm` per SM
inline int capped_blocks(long long want, int per_sm) {
  const long long cap = (long long)(sm_count() > 0 ? sm_count() : 1) * per_sm;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

constexpr int HD = 128;           // head_dim
constexpr int HD2 = 64;           // rotary pairs per head
constexpr int GQA = 4;            // query heads per KV head
constexpr int VQ_GROUPS = 32;     // 4-channel sub-vectors per head vector
constexpr int PART = SHARD_PART_STRIDE;
// float(sqrt(128.0)) -- the divisor of the normalised Hadamard transform
constexpr float SQRT_HD = 11.313708498984761f;
constexpr float INV_SQRT_HD = 0.08838834764831845f;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }

// 128-point Walsh-Hadamard butterfly (no normalisation) over a warp where lane l
// holds elements 4l..4l+3.  Stages run in the order h = 1, 2, 4, ..., 64 and each
// output is a single fp32 add or subtract, so results are bit-identical to a
// sequential stage-by-stage evaluation.
__device__ __forceinline__ void fwht128_lane4(float (&x)[4], int lane) {
  float a0 = __fadd_rn(x[0], x[1]), a1 = __fsub_rn(x[0], x[1]);
  float a2 = __fadd_rn(x[2], x[3]), a3 = __fsub_rn(x[2], x[3]);
  x[0] = __fadd_rn(a0, a2); x[2] = __fsub_rn(a0, a2);
  x[1] = __fadd_rn(a1, a3); x[3] = __fsub_rn(a1, a3);
#pragma unroll
  for (int bit = 1; bit < 32; bit <<= 1) {
    const bool upper = (lane & bit) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float other = __shfl_xor_sync(0xffffffffu, x[i], bit);
      x[i] = upper ? __fsub_rn(other, x[i]) : __fadd_rn(x[i], other);
    }
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Index of the nearest codebook entry as torch.bucketize + the reference's
// strict left-neighbour test do it: idx = #entries < v (capped at n-1); the left
// neighbour wins only if it is strictly closer.
__device__ __forceinline__ int lloyd_max_code(float v, const float* __restrict__ cb, int n) {
  int lo = 0, hi = n;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (cb[mid] < v) lo = mid + 1; else hi = mid;
  }
  int idx = lo < n - 1 ? lo : n - 1;
  int left = idx > 0 ? idx - 1 : 0;
  float dl = fabsf(__fsub_rn(cb[left], v));
  float dr = fabsf(__fsub_rn(cb[idx], v));
  return dl < dr ? left : idx;
}

// The same for four values at once against a 256-entry codebook: a fixed eight-step search
// (lo = number of entries below v, capped at 255) whose four chains of dependent loads run
// side by side instead of one after the other.
__device__ __forceinline__ uint32_t lloyd_max_code4_256(const float (&v)[4], const float* __restrict__ cb) {
  int lo[4] = {0, 0, 0, 0};
#pragma unroll
  for (int step = 128; step >= 1; step >>= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (cb[lo[i] + step - 1] < v[i]) lo[i] += step;
  }
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = lo[i], left = idx > 0 ? idx - 1 : 0;
    const float dl = fabsf(__fsub_rn(cb[left], v[i]));
    const float dr = fabsf(__fsub_rn(cb[idx], v[i]));
    packed |= (uint32_t)(dl < dr ? left : idx) << (8 * i);
  }
  return packed;
}

// 8-bit Lloyd-Max code of one 128-channel fp16 vector, one warp per vector (lane l owns
// channels 4l..4l+3): exact fp64 norm, IEEE division, butterfly in stage order, nearest
// codebook entry with ties to the right.  Writes 128 codes and the fp16 norm.
__device__ __forceinline__ void quantize_vec_warp(const __half* __restrict__ src, const float* __restrict__ signs,
                                                  const float* __restrict__ cb, uint8_t* __restrict__ idx_out,
                                                  __half* __restrict__ norm_out, int lane) {
  const uint2 raw = *reinterpret_cast<const uint2*>(src + 4 * lane);
  const __half2 h01 = *reinterpret_cast<const __half2*>(&raw.x);
  const __half2 h23 = *reinterpret_cast<const __half2*>(&raw.y);
  float x[4] = {__low2float(h01), __high2float(h01), __low2float(h23), __high2float(h23)};
  double ss = 0.0;
#pragma unroll
  for (int i = 0; i < 4; ++i) ss += (double)x[i] * (double)x[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  float n = (float)sqrt(ss);
  n = fmaxf(n, 1e-8f);
  const float4 sg = *reinterpret_cast<const float4*>(signs + 4 * lane);
  const float sgn[4] = {sg.x, sg.y, sg.z, sg.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = __fmul_rn(__fdiv_rn(x[i], n), sgn[i]);
  fwht128_lane4(x, lane);
  float r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) r[i] = __fdiv_rn(x[i], SQRT_HD);
  *reinterpret_cast<uint32_t*>(idx_out + 4 * lane) = lloyd_max_code4_256(r, cb);
  if (lane == 0) *norm_out = __float2half_rn(n);
}

}  // namespace shard
