// 8-bit Lloyd-Max quantiser for tokens appended during decode, and its inverse.
//
// One warp handles one (tensor, KV head) vector of 128 channels; lane l owns
// channels 4l..4l+3.  Every arithmetic step that decides a code is a single
// correctly rounded fp32 operation in a fixed order, so codes are reproducible
// bit for bit from the same fp16 input:
//   n   = fp32(sqrt(sum of squares in fp64))      (exact sum: fp16 squares fit)
//   u   = x / n                                   (IEEE division)
//   rot = H128(u * signs) / fp32(sqrt(128))       (butterfly order h = 1..64)
//   idx = nearest codebook entry, ties to the right neighbour
#include "common.cuh"

namespace shard {

struct StreamParams {
  ShardSeq one;
  const ShardSeq* table;
  const float* codebook;
  int nkv;
  int slot;
};

__global__ void __launch_bounds__(128) stream_quantize_kernel(const __grid_constant__ StreamParams p) {
  __shared__ float cb[256];
  const ShardSeq& s = p.table ? p.table[blockIdx.y] : p.one;
  for (int i = threadIdx.x; i < 256; i += blockDim.x) cb[i] = p.codebook[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int vec = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // 0 .. 2*nkv-1
  if (vec >= 2 * p.nkv) return;
  const bool is_v = vec >= p.nkv;
  const int kv = is_v ? vec - p.nkv : vec;
  const __half* src = reinterpret_cast<const __half*>(is_v ? s.new_v : s.new_k) + kv * HD;
  uint8_t* idx_out = (is_v ? s.st_v_idx : s.st_k_idx) + ((size_t)p.slot * p.nkv + kv) * HD;
  __half* norm_out = reinterpret_cast<__half*>(is_v ? s.st_v_norm : s.st_k_norm) + (size_t)p.slot * p.nkv + kv;
  quantize_vec_warp(src, s.signs, cb, idx_out, norm_out, lane);
}

// out[kv][t][:] = fp16( fp32(fp16(H128(cb[idx]) / sqrt(128) * signs)) * fp32(norm) )
__global__ void __launch_bounds__(128) stream_dequant_kernel(const uint8_t* __restrict__ idx,
                                                             const __half* __restrict__ norm,
                                                             const float* __restrict__ signs,
                                                             const float* __restrict__ codebook,
                                                             int n_stream, int nkv, __half* __restrict__ out) {
  __shared__ float cb[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) cb[i] = codebook[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int vec = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // t * nkv + kv
  if (vec >= n_stream * nkv) return;
  const int t = vec / nkv, kv = vec - t * nkv;
  const uint32_t codes = *reinterpret_cast<const uint32_t*>(idx + (size_t)vec * HD + 4 * lane);
  float x[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = cb[(codes >> (8 * i)) & 0xff];
  fwht128_lane4(x, lane);
  const float4 sg = *reinterpret_cast<const float4*>(signs + 4 * lane);
  const float sgn[4] = {sg.x, sg.y, sg.z, sg.w};
  const float nrm = __half2float(norm[vec]);
  __half o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half unit = __float2half_rn(__fmul_rn(__fdiv_rn(x[i], SQRT_HD), sgn[i]));
    o[i] = __float2half_rn(__fmul_rn(__half2float(unit), nrm));
  }
  uint2 w;
  w.x = (uint32_t)__half_as_ushort(o[0]) | ((uint32_t)__half_as_ushort(o[1]) << 16);
  w.y = (uint32_t)__half_as_ushort(o[2]) | ((uint32_t)__half_as_ushort(o[3]) << 16);
  *reinterpret_cast<uint2*>(out + ((size_t)kv * n_stream + t) * HD + 4 * lane) = w;
}

}  // namespace shard

extern "C" int shard_b200_stream_quantize(const ShardSeq* seqs, int32_t batch, int32_t nkv, int32_t slot,
                                          const float* codebook, void* stream) {
  if (!seqs || !codebook || batch < 1 || nkv < 1 || slot < 0) return SHARD_E_ARG;
  shard::StreamParams p{};
  if (batch == 1) {
    p.one = *seqs;
    p.table = nullptr;
    if (!p.one.new_k || !p.one.new_v || !p.one.st_k_idx || !p.one.st_v_idx || !p.one.st_k_norm ||
        !p.one.st_v_norm || !p.one.signs)
      return SHARD_E_ARG;
  } else {
    p.table = seqs;
  }
  p.codebook = codebook;
  p.nkv = nkv;
  p.slot = slot;
  dim3 grid((2 * nkv + 3) / 4, batch);
  shard::stream_quantize_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(p);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" int shard_b200_stream_dequant(const uint8_t* idx, const void* norm_f16, const float* signs,
                                         const float* codebook, int32_t n_stream, int32_t nkv,
                                         void* out_f16, void* stream) {
  if (!idx || !norm_f16 || !signs || !codebook || !out_f16 || nkv < 1 || n_stream < 0) return SHARD_E_ARG;
  if (n_stream == 0) return SHARD_OK;
  const int vecs = n_stream * nkv;
  shard::stream_dequant_kernel<<<(vecs + 3) / 4, 128, 0, (cudaStream_t)stream>>>(
      idx, (const __half*)norm_f16, signs, codebook, n_stream, nkv, (__half*)out_f16);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}
