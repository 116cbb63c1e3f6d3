// Layout of the exchange buffers of a sequence-split decode (one buffer per rank, identical on all
// ranks), shared by the kernels that deliver records into them and the kernels that merge:
//
//   flags [2 slots][world][nkv] u32      "rank r has delivered its records of epoch e for KV head kv"
//   parts [2 slots][world][n_q][132] f32 rank r's (max, sum-exp, 0, 0, acc[128]) per query head
//
// Epoch e uses slot e % 2.  Two slots suffice: a rank can only be writing epoch e + 2 after every
// rank has published e + 1, i.e. after every rank has finished reading epoch e in stream order.
#pragma once

#include "common.cuh"

namespace shard {

constexpr int PEER_MAX_WORLD = 16;

__host__ __device__ inline size_t peer_flag_bytes(int world, int nkv) {
  return ((size_t)2 * world * nkv * sizeof(unsigned int) + 255) & ~(size_t)255;
}
__host__ __device__ inline size_t peer_slot_floats(int world, int nkv) { return (size_t)world * nkv * GQA * PART; }

constexpr unsigned long long PEER_DEFAULT_WAIT_NS = 200ull * 1000 * 1000;   // 0.2 s

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Waits until *flag == epoch or `limit_ns` nanoseconds of the GPU's global timer have passed;
// false on time-out.
__device__ __forceinline__ bool wait_epoch(volatile unsigned int* flag, unsigned int epoch,
                                           unsigned long long limit_ns) {
  if (*flag == epoch) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (*flag == epoch) return true;
      __nanosleep(32);
    }
    if (global_timer_ns() - t0 > limit_ns) return false;
  }
}

// Merge of the `world` records of query head h, channel d, in slot `slot` of this rank's own
// exchange buffer, in rank order: the operations and order of decode_combine_kernel, so every
// rank computes bit-identical output.
__device__ __forceinline__ __half merge_rank_records(const unsigned char* own_buf, int world, int nkv, int slot,
                                                     int h, int d) {
  const int n_q = nkv * GQA;
  const float* base = reinterpret_cast<const float*>(own_buf + peer_flag_bytes(world, nkv)) +
                      slot * peer_slot_floats(world, nkv) + (size_t)h * PART;
  const size_t pstride = (size_t)n_q * PART;
  // every rank's (max, sum-exp, channel) goes out as one batch of loads: one round trip instead of
  // one per rank
  float m[PEER_MAX_WORLD], l[PEER_MAX_WORLD], a[PEER_MAX_WORLD];
#pragma unroll
  for (int r = 0; r < PEER_MAX_WORLD; ++r) {
    const float* rec = base + r * pstride;
    m[r] = r < world ? __ldcg(rec) : neg_inf();
    l[r] = r < world ? __ldcg(rec + 1) : 0.f;
    a[r] = r < world ? __ldcg(rec + 4 + d) : 0.f;
  }
  float M = neg_inf();
#pragma unroll
  for (int r = 0; r < PEER_MAX_WORLD; ++r) M = fmaxf(M, m[r]);
  float L = 0.f, acc = 0.f;
#pragma unroll
  for (int r = 0; r < PEER_MAX_WORLD; ++r) {
    if (r < world) {
      const float wt = (m[r] == neg_inf()) ? 0.f : exp2f((m[r] - M) * LOG2E);
      L = fmaf(wt, l[r], L);
      acc = fmaf(wt, a[r], acc);
    }
  }
  return __float2half_rn(acc / L);
}

}  // namespace shard
