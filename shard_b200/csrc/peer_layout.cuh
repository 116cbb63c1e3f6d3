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

}  // namespace shard
