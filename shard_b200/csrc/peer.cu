// Sequence-split decode: exchange of the per-rank partial records over NVLink peer memory and
// their log-sum-exp merge, in one kernel.
//
// Every rank owns one exchange buffer (plain cudaMalloc memory, opened by the other ranks of
// the node through CUDA IPC; layout in peer_layout.cuh).  Per layer-step and rank:
//
//   (1) this rank's four records per KV head go into slot e % 2 of EVERY rank's buffer with plain
//       peer stores,
//   (2) system-scope fence, then the epoch number is published in every rank's flag word,
//   (3) wait -- bounded by the global timer -- until all `world` flag words of the own buffer show
//       the epoch,
//   (4) merge the `world` records of the own buffer in rank order: same operations and order as
//       decode_combine_kernel, so every rank gets bit-identical output.
//
// seqsplit_exchange_merge_kernel does (1)-(4) for a record that lies in this rank's memory.
// seqsplit_wait_merge_kernel does (3)-(4) only: (1)-(2) were done by the decode launch itself
// (the CTA that combines a KV head's split-KV records delivers the result, decode_common.cuh).
// It is launched with programmatic stream serialization, so it is resident and polling while
// the decode launch in front of it still runs, and the merge starts the moment the last flag lands.
// No multicast, no multimem: plain loads and stores on peer pointers.
#include <cstring>

#include "peer_layout.cuh"
#include "tcgen05.cuh"

namespace shard {

struct PeerParams {
  unsigned char* bufs[PEER_MAX_WORLD];   // exchange buffer of every rank (own entry = local pointer)
  const float* my_part;                  // [n_q][132]
  void* out;                             // fp16 [n_q][128]
  int* status;                           // set to 1 when the bounded wait gave up (may be null)
  int rank, world, nkv;
  unsigned int epoch;
  unsigned long long wait_ns;            // bound of the flag wait
};

// (4): merge of the `world` records of KV head kv in the own buffer, in rank order
__device__ __forceinline__ void merge_own_buffer(const PeerParams& p, int kv, int tid, int slot) {
  const int h = kv * GQA + (tid >> 7), d = tid & (HD - 1);
  reinterpret_cast<__half*>(p.out)[(size_t)h * HD + d] = merge_rank_records(p.bufs[p.rank], p.world, p.nkv, slot, h, d);
}

__global__ void __launch_bounds__(GQA* HD) seqsplit_exchange_merge_kernel(const __grid_constant__ PeerParams p) {
  __shared__ int timed_out;
  const int kv = blockIdx.x, tid = threadIdx.x;
  const int slot = (int)(p.epoch & 1u);
  const int n_q = p.nkv * GQA;
  const size_t flag_bytes = peer_flag_bytes(p.world, p.nkv);
  const size_t slot_floats = peer_slot_floats(p.world, p.nkv);
  if (tid == 0) timed_out = 0;

  // (1) this rank's four records of KV head kv -> every rank's buffer
  const float4* src = reinterpret_cast<const float4*>(p.my_part + (size_t)kv * GQA * PART);
  constexpr int N4 = GQA * PART / 4;   // 132 float4
  for (int r = 0; r < p.world; ++r) {
    float* parts = reinterpret_cast<float*>(p.bufs[r] + flag_bytes) + slot * slot_floats;
    float4* dst = reinterpret_cast<float4*>(parts + ((size_t)p.rank * n_q + (size_t)kv * GQA) * PART);
    for (int i = tid; i < N4; i += blockDim.x) dst[i] = src[i];
  }
  // (2) make the records visible system-wide, then publish the epoch
  __threadfence_system();
  __syncthreads();
  if (tid < p.world) {
    volatile unsigned int* flag =
        reinterpret_cast<volatile unsigned int*>(p.bufs[tid]) + ((size_t)slot * p.world + p.rank) * p.nkv + kv;
    *flag = p.epoch;
  }
  // (3) bounded wait for everybody's records of this epoch in the own buffer
  if (tid < p.world) {
    volatile unsigned int* flag =
        reinterpret_cast<volatile unsigned int*>(p.bufs[p.rank]) + ((size_t)slot * p.world + tid) * p.nkv + kv;
    if (!wait_epoch(flag, p.epoch, p.wait_ns)) timed_out = 1;
    __threadfence_system();
  }
  __syncthreads();
  if (timed_out) {
    if (tid == 0 && p.status) atomicExch(p.status, 1);
    return;
  }
  merge_own_buffer(p, kv, tid, slot);
}

// Steps (3)-(4) for records that the decode launch in front of this kernel delivers itself.
__global__ void __launch_bounds__(GQA* HD) seqsplit_wait_merge_kernel(const __grid_constant__ PeerParams p) {
  __shared__ int timed_out;
  const int kv = blockIdx.x, tid = threadIdx.x;
  const int slot = (int)(p.epoch & 1u);
  griddep_launch();
  if (tid == 0) timed_out = 0;
  __syncthreads();
  if (tid < p.world) {
    volatile unsigned int* flag =
        reinterpret_cast<volatile unsigned int*>(p.bufs[p.rank]) + ((size_t)slot * p.world + tid) * p.nkv + kv;
    if (!wait_epoch(flag, p.epoch, p.wait_ns)) timed_out = 1;
    __threadfence_system();
  }
  __syncthreads();
  // everything in front of this kernel in the stream has finished (whoever follows this kernel
  // with a programmatic launch of its own relies on that, also when the wait above gave up)
  griddep_wait();
  if (timed_out) {
    if (tid == 0 && p.status) atomicExch(p.status, 1);
    return;
  }
  merge_own_buffer(p, kv, tid, slot);
}

}  // namespace shard

using namespace shard;

extern "C" size_t shard_b200_peer_buffer_bytes(int32_t world, int32_t nkv) {
  if (world < 1 || world > PEER_MAX_WORLD || nkv < 1) return 0;
  return peer_flag_bytes(world, nkv) + 2 * peer_slot_floats(world, nkv) * sizeof(float);
}

extern "C" int shard_b200_peer_alloc(size_t bytes, void** ptr_out, void* handle_out_64) {
  if (!ptr_out || !handle_out_64 || bytes == 0) return SHARD_E_ARG;
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(ptr, 0, bytes);
  if (e != cudaSuccess) { cudaFree(ptr); return (int)e; }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle_out_64), ptr);
  if (e != cudaSuccess) { cudaFree(ptr); return (int)e; }
  *ptr_out = ptr;
  return SHARD_OK;
}

extern "C" int shard_b200_peer_open(const void* handle_64, void** ptr_out) {
  if (!handle_64 || !ptr_out) return SHARD_E_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? SHARD_OK : (int)e;
}

extern "C" int shard_b200_peer_close(void* ptr) {
  if (!ptr) return SHARD_E_ARG;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? SHARD_OK : (int)e;
}

extern "C" int shard_b200_peer_free(void* ptr) {
  if (!ptr) return SHARD_E_ARG;
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? SHARD_OK : (int)e;
}

static int fill_peer_params(PeerParams& p, void* const* bufs_host, int32_t rank, int32_t world, int32_t nkv,
                            uint32_t epoch, void* out_f16, int* status_dev, uint32_t timeout_us) {
  if (!bufs_host || !out_f16 || world < 1 || world > PEER_MAX_WORLD || rank < 0 || rank >= world || nkv < 1 ||
      epoch == 0)
    return SHARD_E_ARG;
  for (int r = 0; r < world; ++r) {
    if (!bufs_host[r]) return SHARD_E_ARG;
    p.bufs[r] = reinterpret_cast<unsigned char*>(bufs_host[r]);
  }
  p.out = out_f16;
  p.status = status_dev;
  p.rank = rank;
  p.world = world;
  p.nkv = nkv;
  p.epoch = epoch;
  p.wait_ns = timeout_us ? (unsigned long long)timeout_us * 1000ull : PEER_DEFAULT_WAIT_NS;
  return SHARD_OK;
}

extern "C" int shard_b200_seqsplit_merge(const float* my_part, void* const* bufs_host, int32_t rank, int32_t world,
                                         int32_t nkv, uint32_t epoch, void* out_f16, int* status_dev,
                                         uint32_t timeout_us, void* stream) {
  if (!my_part) return SHARD_E_ARG;
  if ((uintptr_t)my_part & 15) return SHARD_E_ALIGN;
  PeerParams p{};
  int rc = fill_peer_params(p, bufs_host, rank, world, nkv, epoch, out_f16, status_dev, timeout_us);
  if (rc != SHARD_OK) return rc;
  p.my_part = my_part;
  seqsplit_exchange_merge_kernel<<<nkv, GQA * HD, 0, (cudaStream_t)stream>>>(p);
  SHARD_CHECK_LAUNCH();
  return SHARD_OK;
}

extern "C" int shard_b200_seqsplit_wait_merge(void* const* bufs_host, int32_t rank, int32_t world, int32_t nkv,
                                              uint32_t epoch, void* out_f16, int* status_dev, uint32_t timeout_us,
                                              void* stream) {
  PeerParams p{};
  int rc = fill_peer_params(p, bufs_host, rank, world, nkv, epoch, out_f16, status_dev, timeout_us);
  if (rc != SHARD_OK) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nkv);
  cfg.blockDim = dim3(GQA * HD);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, seqsplit_wait_merge_kernel, p);
  return e == cudaSuccess ? SHARD_OK : (int)e;
}
