// Micro-benchmark of tcgen05.mma (kind::f16, fp16 operands, fp32 accumulation, cta_group::1) on
// one CTA per SM: cycles per instruction as seen by the issuing thread (time until the last
// instruction has been handed over) and until the work has completed (commit + mbarrier wait), for
// the shapes the decode kernel uses.  Operands are all-ones data; results are not checked, only
// timed.  Build and run:
//
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o tcgen05_mma_rate tcgen05_mma_rate.cu
//   ./tcgen05_mma_rate
//
// Every wait is bounded (about 40 ms); a case that times out prints "timeout" and the program
// goes on.
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < 4096; ++i)
    if (mbar_try(bar, parity, 10000)) return true;
  return false;
}
__device__ __forceinline__ void umma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__host__ __device__ constexpr uint32_t mk_idesc(int M, int N, bool a_mn_major = false) {
  return (1u << 4) | ((a_mn_major ? 1u : 0u) << 15) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

enum Case {
  N128_SS, N128_TS, N128_TS_LD, N64_TS, N16_SS, N16_TS, N16_TS_TWO_ACC, M64_N128_SS, M64_N16_SS, TILE_MIX,
  TILE_MIX_MN, TILE_MIX_MN_SMEM_LIGHT, TILE_MIX_MN_SMEM_HEAVY, TILE_MIX_MN_COMMITS, N_CASES
};

// out[0]: cycles until the group has completed, out[1]: cycles the issuing thread spent issuing,
// out[2]: 16-byte shared-memory loads + stores per lane done by the other warps meanwhile
template <int which>
__global__ void __launch_bounds__(512) bench(int reps, long long* out) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint32_t slot;
  __shared__ uint64_t bar;
  __shared__ uint64_t side_bars[8];   // commits nobody waits for (the kernel's per-third and per-product hand-overs)
  __shared__ volatile int stop;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < 128 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (tid == 0) {
    mbar_init(smem_u32(&bar), 1);
    for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&side_bars[i]), 1);
    stop = 0;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tb = slot;
  const uint32_t a_u = smem_u32(smem), b_u = a_u + 64 * 1024;     // A: 4 atoms of 16 KB; B: 4 atoms of 16 KB
  const uint64_t ad = desc_sw128(a_u, 16, 1024), bd = desc_sw128(b_u, 16, 1024);
  long long t_total = 0, t_issue = 0;
  bool timed_out = false;
  uint32_t parity = 0;
  const bool load_warps = which == N128_TS_LD;
  constexpr bool tile_mix = which == TILE_MIX || which >= TILE_MIX_MN;
  constexpr bool smem_warps = which == TILE_MIX_MN_SMEM_LIGHT || which == TILE_MIX_MN_SMEM_HEAVY;
  const uint64_t ad_mn = desc_sw128(a_u, 16384, 1024);   // A as the decode kernel's V tile: MN-major, two 16 KB halves
  if (warp == 0) {
    for (int r = 0; r < reps && !timed_out; ++r) {
      const long long t0 = clock64();
      if (lane == 0) {
#pragma unroll 1
        for (int rr = 0; rr < 4; ++rr) {
          if (tile_mix) {
            // one tile of the decode kernel: 13 k-steps of 128 columns, then 8 + 8 of 16 columns
#pragma unroll
            for (int k = 0; k < 13; ++k) {
              umma_ts(tb, tb + 256 + 8 * k, bd + (uint64_t)(((k >> 2) * 16384u + (k & 3) * 32u) >> 4), mk_idesc(128, 128), k > 0);
              if (which == TILE_MIX_MN_COMMITS && (k == 3 || k == 7 || k == 12)) umma_commit(smem_u32(&side_bars[k >> 2]));
            }
            if (which == TILE_MIX_MN_COMMITS) umma_commit(smem_u32(&side_bars[4]));
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_ts(tb + 128, tb + 8 * k, bd + (uint64_t)(((k >> 2) * 2048u + (k & 3) * 32u) >> 4), mk_idesc(128, 16), k > 0);
            if (which == TILE_MIX_MN_COMMITS) umma_commit(smem_u32(&side_bars[5]));
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_ss(tb + 160, (which == TILE_MIX ? ad : ad_mn) + (uint64_t)((k * 2048u) >> 4),
                      bd + (uint64_t)(((k >> 2) * 2048u + (k & 3) * 32u) >> 4), mk_idesc(128, 16, which != TILE_MIX), k > 0);
            if (which == TILE_MIX_MN_COMMITS) umma_commit(smem_u32(&side_bars[6]));
          } else {
#pragma unroll
            for (int k = 0; k < 12; ++k) {
              const uint64_t off = (uint64_t)(((k >> 2) * 16384u + (k & 3) * 32u) >> 4);
              const uint32_t acc = (uint32_t)((k | rr) > 0);
              switch (which) {
                case N128_SS: umma_ss(tb, ad + off, bd + off, mk_idesc(128, 128), acc); break;
                case N128_TS: case N128_TS_LD: umma_ts(tb, tb + 256 + 8 * k, bd + off, mk_idesc(128, 128), acc); break;
                case N64_TS: umma_ts(tb, tb + 256 + 8 * k, bd + off, mk_idesc(128, 64), acc); break;
                case N16_SS: umma_ss(tb, ad + off, bd + off, mk_idesc(128, 16), acc); break;
                case N16_TS: umma_ts(tb, tb + 256 + 8 * k, bd + off, mk_idesc(128, 16), acc); break;
                case N16_TS_TWO_ACC: umma_ts(tb + 32 * (k & 1), tb + 256 + 8 * k, bd + off, mk_idesc(128, 16), (uint32_t)((k | rr) > 1)); break;
                case M64_N128_SS: umma_ss(tb, ad + off, bd + off, mk_idesc(64, 128), acc); break;
                case M64_N16_SS: umma_ss(tb, ad + off, bd + off, mk_idesc(64, 16), acc); break;
                default: break;
              }
            }
          }
        }
        t_issue += clock64() - t0;
        umma_commit(smem_u32(&bar));
      }
      __syncwarp();
      timed_out = !mbar_wait(smem_u32(&bar), parity);
      parity ^= 1u;
      t_total += clock64() - t0;
    }
    if (lane == 0) stop = 1;
    if (lane == 0 && blockIdx.x == 0) { out[0] = timed_out ? -1 : t_total; out[1] = t_issue; }
  } else if (load_warps && warp < 4) {
    // keep tensor memory busy: every warp reads 16 columns of its lane quarter over and over
    uint32_t acc = 0;
    const uint32_t taddr = tb + 128 + ((uint32_t)(warp * 32) << 16);
    for (int i = 0; i < 200000 && !stop; ++i) {
      uint32_t r[16];
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                   : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                     "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                   : "r"(taddr + 16 * (i & 7)));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      acc ^= r[0] ^ r[15];
    }
    if (acc == 0x12345678u) out[3] = acc;
  } else if (smem_warps) {
    // keep the shared-memory pipe busy the way the decode kernel's V expansion does: every lane
    // loads and stores 16 bytes of a scratch area (2 KB per warp, inside the B operand: only the
    // timing matters), with idle arithmetic in between in the light case
    uint4* scratch = reinterpret_cast<uint4*>(smem + 128 * 1024 - 15 * 2048) + (warp - 1) * 128;
    uint4 v = make_uint4(tid, 0u, 0u, 0u);
    long long n = 0;
    for (int i = 0; i < 4000000 && !stop; ++i) {
      uint4 x[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) x[j] = scratch[((i + j) * 32 + lane) & 127];
#pragma unroll
      for (int j = 0; j < 4; ++j) { v.x ^= x[j].x; v.y += x[j].y; }
#pragma unroll
      for (int j = 0; j < 4; ++j) scratch[((i + j + 2) * 32 + lane) & 127] = v;
      n += 8;
      if (which == TILE_MIX_MN_SMEM_LIGHT) {
#pragma unroll 1
        for (int j = 0; j < 48; ++j) v.z = v.z * 1664525u + 1013904223u;
      }
    }
    if (lane == 0 && blockIdx.x == 0) atomicAdd(reinterpret_cast<unsigned long long*>(out + 2), (unsigned long long)n);
    if (v.z == 0x12345678u) out[3] = v.x;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(512) : "memory");
}

template <int C>
void launch_one(int reps, long long* d) {
  cudaFuncSetAttribute(bench<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, 130 * 1024);
  // the cases with shared-memory traffic run 15 traffic warps beside the issuing warp
  const int threads = (C == TILE_MIX_MN_SMEM_LIGHT || C == TILE_MIX_MN_SMEM_HEAVY) ? 512 : 128;
  bench<C><<<148, threads, 130 * 1024>>>(reps, d);
}
void launch(int c, int reps, long long* d) {
  switch (c) {
    case N128_SS: launch_one<N128_SS>(reps, d); break;
    case N128_TS: launch_one<N128_TS>(reps, d); break;
    case N128_TS_LD: launch_one<N128_TS_LD>(reps, d); break;
    case N64_TS: launch_one<N64_TS>(reps, d); break;
    case N16_SS: launch_one<N16_SS>(reps, d); break;
    case N16_TS: launch_one<N16_TS>(reps, d); break;
    case N16_TS_TWO_ACC: launch_one<N16_TS_TWO_ACC>(reps, d); break;
    case M64_N128_SS: launch_one<M64_N128_SS>(reps, d); break;
    case M64_N16_SS: launch_one<M64_N16_SS>(reps, d); break;
    case TILE_MIX_MN: launch_one<TILE_MIX_MN>(reps, d); break;
    case TILE_MIX_MN_SMEM_LIGHT: launch_one<TILE_MIX_MN_SMEM_LIGHT>(reps, d); break;
    case TILE_MIX_MN_SMEM_HEAVY: launch_one<TILE_MIX_MN_SMEM_HEAVY>(reps, d); break;
    case TILE_MIX_MN_COMMITS: launch_one<TILE_MIX_MN_COMMITS>(reps, d); break;
    default: launch_one<TILE_MIX>(reps, d); break;
  }
}

int main() {
  const char* names[N_CASES] = {
      "m128 n128 SS", "m128 n128 TS (A in tensor memory)", "m128 n128 TS + 3 warps of tcgen05.ld", "m128 n64 TS",
      "m128 n16 SS", "m128 n16 TS", "m128 n16 TS, two accumulators alternating", "m64 n128 SS", "m64 n16 SS",
      "one decode tile: 13 x n128 + 8 x n16 TS + 8 x n16 SS",
      "one decode tile, P.V operand MN-major as in the kernel",
      "one decode tile (MN-major) + 15 warps of light shared-memory traffic",
      "one decode tile (MN-major) + 15 warps of heavy shared-memory traffic",
      "one decode tile (MN-major) with the kernel's 6 commits per tile"};
  long long* d;
  if (cudaMalloc(&d, 64) != cudaSuccess) { printf("no CUDA device\n"); return 2; }
  int bad = 0;
  for (int c = 0; c < N_CASES; ++c) {
    const int reps = 20, per_rep = c >= TILE_MIX ? 4 * 29 : 48;
    cudaMemset(d, 0, 64);
    launch(c, reps, d);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[3] = {0, 0, 0};
    cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess || h[0] < 0) {
      printf("%-56s: %s\n", names[c], e != cudaSuccess ? cudaGetErrorString(e) : "timeout");
      bad = 1;
      if (e != cudaSuccess) break;
      continue;
    }
    if (c == TILE_MIX_MN_SMEM_LIGHT || c == TILE_MIX_MN_SMEM_HEAVY)
      // a 16-byte access per lane is 4 wavefronts per warp instruction; the traffic warps' totals over the measured time
      printf("%-56s: %8.1f cycles per tile until complete, %8.1f cycles of the issuing thread, %.2f load/store wavefronts per cycle\n",
             names[c], h[0] / (double)reps / 4, h[1] / (double)reps / 4, 4.0 * h[2] / (double)h[0]);
    else if (c >= TILE_MIX)
      printf("%-56s: %8.1f cycles per tile until complete, %8.1f cycles of the issuing thread\n", names[c],
             h[0] / (double)reps / 4, h[1] / (double)reps / 4);
    else
      printf("%-56s: %6.1f cycles/mma until complete, %6.1f cycles/mma of the issuing thread\n", names[c],
             h[0] / (double)reps / per_rep, h[1] / (double)reps / per_rep);
  }
  cudaFree(d);
  return bad;
}
