// Small-M bf16 GEMM for decode steps (M <= 256 rows of activations against a large weight matrix):
//     C[M, N] = X[M, K] * W[N, K]^T (+ R[M, N]),   bf16 in, fp32 accumulate, bf16 out.
//
// With so few rows the work is streaming W once from HBM, and a 128-row MMA tile of X would be mostly padding.
// So the operands are swapped: W supplies the 128-row side of tcgen05.mma (a CTA owns 128 output columns) and the
// activations are the narrow N side (M rounded up to 16).  One thread-block cluster of S CTAs shares a column
// tile and splits K between its CTAs, so that even N = 2048 puts 128 CTAs on the GPU, each with its whole K slice
// in flight at once.  The S partial tiles (fp32, TMEM -> registers -> the CTA's own shared memory, which the
// finished operand ring no longer needs) are added up through distributed shared memory in a fixed order: CTA r of
// the cluster reduces rows [128 r / S, 128 (r + 1) / S) of the tile from every peer's shared memory, adds the
// residual and writes the bf16 output.  No global workspace, no atomics, bitwise reproducible.
//
// Roles per CTA: warp 0 TMA producer, warp 1 tcgen05.mma issuer, warps 2-5 accumulator drain and the reduction.
// Every wait is bounded (see ptx.cuh); loads are plain (non-multicast) TMA loads.
#include "gemm_common.cuh"

#include <stdlib.h>

namespace b200 {

int make_tmap_bf16_2d(CUtensorMap* tm, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                      uint32_t box_rows);

constexpr int SM_THREADS = 192;
constexpr int SM_W_BYTES = 128 * BK * 2;         // 16 KB: 128 weight rows x 64 k
constexpr int SM_RING_BYTES = 196608;            // operand ring, reused for the fp32 partial tile
constexpr int SM_MAX_STAGES = 12;
constexpr int SM_SMEM = SM_RING_BYTES + (2 * SM_MAX_STAGES + 1) * 8 + 16 + 1024;

struct SmallMParams {
  int M, N, K;
  int np;            // M rounded up to a multiple of 16 (MMA N), <= 256
  int stages;        // stages of the operand ring that fit
  int split;         // CTAs per cluster = K splits (1, 2, 4 or 8)
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* R;   // residual or null
  long long ldr;
  uint32_t* status;
};

__device__ __forceinline__ uint32_t sm_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void sm_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t sm_map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 sm_ld_cluster_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}

__global__ void __launch_bounds__(SM_THREADS, 1)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const SmallMParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int x_bytes = p.np * BK * 2;
  const int stage_bytes = SM_W_BYTES + x_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SM_RING_BYTES);
  uint64_t* empty_bar = full_bar + SM_MAX_STAGES;
  uint64_t* tmem_full = empty_bar + SM_MAX_STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_full + 1);
  volatile uint32_t* abort_word = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = sm_cluster_ctarank();
  const int tile = blockIdx.x / p.split;
  const int n0 = tile * 128;
  const int num_kb = (p.K + BK - 1) / BK;
  const int kb_per = (num_kb + p.split - 1) / p.split;
  const int kb0 = min(num_kb, (int)crank * kb_per);
  const int kb1 = min(num_kb, kb0 + kb_per);
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < p.np) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    *abort_word = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word)) {
          *abort_word = ERR_WAIT_EMPTY;
          if (p.status != nullptr) atomicCAS(p.status, 0u, ERR_WAIT_EMPTY | (blockIdx.x << 8));
          break;
        }
        mbar_expect_tx(&full_bar[stage], stage_bytes);
        uint8_t* dst = smem + stage * stage_bytes;
        tma_load_2d(dst, &tmW, &full_bar[stage], kb * BK, n0);
        tma_load_2d(dst + SM_W_BYTES, &tmX, &full_bar[stage], kb * BK, 0);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(128, p.np, false, false);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, abort_word)) {
          *abort_word = ERR_WAIT_FULL;
          if (p.status != nullptr) atomicCAS(p.status, 0u, ERR_WAIT_FULL | (blockIdx.x << 8));
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t w_base = smem_u32(smem + stage * stage_bytes);
        const uint32_t x_base = w_base + SM_W_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t a_desc = make_smem_desc(w_base + k * (UMMA_K * 2), 16, 1024);
          const uint64_t b_desc = make_smem_desc(x_base + k * (UMMA_K * 2), 16, 1024);
          umma_f16_ss(tmem_base, a_desc, b_desc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      umma_commit(tmem_full);      // also arrives when this CTA's K slice is empty (nothing was issued)
    }
  }

  // ---- accumulator -> registers -> this CTA's shared memory, as a column-major fp32 tile part[col][row]
  float* part = reinterpret_cast<float*>(smem);          // the ring is free once every MMA has completed
  bool drained = true;
  if (warp >= 2) {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                  // weight row inside the tile = TMEM lane
    if (!mbar_wait(tmem_full, 0, abort_word)) {
      if (lane == 0) {
        *abort_word = ERR_WAIT_TMEM_FULL;
        if (p.status != nullptr) atomicCAS(p.status, 0u, ERR_WAIT_TMEM_FULL | (blockIdx.x << 8));
      }
      drained = false;
    }
    tc_fence_after();
    const bool has_k = kb1 > kb0;
    for (int c0 = 0; c0 < p.np; c0 += 32) {
      uint32_t r[32];
      if (drained && has_k) {
        if (p.np - c0 >= 32) {
          tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + c0, r);
        } else {                                          // np is a multiple of 16: one 16-column remainder
          uint32_t h[16];
          tmem_ld_32x16(tmem_base + (uint32_t(quarter * 32) << 16) + c0, h);
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = h[j];
#pragma unroll
          for (int j = 16; j < 32; ++j) r[j] = 0;
        }
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0;            // an empty K slice contributes zeros
      }
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c0 + j < p.np) part[(c0 + j) * 128 + row] = __uint_as_float(r[j]);
    }
  }
  tc_fence_before();
  __syncthreads();
  sm_cluster_sync();            // every CTA's partial tile is complete and visible to the cluster

  // ---- CTA `crank` reduces rows [rc * crank, rc * (crank + 1)) of the tile over all CTAs of the cluster
  if (warp >= 2 && *abort_word == 0) {
    const int rc = 128 / p.split;                          // rows per CTA: 128, 64, 32 or 16
    const int groups = rc / 8;                             // 8-row groups -> one 16-byte output store each
    const int t = threadIdx.x - 64;                        // 0..127
    const int rg = t % groups;
    const int row = (int)crank * rc + rg * 8;              // first of this thread's 8 rows inside the tile
    const int cols_per_pass = 128 / groups;
    const uint32_t part_addr = smem_u32(part);
    for (int c = t / groups; c < p.M; c += cols_per_pass) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int peer = 0; peer < p.split; ++peer) {         // fixed order: bitwise reproducible
        const uint32_t a = sm_map_to_cta(part_addr + (uint32_t)(c * 128 + row) * 4u, (uint32_t)peer);
        const float4 lo = sm_ld_cluster_f4(a), hi = sm_ld_cluster_f4(a + 16);
        acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
        acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
      }
      const int n = n0 + row;
      if (n >= p.N) continue;
      __nv_bfloat16* out = p.C + (long long)c * p.ldc + n;
      const bool full8 = n + 8 <= p.N;
      if (p.R != nullptr) {
        const __nv_bfloat16* res = p.R + (long long)c * p.ldr + n;
        if (full8 && (reinterpret_cast<uintptr_t>(res) & 15) == 0) {
          const uint4 rv = *reinterpret_cast<const uint4*>(res);
          const float2 a = unpack_bf16x2(rv.x), b = unpack_bf16x2(rv.y), c2 = unpack_bf16x2(rv.z), d = unpack_bf16x2(rv.w);
          acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
          acc[4] += c2.x; acc[5] += c2.y; acc[6] += d.x; acc[7] += d.y;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (n + j < p.N) acc[j] += __bfloat162float(res[j]);
        }
      }
      if (full8 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        *reinterpret_cast<uint4*>(out) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                    pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (n + j < p.N) out[j] = __float2bfloat16(acc[j]);
      }
    }
  }
  __syncthreads();
  if (*abort_word != 0) {
    // Give copies that may still be in flight time to land before shared memory is released.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  sm_cluster_sync();            // no CTA leaves (and frees its shared memory) while a peer may still read it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

}  // namespace b200

using namespace b200;

// K splits for N columns on `sms` SMs: the largest of 8, 4, 2, 1 that keeps the grid within about one wave and
// leaves every CTA at least two k-blocks.
static int smallm_split(int N, int K, int sms) {
  const int tiles = (N + 127) / 128;
  const int num_kb = (K + BK - 1) / BK;
  for (int s = 8; s > 1; s >>= 1)
    if (tiles * s <= sms + sms / 8 && num_kb / s >= 2) return s;
  return 1;
}

// C (M x N, bf16) = X (M x K) * W (N x K)^T (+ R), M <= 256.  lda / ldw multiples of 8 elements, pointers 16-byte
// aligned; `split` 0 = choose.  Returns 0, or a negative code for arguments this kernel does not take.
extern "C" int b200_gemm_smallm(const void* X, const void* W, void* C, const void* R, int M, int N, int K, long long ldx,
                                long long ldw, long long ldc, long long ldr, int split, uint32_t* status,
                                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 256) return -12;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (ldx & 7) || (ldw & 7)) return -10;
  if (C == nullptr) return -11;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  SmallMParams p;
  p.M = M; p.N = N; p.K = K;
  p.np = (M + 15) / 16 * 16;
  p.split = (split == 1 || split == 2 || split == 4 || split == 8) ? split : smallm_split(N, K, sms);
  const int stage_bytes = SM_W_BYTES + p.np * BK * 2;
  p.stages = SM_RING_BYTES / stage_bytes;
  if (p.stages > SM_MAX_STAGES) p.stages = SM_MAX_STAGES;
  if (p.stages < 2 || 128 * p.np * 4 > SM_RING_BYTES) return -13;
  p.C = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.R = reinterpret_cast<const __nv_bfloat16*>(R); p.ldr = ldr;
  p.status = status;
  CUtensorMap tmW, tmX;
  if (make_tmap_bf16_2d(&tmW, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 64, 128)) return -20;
  if (make_tmap_bf16_2d(&tmX, X, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, 64, (uint32_t)p.np)) return -30;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_smallm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_SMEM) != cudaSuccess) return -3;
    configured = true;
  }
  const int tiles = (N + 127) / 128;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * p.split), 1, 1);
  cfg.blockDim = dim3(SM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SM_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)p.split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm_smallm_kernel, tmW, tmX, p) != cudaSuccess) {
    cudaGetLastError();
    return -4;
  }
  return 0;
}
