// Persistent, warp-specialised bf16 GEMM for sm_100a:  D[m,n] = sum_k A(m,k) * B(n,k)
//
//   warp 0      TMA producer   (cp.async.bulk.tensor -> 128B-swizzled smem ring, mbarrier tx-count)
//   warp 1      MMA issuer     (one thread: tcgen05.mma kind::f16, 128 x BN x 16, accumulators in TMEM)
//   warps 2-5   epilogue       (tcgen05.ld -> registers -> fused epilogue -> global)
//
// Two TMEM accumulators (2 x BN columns) let the epilogue of tile i overlap the main loop of
// tile i+1.  Either operand may be K-major (rows of K contiguous) or MN-major (stored as
// (K, MN) with MN contiguous), which covers forward (x W^T), dgrad (dy W) and wgrad (dy^T x)
// without any transposed copies.  This replaces the library GEMM behind the reference's
// `Linear.forward` (llm-core/llm_core/model.py:31-32) and its autograd-generated backward.
//
// Edge tiles: TMA zero-fills out-of-range rows / K tail; stores are predicated.
#include "gemm_common.cuh"

#include <stdio.h>

namespace b200 {

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int DATA_BYTES = STAGES * (A_BYTES + B_BYTES);
  // barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then tmem holder + abort word
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int TOTAL = DATA_BYTES + BAR_BYTES + 1024;  // + alignment slack
};

template <int BN, bool A_MN, bool B_MN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmParams p) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * S::A_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::DATA_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_word = tmem_holder + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 128);
    }
    *abort_word = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    if (!B_MN && p.b_early) {
      // first work unit of this CTA: the B tiles of its first STAGES k-blocks are requested now; the producer below
      // adds the A tiles to the same barriers after the wait for the previous kernel
      const int sp = p.splits > 1 ? p.splits : 1;
      const int nkb = (p.K + BK - 1) / BK;
      const int unit = blockIdx.x;
      if (unit < p.num_m_tiles * p.num_n_tiles * sp) {
        const int tile = unit / sp, split = unit - tile * sp;
        const int kb_lo = split * nkb / sp, kb_hi = (split + 1) * nkb / sp;
        int m_blk, n_blk;
        tile_coords(tile, p, m_blk, n_blk);
        for (int i = 0; i < STAGES && kb_lo + i < kb_hi; ++i) {
          mbar_expect_tx(&full_bar[i], S::A_BYTES + S::B_BYTES);
          tma_load_2d(smem_b + i * S::B_BYTES, &tmB, &full_bar[i], (kb_lo + i) * BK, n_blk * BN);
        }
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  // Everything above touches only shared and tensor memory, so as a programmatic dependent it overlaps the tail of
  // the kernel before this one; from here on global memory is read and written.
  pdl_sync();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;
  // work unit = (tile, K slice); consecutive units are the slices of one tile, so they run at the same time on
  // neighbouring CTAs
  const int splits = p.splits > 1 ? p.splits : 1;
  const int num_units = num_tiles * splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {   // elect.sync keeps the issuing code warp-uniform (descriptors in uniform registers)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int early = (!B_MN && p.b_early) ? STAGES : 0;   // k-blocks whose B tile and byte count were posted in the prologue
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        const int tile = unit / splits, split = unit - tile * splits;
        const int kb_lo = split * num_kb / splits, kb_hi = (split + 1) * num_kb / splits;
        int m_blk, n_blk;
        tile_coords(tile, p, m_blk, n_blk);
        const int m0 = m_blk * BM, n0 = n_blk * BN;
        if (unit != (int)blockIdx.x) early = 0;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          const bool posted = kb - kb_lo < early;
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word)) {
            report(p, abort_word, ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          if (!posted) mbar_expect_tx(&full_bar[stage], S::A_BYTES + S::B_BYTES);
          uint8_t* a_dst = smem_a + stage * S::A_BYTES;
          uint8_t* b_dst = smem_b + stage * S::B_BYTES;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full_bar[stage], m0 + j * 64, k0);
          } else {
            tma_load_2d(a_dst, &tmA, &full_bar[stage], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, &full_bar[stage], n0 + j * 64, k0);
          } else if (!posted) {
            tma_load_2d(b_dst, &tmB, &full_bar[stage], k0, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------- MMA issuer
    if (elect_one()) {   // elect.sync keeps the issuing code warp-uniform (descriptors in uniform registers)
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++local) {
        const int split = unit % splits;
        const int kb_lo = split * num_kb / splits, kb_hi = (split + 1) * num_kb / splits;
        const int acc = local & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase[acc] ^ 1, abort_word)) {
          report(p, abort_word, ERR_WAIT_TMEM_EMPTY);
          ok = false;
          break;
        }
        acc_phase[acc] ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_word)) {
            report(p, abort_word, ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem_a + stage * S::A_BYTES);
          const uint32_t b_base = smem_u32(smem_b + stage * S::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = A_MN ? make_smem_desc(a_base + k * (UMMA_K * 128), 8192, 1024)
                                         : make_smem_desc(a_base + k * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = B_MN ? make_smem_desc(b_base + k * (UMMA_K * 128), 8192, 1024)
                                         : make_smem_desc(b_base + k * (UMMA_K * 2), 16, 1024);
            umma_f16_ss(d_tmem, a_desc, b_desc, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // smem stage is free once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tmem_full[acc]);  // accumulator complete
      }
    }
  } else {
    // --------------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are visible to this warp
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++local) {
      const int tile = unit / splits;
      int m_blk, n_blk;
      tile_coords(tile, p, m_blk, n_blk);
      const int acc = local & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc], abort_word)) {
        if (lane == 0) report(p, abort_word, ERR_WAIT_TMEM_FULL);
        ok = false;
        break;
      }
      acc_phase[acc] ^= 1;
      tc_fence_after();
      const int row_in_tile = quarter * 32 + lane;
      const int row = m_blk * BM + row_in_tile;
      const int n0 = n_blk * BN;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      if (splits == 1) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (n0 + c * 32 >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          epilogue_store(p, row, n0 + c * 32, r);
        }
        tc_fence_before();
        mbar_arrive(&tmem_empty[acc]);
        continue;
      }
      // Split-K.  The partial tile goes to the workspace as (BN / 4) x BM float4: piece j of every row is contiguous
      // over the rows, so a warp's store (and the matching load of the reduction) is one 512-byte run.
      float4* part = reinterpret_cast<float4*>(p.ws) + (size_t)unit * (BM * BN / 4);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        if (n0 + c * 32 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          __stcg(part + (size_t)(c * 8 + j) * BM + row_in_tile,
                 make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                             __uint_as_float(r[4 * j + 3])));
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);        // the accumulator is free: the next unit's MMAs may start
      // Rows [32 * quarter, 32 * quarter + 32) of the tile are written by this warp in every one of the `splits`
      // CTAs, so they have a counter of their own: the warp that arrives last adds the partials of its 32 rows.
      // No CTA-wide barrier is involved.
      __threadfence();                      // this lane's partial is visible before the warp is counted
      __syncwarp();
      uint32_t seen = 0;
      if (lane == 0) {
        __threadfence();
        seen = atomicAdd(&p.tile_counters[tile * 4 + quarter], 1u);
        if (seen == (uint32_t)splits - 1) p.tile_counters[tile * 4 + quarter] = 0;    // clean for the next launch
      }
      seen = __shfl_sync(0xffffffffu, seen, 0);
      if (seen == (uint32_t)splits - 1) {
        __threadfence();
        const float4* first = reinterpret_cast<const float4*>(p.ws) + (size_t)tile * splits * (BM * BN / 4);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (n0 + c * 32 >= p.N) break;
          float sum[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[j] = 0.f;
          // added in slice order whichever CTA does the adding; four slices' loads are in flight at a time
          for (int sp0 = 0; sp0 < splits; sp0 += 4) {
            float4 v[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (sp0 + u < splits) {
                const float4* src = first + (size_t)(sp0 + u) * (BM * BN / 4) + (size_t)(c * 8) * BM + row_in_tile;
#pragma unroll
                for (int j = 0; j < 8; ++j) v[u][j] = __ldcg(src + (size_t)j * BM);
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (sp0 + u < splits) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  sum[4 * j] += v[u][j].x; sum[4 * j + 1] += v[u][j].y;
                  sum[4 * j + 2] += v[u][j].z; sum[4 * j + 3] += v[u][j].w;
                }
              }
            }
          }
          uint32_t r[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(sum[j]);
          epilogue_store(p, row, n0 + c * 32, r);
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    // Give copies that may still be in flight time to land before shared memory is released.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// bf16 matrix with `rows` rows of `cols` contiguous elements, row stride `ld` elements;
// box = (box_cols, box_rows), 128-byte swizzle.
int make_tmap_bf16_2d(CUtensorMap* tm, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                      uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// Output matrix (bf16 or fp32) for TMA stores: box = (box_cols, box_rows) with box_cols * element size == 128 bytes,
// 128-byte swizzle.  Boxes that reach past the matrix are clipped by the hardware, so edge tiles need no predication.
int make_tmap_out_2d(CUtensorMap* tm, bool f32, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                     uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  const uint64_t esz = f32 ? 4 : 2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esz};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

static int g_num_sms = 0;
static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_num_sms <= 0) {
      cudaGetLastError();
      return 148;      // no device visible (planning helpers called on a CPU-only machine): a B200's count
    }
  }
  return g_num_sms;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams p, int max_ctas, cudaStream_t stream) {
  constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  using S = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN, STAGES>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) != cudaSuccess) return -3;
    configured = true;
  }
  p.num_m_tiles = (p.M + BM - 1) / BM;
  p.num_n_tiles = (p.N + BN - 1) / BN;
  p.group_m = 16;
  const int units = p.num_m_tiles * p.num_n_tiles * (p.splits > 1 ? p.splits : 1);
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (units < grid) grid = units;
  if (launch_dep(kern, grid, 192, S::TOTAL, stream, tmA, tmB, p) != cudaSuccess) return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace b200

using namespace b200;

// D (M x N) = A * B^T-style contraction over K.
//   a_mn == 0: A is (M, K) row-major with row stride lda;  a_mn == 1: A is stored (K, M) with row stride lda.
//   b_mn == 0: B is (N, K) row-major with row stride ldb;  b_mn == 1: B is stored (K, N) with row stride ldb.
//   epi: 0 bf16 out, 1 fp32 out, 2 bf16 out + bf16 residual R, 3 fp32 accumulate into C.
// Requirements (checked): base pointers 16-byte aligned; lda, ldb multiples of 8 elements.
// Returns 0 on success, negative on argument / launch errors.  `status` (device uint32, may be null)
// receives a non-zero code if a bounded wait inside the kernel gave up.
static int gemm_bf16_impl(const void* A, const void* B, void* C, const void* R, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, long long ldr, int a_mn, int b_mn, int epi, int bn_hint,
                          int max_ctas, int splits, float* ws, uint32_t* tile_counters, uint32_t* status,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7))
    return -10;
  const int b_early = (epi & EPI_B_STABLE) ? 1 : 0;
  epi &= ~EPI_B_STABLE;
  if (epi == EPI_BF16_RES && R == nullptr) return -11;
  if (epi == EPI_SWIGLU_BWD &&
      (R == nullptr || (N & 7) || (ldr & 7) || (ldc & 7) || ((reinterpret_cast<uintptr_t>(R) | reinterpret_cast<uintptr_t>(C)) & 15)))
    return -11;
  int bn = bn_hint;
  const bool small_ok = !a_mn && !b_mn;   // narrow tiles exist for the K-major (decode) layout only
  if (small_ok && (bn == 32 || bn == 64)) {
    // explicit request
  } else if (small_ok && bn != 128 && bn != 256 && M <= 2 * BM) {
    // One or two rows of tiles (decode): every CTA streams its B rows once and all of A's rows over the whole of K,
    // so a CTA's time goes with BM + bn and the launch's with the number of waves.  Narrow tiles spread the weights
    // over more SMs but re-read A more often; a tile count just above the SM count costs a whole second wave.
    const int sms = num_sms();
    const int mt = (M + BM - 1) / BM;
    long long best = -1;
    const int cand[4] = {32, 64, 128, 256};
    for (int ci = 0; ci < 4; ++ci) {
      const long long tiles = (long long)mt * ((N + cand[ci] - 1) / cand[ci]);
      const long long cost = ((tiles + sms - 1) / sms) * (BM + cand[ci]);
      if (best < 0 || cost < best) {
        best = cost;
        bn = cand[ci];
      }
    }
  } else if (bn != 128 && bn != 256) {
    const long long mt = (M + BM - 1) / BM;
    const long long sms = num_sms();
    const long long w256 = (mt * ((N + 255) / 256) + sms - 1) / sms * 256 * 10;
    const long long w128 = (mt * ((N + 127) / 128) + sms - 1) / sms * 128 * 11;
    bn = (w128 < w256) ? 128 : 256;
  }
  CUtensorMap tmA, tmB;
  int rc;
  if (a_mn)
    rc = make_tmap_bf16_2d(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 64);
  else
    rc = make_tmap_bf16_2d(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BM);
  if (rc) return -20 + rc;
  if (b_mn)
    rc = make_tmap_bf16_2d(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 64);
  else
    rc = make_tmap_bf16_2d(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, bn);
  if (rc) return -30 + rc;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.R = R; p.ldr = ldr; p.epi = epi; p.status = status;
  p.num_m_tiles = p.num_n_tiles = p.group_m = 0;
  p.gather.dst = nullptr; p.gather.done = nullptr; p.gather.shard_vec = 0; p.gather.world = 0; p.gather.rank = 0;
  p.reduce.n = 0;
  p.tma_store = 0;
  p.wait_counter = nullptr; p.wait_value = 0; p.wait_limit_ns = 0;
  p.rope_cs = nullptr; p.rope_seq = p.rope_d = p.rope_dh = p.rope_ctx = 0;
  p.swiglu_f = 0; p.H = nullptr; p.ldh = 0;
  p.splits = splits > 1 ? splits : 1; p.ws = ws; p.tile_counters = tile_counters;
  p.b_early = b_early;

#define DISPATCH(BN_)                                                                    \
  if (a_mn && b_mn) return launch_gemm<BN_, true, true>(tmA, tmB, p, max_ctas, stream);   \
  if (a_mn) return launch_gemm<BN_, true, false>(tmA, tmB, p, max_ctas, stream);          \
  if (b_mn) return launch_gemm<BN_, false, true>(tmA, tmB, p, max_ctas, stream);          \
  return launch_gemm<BN_, false, false>(tmA, tmB, p, max_ctas, stream);
  if (bn == 256) { DISPATCH(256) }
  if (bn == 64) return launch_gemm<64, false, false>(tmA, tmB, p, max_ctas, stream);
  if (bn == 32) return launch_gemm<32, false, false>(tmA, tmB, p, max_ctas, stream);
  DISPATCH(128)
#undef DISPATCH
}

extern "C" int b200_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                              long long lda, long long ldb, long long ldc, long long ldr, int a_mn, int b_mn,
                              int epi, int bn_hint, int max_ctas, uint32_t* status, cudaStream_t stream) {
  return gemm_bf16_impl(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn, b_mn, epi, bn_hint, max_ctas, 1, nullptr,
                        nullptr, status, stream);
}

// Tile width and number of K slices for a GEMM with at most two rows of tiles (decode: M <= 256, weights streamed
// once).  A plain launch would use N / BN CTAs, each reading all of A and a BN-row slab of B over the whole of K; with
// `splits` slices there are splits times as many CTAs, each reading a slice of both.  The estimate counts, per wave of
// CTAs, the 128-byte operand rows a CTA loads, a fixed cost per CTA and the partial tiles the last CTA adds up.
extern "C" void b200_gemm_splitk_plan(int M, int N, int K, int* bn_out, int* splits_out) {
  const int sms = num_sms();
  const int mt = (M + BM - 1) / BM;
  const int num_kb = (K + BK - 1) / BK;
  long long best = -1;
  *bn_out = 0;
  *splits_out = 1;
  const int cand[3] = {256, 128, 64};
  for (int ci = 0; ci < 3; ++ci) {
    const int bn = cand[ci];
    const int tiles = mt * ((N + bn - 1) / bn);
    int s = sms / tiles;
    if (s > 8) s = 8;
    if (s > num_kb / 4) s = num_kb / 4;
    if (s < 1) s = 1;
    const int units = tiles * s;
    const long long waves = (units + sms - 1) / sms;
    const long long kb_per = (num_kb + s - 1) / s;
    const long long cost = waves * (kb_per * (BM + bn) + 2048 + (s > 1 ? 2LL * s * bn : 0));
    if (best < 0 || cost < best) {
      best = cost;
      *bn_out = bn;
      *splits_out = s;
    }
  }
}

// Workspace a split-K launch needs: floats of partial tiles and tile counters (one CTA per unit, at most one wave
// by construction of the plan, so 148 units of 128 x 256 floats bound it).
extern "C" long long b200_gemm_splitk_ws_floats(void) { return (long long)num_sms() * BM * 256; }
extern "C" int b200_gemm_splitk_counters(void) { return 4 * num_sms() * 4; }

// b200_gemm_bf16 for K-major operands and M <= 256 with K split over CTAs (see b200_gemm_splitk_plan).  `ws` and
// `tile_counters` are scratch of the sizes above; the counters must be zero on entry and are zero again on exit.
// One launch at a time may use a given workspace (launches on one stream are ordered; other streams need their own).
extern "C" int b200_gemm_bf16_splitk(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                                     long long lda, long long ldb, long long ldc, long long ldr, int epi, float* ws,
                                     long long ws_floats, uint32_t* tile_counters, int n_counters, uint32_t* status,
                                     cudaStream_t stream) {
  int bn = 0, splits = 1;
  b200_gemm_splitk_plan(M, N, K, &bn, &splits);
  const long long tiles = (long long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  if (splits > 1 && (ws == nullptr || tile_counters == nullptr || (reinterpret_cast<uintptr_t>(ws) & 15) ||
                     tiles * splits * BM * bn > ws_floats || tiles * 4 > n_counters))
    return -12;
  const int base_epi = epi & ~EPI_B_STABLE;
  if (base_epi != EPI_BF16 && base_epi != EPI_F32 && base_epi != EPI_BF16_RES && base_epi != EPI_F32_ACC) return -11;
  if (splits <= 1)
    return gemm_bf16_impl(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, 0, 0, epi, 0, 0, 1, nullptr, nullptr, status, stream);
  return gemm_bf16_impl(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, 0, 0, epi, bn, 0, splits, ws, tile_counters, status,
                        stream);
}
