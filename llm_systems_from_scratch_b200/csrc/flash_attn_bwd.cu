// Causal FlashAttention backward for sm_100a on the packed (batch*seq, 3*H*dh) QKV layout.
// Gradient of the reference's attention call (llm-core/llm_core/model.py:381-385) without ever
// materialising the (S, S) probabilities: they are recomputed tile by tile from Q, K and the saved
// log-sum-exp.  Three kernels, each value of dQ, dK and dV is written exactly once (no atomics, so
// results are bitwise reproducible):
//
//   flash_delta_kernel   delta[b,h,s] = sum_d dO * O
//   flash_dkdv_kernel    CTA = 128 keys of one (b,h); walks 64-query steps i >= diagonal:
//                          S^T = K Q_i^T, dP^T = V dO_i^T        (TMEM, double buffered)
//                          P^T = exp2(S^T*c - lse), dS^T = P^T*(dP^T - delta)*scale -> swizzled smem
//                          dV += P^T dO_i,  dK += dS^T Q_i        (TMEM accumulators)
//   flash_dq_kernel      CTA = 128 queries; walks 128-key steps j <= diagonal:
//                          S = Q K_j^T, dP = dO V_j^T ; dS -> tensor memory ; dQ += dS K_j
//
// Roles per CTA: warp 0 TMA producer, warp 1 tcgen05.mma issuer, warps 2-5 one tile row per thread.
#include "ptx.cuh"

namespace b200 {

int make_tmap_bf16_2d(CUtensorMap* tm, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                      uint32_t box_rows);

struct FlashBwdParams {
  const float* lse;     // (batch, heads, seq)
  const float* delta;   // (batch, heads, seq)
  __nv_bfloat16* dqkv;  // (rows, 3d)
  int batch, seq, heads, d;
  float scale, scale_log2;
  uint32_t* status;
  // Optional: dQ and dK are rotated back (transpose of the forward rotary embedding) before they are
  // stored, so the caller receives gradients with respect to the un-rotated projections.
  // (2, rope_ctx, dh/2) fp32 table; null = off.
  const float* rope_cs;
  int rope_ctx;
  // Optional timeline of one CTA (clock64 stamps per role, step and event) for tuning; null = off.
  long long* trace;
  int trace_cta;
};

// CTA log (trace_cta == BWD_CTA_LOG): every CTA records its SM, start / end time and step count
constexpr int BWD_CTA_LOG = 100000;
__device__ __forceinline__ uint32_t smid() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
  return r;
}
#define BWD_CTA_LOG_END(kernel_id, t_start, steps)                                             \
  do {                                                                                         \
    if (p.trace != nullptr && p.trace_cta == BWD_CTA_LOG && threadIdx.x == 0) {                \
      long long* rec = p.trace + ((kernel_id) * 4096 + blockIdx.x) * 4;                        \
      rec[0] = smid(); rec[1] = (long long)(t_start); rec[2] = (long long)globaltimer_ns(); rec[3] = (steps); \
    }                                                                                          \
  } while (0)

// stamp[(role * 64 + step) * 8 + slot] = SM clock, written by one lane of the traced CTA
#define BWD_TRACE(role, step, slot)                                                          \
  do {                                                                                       \
    if (p.trace != nullptr && (int)blockIdx.x == p.trace_cta && lane == 0 && (step) < 64)    \
      p.trace[((role) * 64 + (step)) * 8 + (slot)] = clock64();                              \
  } while (0)

// Inverse interleaved-pair rotation of 32 consecutive head columns starting at column e of the head.
template <int DH>
__device__ __forceinline__ void unrotate32(const FlashBwdParams& p, int pos, int e, uint32_t (&a)[32]) {
  const float* cs = p.rope_cs + (size_t)pos * (DH / 2) + e / 2;
  const float* sn = cs + (size_t)p.rope_ctx * (DH / 2);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 c4 = *reinterpret_cast<const float4*>(cs + q * 4);
    const float4 s4 = *reinterpret_cast<const float4*>(sn + q * 4);
    const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float x0 = __uint_as_float(a[q * 8 + 2 * t]), x1 = __uint_as_float(a[q * 8 + 2 * t + 1]);
      a[q * 8 + 2 * t] = __float_as_uint(cc[t] * x0 + ss[t] * x1);
      a[q * 8 + 2 * t + 1] = __float_as_uint(cc[t] * x1 - ss[t] * x0);
    }
  }
}

// delta = rowsum(dO * O) per (row, head).  dh/8 lanes cover one (row, head) with 16-byte loads, so a warp
// handles 32/(dh/8) of them at once, and every thread keeps two items in flight.
template <int DH>
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                   float* __restrict__ delta, long long items, int seq, int heads) {
  constexpr int LPI = DH / 8;                       // lanes per item
  const int lane = threadIdx.x & 31;
  const int li = lane % LPI;
  const long long group = (blockIdx.x * (long long)blockDim.x + threadIdx.x) / LPI;   // item index, first pass
  const long long n_groups = (long long)gridDim.x * blockDim.x / LPI;
  for (long long w0 = group; w0 < items; w0 += 2 * n_groups) {
    const long long w1 = w0 + n_groups;
    const bool has1 = w1 < items;                   // uniform across the LPI lanes of an item
    const uint4 a0 = *reinterpret_cast<const uint4*>(o + w0 * DH + li * 8);
    const uint4 b0 = *reinterpret_cast<const uint4*>(dout + w0 * DH + li * 8);
    uint4 a1 = make_uint4(0, 0, 0, 0), b1 = a1;
    if (has1) {
      a1 = *reinterpret_cast<const uint4*>(o + w1 * DH + li * 8);
      b1 = *reinterpret_cast<const uint4*>(dout + w1 * DH + li * 8);
    }
    float s0 = 0.f, s1 = 0.f;
    const uint32_t aa0[4] = {a0.x, a0.y, a0.z, a0.w}, bb0[4] = {b0.x, b0.y, b0.z, b0.w};
    const uint32_t aa1[4] = {a1.x, a1.y, a1.z, a1.w}, bb1[4] = {b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x = unpack_bf16x2(aa0[i]), y = unpack_bf16x2(bb0[i]);
      s0 += x.x * y.x + x.y * y.y;
      x = unpack_bf16x2(aa1[i]); y = unpack_bf16x2(bb1[i]);
      s1 += x.x * y.x + x.y * y.y;
    }
    // the loop bound depends on the item index, which differs between the item groups of a warp, so the
    // reduction uses a mask of the lanes that belong to this item only
    const unsigned mask = (LPI == 32) ? 0xffffffffu : (((1u << LPI) - 1u) << (lane - li));
#pragma unroll
    for (int off = LPI / 2; off > 0; off >>= 1) {
      s0 += __shfl_xor_sync(mask, s0, off);
      s1 += __shfl_xor_sync(mask, s1, off);
    }
    if (li == 0) {
      const long long row0 = w0 / heads;
      delta[((row0 / seq) * heads + (w0 % heads)) * seq + row0 % seq] = s0;
      if (has1) {
        const long long row1 = w1 / heads;
        delta[((row1 / seq) * heads + (w1 % heads)) * seq + row1 % seq] = s1;
      }
    }
  }
}

// The element-wise stage of both kernels is spread over BWD_CG warpgroups: warpgroup g handles
// columns [g*BWD_COLS, (g+1)*BWD_COLS) of every 64-column step, so 8 warps (2 per scheduler) hide each
// other's TMEM-load, exp2 and shared-memory latencies instead of one warp per scheduler.
constexpr int BWD_RING = 4;   // TMA ring depth of the dK/dV kernel's per-step Q / dO tiles
constexpr int DKDV_VEC_STEPS = 32;   // steps whose lse / delta are staged in shared memory at a time
constexpr int BWD_CG = 2;
constexpr int BWD_COLS = 64 / BWD_CG;                 // 32 columns per thread and step
constexpr int BWD_COMPUTE_THREADS = 128 * BWD_CG;     // 256
constexpr int BWD_THREADS = 64 + BWD_COMPUTE_THREADS; // + TMA warp + MMA warp

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ------------------------------------------------------------------------------ dK / dV
// P^T and dS^T never touch shared memory: the compute warps write them as packed bf16 over the S^T / dP^T
// columns they have just read (tcgen05.st) and the dV / dK MMAs take their A operand from tensor memory.
// The shared memory that frees holds a five-stage Q / dO ring.
template <int DH>
struct DkDvSmem {
  static constexpr int PANELS = DH / 64;
  static constexpr int KV_TILE = 128 * DH * 2;   // K_j or V_j (128 keys)
  static constexpr int Q_TILE = 64 * DH * 2;     // Q_i or dO_i (64 queries)
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + KV_TILE;
  static constexpr int OFF_Q = OFF_V + KV_TILE;                // BWD_RING stages
  static constexpr int OFF_DO = OFF_Q + BWD_RING * Q_TILE;     // BWD_RING stages
  static constexpr int OFF_VEC = OFF_DO + BWD_RING * Q_TILE;   // lse and delta of DKDV_VEC_STEPS steps (floats)
  static constexpr int OFF_BAR = OFF_VEC + 2 * DKDV_VEC_STEPS * 64 * 4;
  static constexpr int NUM_BARS = 1 + 2 * BWD_RING + 5;
  static constexpr int TOTAL = OFF_BAR + NUM_BARS * 8 + 16 + 1024;
};

template <int DH>
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_dkdv_kernel(const __grid_constant__ CUtensorMap tm_kv,   // box 64 x 128 over qkv
                  const __grid_constant__ CUtensorMap tm_q,    // box 64 x 64 over qkv
                  const __grid_constant__ CUtensorMap tm_do,   // box 64 x 64 over dO
                  const FlashBwdParams p) {
  using L = DkDvSmem<DH>;
  const uint64_t t_cta_start = globaltimer_ns();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = bars;
  uint64_t* qd_full = bars + 1;                    // [BWD_RING]
  uint64_t* qd_empty = qd_full + BWD_RING;         // [BWD_RING]
  uint64_t* s_full = qd_empty + BWD_RING;          // [2]  S^T_t and dP^T_t are in tensor memory
  uint64_t* p_full = s_full + 2;                   // [2]  P^T_t and dS^T_t are in tensor memory
  uint64_t* all_done = p_full + 2;                 // every MMA of the CTA has completed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
  volatile uint32_t* abort_word = tmem_holder + 1;
  float* lse_s = reinterpret_cast<float*>(smem + L::OFF_VEC);   // [DKDV_VEC_STEPS * 64]
  float* delta_s = lse_s + DKDV_VEC_STEPS * 64;                 // [DKDV_VEC_STEPS * 64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Longest-first order over the whole grid (small j = most query steps), so the tail of the launch is made of
  // short CTAs; the (b, h) index varies fastest.
  const int bh = blockIdx.x % (p.batch * p.heads);
  const int jblk = blockIdx.x / (p.batch * p.heads);
  const int b = bh / p.heads, h = bh % p.heads;
  const int row_base = b * p.seq;
  const int k0 = jblk * 128;
  const int n_q64 = (p.seq + 63) / 64;
  const int i0 = 2 * jblk;
  const int n_steps = n_q64 - i0;   // >= 1 because k0 < seq

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < BWD_RING; ++i) {
      mbar_init(&qd_full[i], 1);
      mbar_init(&qd_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], BWD_COMPUTE_THREADS);
    }
    mbar_init(all_done, 1);
    *abort_word = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_kv);
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tm_st = tmem_base;         // S^T: 2 x 64 columns
  const uint32_t tm_dpt = tmem_base + 128;  // dP^T: 2 x 64 columns
  const uint32_t tm_dv = tmem_base + 256;   // DH columns
  const uint32_t tm_dk = tmem_base + 384;   // DH columns

  const int col_q = h * DH, col_k = p.d + h * DH, col_v = 2 * p.d + h * DH;

  if (warp == 0) {
    if (elect_one()) {   // elect.sync keeps the issuing code warp-uniform (descriptors in uniform registers)
      const int lane = 0;   // the tracing macro stamps from the issuing thread
      (void)lane;
      mbar_expect_tx(kv_full, 2 * L::KV_TILE);
#pragma unroll
      for (int pn = 0; pn < L::PANELS; ++pn) {
        tma_load_2d(smem + L::OFF_K + pn * 16384, &tm_kv, kv_full, col_k + pn * 64, row_base + k0);
        tma_load_2d(smem + L::OFF_V + pn * 16384, &tm_kv, kv_full, col_v + pn * 64, row_base + k0);
      }
      for (int t = 0; t < n_steps; ++t) {
        const int st = t % BWD_RING;
        const uint32_t ph = (t / BWD_RING) & 1;
        const int qrow = row_base + (i0 + t) * 64;
        if (!mbar_wait(&qd_empty[st], ph ^ 1, abort_word)) { *abort_word = ERR_WAIT_EMPTY; break; }
        mbar_expect_tx(&qd_full[st], 2 * L::Q_TILE);
#pragma unroll
        for (int pn = 0; pn < L::PANELS; ++pn) {
          tma_load_2d(smem + L::OFF_Q + st * L::Q_TILE + pn * 8192, &tm_q, &qd_full[st], col_q + pn * 64, qrow);
          tma_load_2d(smem + L::OFF_DO + st * L::Q_TILE + pn * 8192, &tm_do, &qd_full[st], h * DH + pn * 64, qrow);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {   // elect.sync keeps the issuing code warp-uniform (descriptors in uniform registers)
      const int lane = 0;   // the tracing macro stamps from the issuing thread
      (void)lane;
      constexpr uint32_t idesc_12 = make_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_34 = make_idesc_bf16(128, DH, false, true);
      const uint32_t k_addr = smem_u32(smem + L::OFF_K), v_addr = smem_u32(smem + L::OFF_V);
      auto issue12 = [&](int t) {
        const int st = t & 1, rs = t % BWD_RING;
        const uint32_t q_addr = smem_u32(smem + L::OFF_Q + rs * L::Q_TILE);
        const uint32_t do_addr = smem_u32(smem + L::OFF_DO + rs * L::Q_TILE);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t offa = (k / 4) * 16384 + (k % 4) * 32;   // 128-row panels
          const uint32_t offb = (k / 4) * 8192 + (k % 4) * 32;    // 64-row panels
          umma_f16_ss(tm_st + st * 64, make_smem_desc(k_addr + offa, 16, 1024), make_smem_desc(q_addr + offb, 16, 1024),
                      idesc_12, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t offa = (k / 4) * 16384 + (k % 4) * 32;
          const uint32_t offb = (k / 4) * 8192 + (k % 4) * 32;
          umma_f16_ss(tm_dpt + st * 64, make_smem_desc(v_addr + offa, 16, 1024),
                      make_smem_desc(do_addr + offb, 16, 1024), idesc_12, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
      };
      bool ok = mbar_wait(kv_full, 0, abort_word) && mbar_wait(&qd_full[0], 0, abort_word);
      if (ok) { tc_fence_after(); issue12(0); }
      for (int t = 0; t < n_steps && ok; ++t) {
        const int st = t & 1;
        if (t + 1 < n_steps) {
          // Buffer (t+1)&1 is free: its last readers, the compute warps of step t-1, arrived on p_full before the
          // dV / dK MMAs of step t-1 were issued, and those MMAs precede this issue in the tensor pipe.
          ok = mbar_wait(&qd_full[(t + 1) % BWD_RING], ((t + 1) / BWD_RING) & 1, abort_word);
          if (!ok) break;
          tc_fence_after();
          BWD_TRACE(1, t, 0);
          issue12(t + 1);
          BWD_TRACE(1, t, 1);
        }
        ok = mbar_wait(&p_full[st], (t >> 1) & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
        BWD_TRACE(1, t, 2);
        const int rs = t % BWD_RING;
        const uint32_t q_addr = smem_u32(smem + L::OFF_Q + rs * L::Q_TILE);
        const uint32_t do_addr = smem_u32(smem + L::OFF_DO + rs * L::Q_TILE);
        // K = 64 queries.  A: column group g of the compute warps left queries [32g, 32g+32) as 16 packed columns
        // at column 32g of the S^T / dP^T buffer.  B operands are MN-major: dh contiguous, 16 queries = 2048 B per
        // step, dh panels 8192 B apart.
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t a_off = st * 64 + (k >> 1) * BWD_COLS + (k & 1) * 8;
          umma_f16_ts(tm_dv, tm_st + a_off, make_smem_desc(do_addr + k * 2048, 8192, 1024), idesc_34,
                      (t > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t a_off = st * 64 + (k >> 1) * BWD_COLS + (k & 1) * 8;
          umma_f16_ts(tm_dk, tm_dpt + a_off, make_smem_desc(q_addr + k * 2048, 8192, 1024), idesc_34,
                      (t > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&qd_empty[rs]);
        if (t == n_steps - 1) umma_commit(all_done);
        BWD_TRACE(1, t, 3);
      }
      if (!ok) *abort_word = ERR_WAIT_FULL;
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;      // key row inside the tile
    const int tid = (warp - 2) * 32 + lane; // 0..511 among the compute threads
    const int cg = (warp - 2) >> 2;         // column group of this warpgroup
    const int key_idx = k0 + r;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const float* lse_g = p.lse + ((size_t)b * p.heads + h) * p.seq;
    const float* delta_g = p.delta + ((size_t)b * p.heads + h) * p.seq;
    bool ok = true;
    // lse (in log2 units; +inf zeroes the probabilities of padded queries) and delta * scale of the next
    // DKDV_VEC_STEPS steps are staged in shared memory by all compute threads together, so no step waits on a
    // global load; the two barriers around a refill are reached by every compute thread, also after a failed wait.
    for (int t = 0; t < n_steps; ++t) {
      const int st = t & 1;
      const uint32_t ph = (t >> 1) & 1;
      const int qb = (i0 + t) * 64;
      BWD_TRACE(warp, t, 0);
      if (t % DKDV_VEC_STEPS == 0) {
        if (t > 0) named_barrier_sync(1, BWD_COMPUTE_THREADS);   // everyone is done with the previous chunk
        const int q_first = (i0 + t) * 64;
        constexpr int PER = DKDV_VEC_STEPS * 64 / BWD_COMPUTE_THREADS;
        float lv[PER], dv[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) {   // all loads in flight before the first store
          const int qi = q_first + tid + i * BWD_COMPUTE_THREADS;
          lv[i] = (qi < p.seq) ? lse_g[qi] : INFINITY;
          dv[i] = (qi < p.seq) ? delta_g[qi] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          lse_s[tid + i * BWD_COMPUTE_THREADS] = lv[i] * 1.4426950408889634f;
          delta_s[tid + i * BWD_COMPUTE_THREADS] = dv[i] * p.scale;
        }
        named_barrier_sync(1, BWD_COMPUTE_THREADS);
      }
      if (!ok) continue;
      BWD_TRACE(warp, t, 1);
      if (!mbar_wait(&s_full[st], ph, abort_word)) { ok = false; continue; }
      tc_fence_after();
      BWD_TRACE(warp, t, 2);
      uint32_t sreg[BWD_COLS], dreg[BWD_COLS];
      tmem_ld_32x32(tm_st + lane_addr + st * 64 + cg * BWD_COLS, sreg);
      tmem_ld_32x32(tm_dpt + lane_addr + st * 64 + cg * BWD_COLS, dreg);
      tmem_ld_wait();
      BWD_TRACE(warp, t, 3);
      const bool need_mask = (qb < k0 + 128);   // tile touches the diagonal
      const float* lse_v = lse_s + (t % DKDV_VEC_STEPS) * 64 + cg * BWD_COLS;   // lse * log2(e); +inf marks a padded query
      const float* dlt_v = delta_s + (t % DKDV_VEC_STEPS) * 64 + cg * BWD_COLS;  // delta * scale
      // Eight columns at a time: two 16-byte broadcast reads each of lse and delta, eight independent
      // exp2 / multiply chains, four packed results each of P^T and dS^T (bf16 packing on the integer pipe).
      uint32_t pk[BWD_COLS / 2], dk[BWD_COLS / 2];
#pragma unroll
      for (int c0 = 0; c0 < BWD_COLS; c0 += 8) {
        float lr[8], dr[8], pe[8], ds[8];
        *reinterpret_cast<float4*>(lr) = *reinterpret_cast<const float4*>(lse_v + c0);
        *reinterpret_cast<float4*>(lr + 4) = *reinterpret_cast<const float4*>(lse_v + c0 + 4);
        *reinterpret_cast<float4*>(dr) = *reinterpret_cast<const float4*>(dlt_v + c0);
        *reinterpret_cast<float4*>(dr + 4) = *reinterpret_cast<const float4*>(dlt_v + c0 + 4);
#pragma unroll
        for (int e = 0; e < 8; ++e) pe[e] = fast_exp2(__uint_as_float(sreg[c0 + e]) * p.scale_log2 - lr[e]);
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 8; ++e) pe[e] = (qb + cg * BWD_COLS + c0 + e < key_idx) ? 0.f : pe[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ds[e] = pe[e] * (__uint_as_float(dreg[c0 + e]) * p.scale - dr[e]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          pk[c0 / 2 + e] = pack_bf16x2_alu(pe[2 * e], pe[2 * e + 1]);
          dk[c0 / 2 + e] = pack_bf16x2_alu(ds[2 * e], ds[2 * e + 1]);
        }
      }
      BWD_TRACE(warp, t, 4);
      tmem_st_32x16(tm_st + lane_addr + st * 64 + cg * BWD_COLS, pk);
      tmem_st_32x16(tm_dpt + lane_addr + st * 64 + cg * BWD_COLS, dk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[st]);
      BWD_TRACE(warp, t, 5);
    }
    if (ok) ok = mbar_wait(all_done, 0, abort_word);
    if (ok) {
      tc_fence_after();
      const bool valid = key_idx < p.seq;
      __nv_bfloat16* dk_row = p.dqkv + (size_t)(row_base + key_idx) * 3 * p.d + col_k;
      __nv_bfloat16* dv_row = p.dqkv + (size_t)(row_base + key_idx) * 3 * p.d + col_v;
#pragma unroll 1
      for (int c = cg; c < DH / 32; c += BWD_CG) {   // each warpgroup stores its own 32-column slices
        uint32_t a[32], g[32];
        tmem_ld_32x32(tm_dk + lane_addr + c * 32, a);
        tmem_ld_32x32(tm_dv + lane_addr + c * 32, g);
        tmem_ld_wait();
        if (valid && p.rope_cs != nullptr) unrotate32<DH>(p, key_idx, c * 32, a);
        if (valid) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            *reinterpret_cast<uint4*>(dk_row + c * 32 + q * 8) =
                make_uint4(pack_bf16x2(__uint_as_float(a[q * 8 + 0]), __uint_as_float(a[q * 8 + 1])),
                           pack_bf16x2(__uint_as_float(a[q * 8 + 2]), __uint_as_float(a[q * 8 + 3])),
                           pack_bf16x2(__uint_as_float(a[q * 8 + 4]), __uint_as_float(a[q * 8 + 5])),
                           pack_bf16x2(__uint_as_float(a[q * 8 + 6]), __uint_as_float(a[q * 8 + 7])));
            *reinterpret_cast<uint4*>(dv_row + c * 32 + q * 8) =
                make_uint4(pack_bf16x2(__uint_as_float(g[q * 8 + 0]), __uint_as_float(g[q * 8 + 1])),
                           pack_bf16x2(__uint_as_float(g[q * 8 + 2]), __uint_as_float(g[q * 8 + 3])),
                           pack_bf16x2(__uint_as_float(g[q * 8 + 4]), __uint_as_float(g[q * 8 + 5])),
                           pack_bf16x2(__uint_as_float(g[q * 8 + 6]), __uint_as_float(g[q * 8 + 7])));
          }
        }
      }
    } else if (lane == 0) {
      *abort_word = ERR_WAIT_TMEM_FULL;
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0u, (*abort_word) | (blockIdx.x << 8));
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  BWD_CTA_LOG_END(0, t_cta_start, n_steps);
}

// ----------------------------------------------------------------------------------- dQ
// CTA = 128 queries of one (b, h); walks 128-key steps j up to the diagonal:
//   S = Q K_j^T and dP = dO V_j^T  (128 x 128 fp32 each, single buffered in tensor memory)
//   dS = P * (dP - delta) * scale   written by the compute warps as packed bf16 into tensor memory
//   dQ += dS K_j                    A operand straight from tensor memory, B = K_j MN-major
// dS never touches shared memory, which therefore holds Q, dO, three K stages and two V stages (a K tile
// stays live until its dQ MMA, a V tile only until its dP MMA).  Tensor pipe order per step:
// [S, dP of step t+1] [dQ of step t], so the element-wise work on step t+1 overlaps the dQ MMAs of step t.
constexpr int DQ_KSTAGES = 3;
constexpr int DQ_VSTAGES = 2;

template <int DH>
struct DqSmem {
  static constexpr int PANELS = DH / 64;
  static constexpr int TILE = 128 * DH * 2;   // Q_i, dO_i, K_j or V_j (128 rows)
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = OFF_Q + TILE;
  static constexpr int OFF_K = OFF_DO + TILE;                 // DQ_KSTAGES stages
  static constexpr int OFF_V = OFF_K + DQ_KSTAGES * TILE;     // DQ_VSTAGES stages
  static constexpr int OFF_BAR = OFF_V + DQ_VSTAGES * TILE;
  static constexpr int NUM_BARS = 1 + 2 * DQ_KSTAGES + 2 * DQ_VSTAGES + 2 + 2 + 1;
  static constexpr int TOTAL = OFF_BAR + NUM_BARS * 8 + 16 + 1024;
};

template <int DH>
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_dq_kernel(const __grid_constant__ CUtensorMap tm_qkv,   // box 64 x 128 over qkv
                const __grid_constant__ CUtensorMap tm_do,    // box 64 x 128 over dO
                const FlashBwdParams p) {
  using L = DqSmem<DH>;
  const uint64_t t_cta_start = globaltimer_ns();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* qd_full = bars;
  uint64_t* k_full = bars + 1;                     // [DQ_KSTAGES]
  uint64_t* k_empty = k_full + DQ_KSTAGES;         // [DQ_KSTAGES]  dQ MMAs of the step have completed
  uint64_t* v_full = k_empty + DQ_KSTAGES;         // [DQ_VSTAGES]
  uint64_t* v_empty = v_full + DQ_VSTAGES;         // [DQ_VSTAGES]  dP MMAs of the step have completed
  uint64_t* s_full = v_empty + DQ_VSTAGES;         // S_t and dP_t are in tensor memory
  uint64_t* s_empty = s_full + 1;                  // every compute thread has S_t and dP_t in registers
  uint64_t* p_full = s_empty + 1;                  // [2] dS_t is in tensor memory
  uint64_t* dq_done = p_full + 2;                  // all MMAs of the CTA have completed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
  volatile uint32_t* abort_word = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qblk = (p.seq + 127) / 128;
  // Longest-first order over the whole grid (latest query tile = most key steps), so the tail of the launch is
  // made of short CTAs; the (b, h) index varies fastest.
  const int bh = blockIdx.x % (p.batch * p.heads);
  const int iblk = n_qblk - 1 - blockIdx.x / (p.batch * p.heads);
  const int b = bh / p.heads, h = bh % p.heads;
  const int row_base = b * p.seq;
  const int q0 = iblk * 128;
  const int n_steps = iblk + 1;   // 128-key steps up to and including the diagonal tile

  if (threadIdx.x == 0) {
    mbar_init(qd_full, 1);
    for (int i = 0; i < DQ_KSTAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < DQ_VSTAGES; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, BWD_COMPUTE_THREADS);
    mbar_init(&p_full[0], BWD_COMPUTE_THREADS);
    mbar_init(&p_full[1], BWD_COMPUTE_THREADS);
    mbar_init(dq_done, 1);
    *abort_word = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_qkv);
    prefetch_tensormap(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tm_s = tmem_base;           // 128 columns
  const uint32_t tm_dp = tmem_base + 128;    // 128 columns
  const uint32_t tm_ds = tmem_base + 256;    // 2 x 64 columns of packed bf16 pairs
  const uint32_t tm_dq = tmem_base + 384;    // DH columns

  const int col_q = h * DH, col_k = p.d + h * DH, col_v = 2 * p.d + h * DH;

  if (warp == 0) {
    if (elect_one()) {   // elect.sync keeps the issuing code warp-uniform (descriptors in uniform registers)
      const int lane = 0;   // the tracing macro stamps from the issuing thread
      (void)lane;
      mbar_expect_tx(qd_full, 2 * L::TILE);
#pragma unroll
      for (int pn = 0; pn < L::PANELS; ++pn) {
        tma_load_2d(smem + L::OFF_Q + pn * 16384, &tm_qkv, qd_full, col_q + pn * 64, row_base + q0);
        tma_load_2d(smem + L::OFF_DO + pn * 16384, &tm_do, qd_full, h * DH + pn * 64, row_base + q0);
      }
      for (int t = 0; t < n_steps; ++t) {
        const int ks = t % DQ_KSTAGES, vs = t % DQ_VSTAGES;
        const int krow = row_base + t * 128;
        if (!mbar_wait(&k_empty[ks], ((t / DQ_KSTAGES) & 1) ^ 1, abort_word)) { *abort_word = ERR_WAIT_EMPTY; break; }
        BWD_TRACE(0, t, 0);
        mbar_expect_tx(&k_full[ks], L::TILE);
#pragma unroll
        for (int pn = 0; pn < L::PANELS; ++pn)
          tma_load_2d(smem + L::OFF_K + ks * L::TILE + pn * 16384, &tm_qkv, &k_full[ks], col_k + pn * 64, krow);
        if (!mbar_wait(&v_empty[vs], ((t / DQ_VSTAGES) & 1) ^ 1, abort_word)) { *abort_word = ERR_WAIT_EMPTY; break; }
        BWD_TRACE(0, t, 1);
        mbar_expect_tx(&v_full[vs], L::TILE);
#pragma unroll
        for (int pn = 0; pn < L::PANELS; ++pn)
          tma_load_2d(smem + L::OFF_V + vs * L::TILE + pn * 16384, &tm_qkv, &v_full[vs], col_v + pn * 64, krow);
      }
    } else if (lane == 1 && p.trace != nullptr && (int)blockIdx.x == p.trace_cta) {
      // tuning aid: arrival time of every K and V tile
      for (int t = 0; t < n_steps && t < 64; ++t) {
        if (!mbar_wait(&k_full[t % DQ_KSTAGES], (t / DQ_KSTAGES) & 1, abort_word)) break;
        p.trace[(0 * 64 + t) * 8 + 2] = clock64();
        if (!mbar_wait(&v_full[t % DQ_VSTAGES], (t / DQ_VSTAGES) & 1, abort_word)) break;
        p.trace[(0 * 64 + t) * 8 + 3] = clock64();
      }
    }
  } else if (warp == 1) {
    // elect.sync keeps the issuing code warp-uniform for the compiler (descriptors in uniform registers)
    if (elect_one()) {
      const int lane = 0;   // the tracing macro stamps from the issuing thread
      (void)lane;
      constexpr uint32_t idesc_12 = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_3 = make_idesc_bf16(128, DH, false, true);
      const uint64_t q_desc = make_smem_desc(smem_u32(smem + L::OFF_Q), 16, 1024);
      const uint64_t do_desc = make_smem_desc(smem_u32(smem + L::OFF_DO), 16, 1024);
      auto issue12 = [&](int t) {
        const uint64_t k_desc = make_smem_desc(smem_u32(smem + L::OFF_K + (t % DQ_KSTAGES) * L::TILE), 16, 1024);
        const uint64_t v_desc = make_smem_desc(smem_u32(smem + L::OFF_V + (t % DQ_VSTAGES) * L::TILE), 16, 1024);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t off = ((k / 4) * 16384 + (k % 4) * 32) >> 4;
          umma_f16_ss(tm_s, q_desc + off, k_desc + off, idesc_12, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t off = ((k / 4) * 16384 + (k % 4) * 32) >> 4;
          umma_f16_ss(tm_dp, do_desc + off, v_desc + off, idesc_12, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        umma_commit(&v_empty[t % DQ_VSTAGES]);
      };
      bool ok = mbar_wait(qd_full, 0, abort_word) && mbar_wait(&k_full[0], 0, abort_word) &&
                mbar_wait(&v_full[0], 0, abort_word);
      if (ok) { tc_fence_after(); issue12(0); }
      for (int t = 0; t < n_steps && ok; ++t) {
        if (t + 1 < n_steps) {
          ok = mbar_wait(&k_full[(t + 1) % DQ_KSTAGES], ((t + 1) / DQ_KSTAGES) & 1, abort_word) &&
               mbar_wait(&v_full[(t + 1) % DQ_VSTAGES], ((t + 1) / DQ_VSTAGES) & 1, abort_word) &&
               mbar_wait(s_empty, t & 1, abort_word);
          if (!ok) break;
          tc_fence_after();
          BWD_TRACE(1, t, 0);
          issue12(t + 1);
          BWD_TRACE(1, t, 1);
        }
        ok = mbar_wait(&p_full[t & 1], (t >> 1) & 1, abort_word);
        if (!ok) break;
        tc_fence_after();
        BWD_TRACE(1, t, 2);
        // K = 128 keys; A = dS_t from tensor memory (16 keys = 8 packed columns); B = K_t MN-major: 16 keys are
        // 2048 B apart inside a 64-column panel, the dh panels 16384 B apart.
        const uint64_t kmn_desc = make_smem_desc(smem_u32(smem + L::OFF_K + (t % DQ_KSTAGES) * L::TILE), 16384, 1024);
        const uint32_t a_tmem = tm_ds + (t & 1) * 64;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ts(tm_dq, a_tmem + k * 8, kmn_desc + ((k * 2048) >> 4), idesc_3, (t > 0 || k > 0) ? 1u : 0u);
        umma_commit(&k_empty[t % DQ_KSTAGES]);
        if (t == n_steps - 1) umma_commit(dq_done);
        BWD_TRACE(1, t, 3);
      }
      if (!ok) *abort_word = ERR_WAIT_FULL;
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int q_idx = q0 + r;
    const int cg = (warp - 2) >> 2;          // this thread's 64 of the step's 128 keys
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const bool valid = q_idx < p.seq;
    const size_t vec = ((size_t)b * p.heads + h) * p.seq + q_idx;
    const float lse2 = valid ? p.lse[vec] * 1.4426950408889634f : INFINITY;   // +inf: padded rows get P = 0
    const float dlt_scaled = valid ? p.delta[vec] * p.scale : 0.f;
    bool ok = true;
    for (int t = 0; t < n_steps; ++t) {
      const int trole = warp;
      BWD_TRACE(trole, t, 0);
      if (!mbar_wait(s_full, t & 1, abort_word)) { ok = false; break; }
      tc_fence_after();
      BWD_TRACE(trole, t, 1);
      uint32_t sreg[2][32], dreg[2][32];
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        tmem_ld_32x32(tm_s + lane_addr + cg * 64 + hf * 32, sreg[hf]);
        tmem_ld_32x32(tm_dp + lane_addr + cg * 64 + hf * 32, dreg[hf]);
      }
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_empty);      // S and dP may be overwritten by the MMAs of step t+1
      BWD_TRACE(trole, t, 2);
      const int kb = t * 128 + cg * 64;
      uint32_t packed[32];
      if (t == n_steps - 1) {   // diagonal tile: causal mask
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float ds[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              float pe = fast_exp2(__uint_as_float(sreg[hf][c + e]) * p.scale_log2 - lse2);
              pe = (kb + hf * 32 + c + e > q_idx) ? 0.f : pe;
              ds[e] = pe * (__uint_as_float(dreg[hf][c + e]) * p.scale - dlt_scaled);
            }
            packed[hf * 16 + c / 2] = pack_bf16x2_alu(ds[0], ds[1]);
          }
      } else {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float ds[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float pe = fast_exp2(__uint_as_float(sreg[hf][c + e]) * p.scale_log2 - lse2);
              ds[e] = pe * (__uint_as_float(dreg[hf][c + e]) * p.scale - dlt_scaled);
            }
            packed[hf * 16 + c / 2] = pack_bf16x2_alu(ds[0], ds[1]);
          }
      }
      BWD_TRACE(trole, t, 3);
      // Buffer t&1 was last read by the dQ MMAs of step t-2, which precede the S MMAs of step t in the tensor pipe.
      tmem_st_32x32(tm_ds + lane_addr + (t & 1) * 64 + cg * 32, packed);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[t & 1]);
      BWD_TRACE(trole, t, 4);
    }
    if (ok) ok = mbar_wait(dq_done, 0, abort_word);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dq_row = p.dqkv + (size_t)(row_base + q_idx) * 3 * p.d + col_q;
#pragma unroll 1
      for (int c = cg; c < DH / 32; c += BWD_CG) {
        uint32_t a[32];
        tmem_ld_32x32(tm_dq + lane_addr + c * 32, a);
        tmem_ld_wait();
        if (valid && p.rope_cs != nullptr) unrotate32<DH>(p, q_idx, c * 32, a);
        if (valid) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(dq_row + c * 32 + q * 8) =
                make_uint4(pack_bf16x2(__uint_as_float(a[q * 8 + 0]), __uint_as_float(a[q * 8 + 1])),
                           pack_bf16x2(__uint_as_float(a[q * 8 + 2]), __uint_as_float(a[q * 8 + 3])),
                           pack_bf16x2(__uint_as_float(a[q * 8 + 4]), __uint_as_float(a[q * 8 + 5])),
                           pack_bf16x2(__uint_as_float(a[q * 8 + 6]), __uint_as_float(a[q * 8 + 7])));
        }
      }
    } else if (lane == 0) {
      *abort_word = ERR_WAIT_TMEM_FULL;
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0u, (*abort_word) | (blockIdx.x << 8));
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  BWD_CTA_LOG_END(1, t_cta_start, n_steps);
}

template <int DH>
static int launch_flash_bwd(const void* qkv, const void* dout, const FlashBwdParams& p, cudaStream_t stream) {
  const uint64_t rows = (uint64_t)p.batch * p.seq;
  CUtensorMap tm_qkv128, tm_qkv64, tm_do128, tm_do64;
  if (make_tmap_bf16_2d(&tm_qkv128, qkv, rows, 3ull * p.d, 3ull * p.d, 64, 128)) return -20;
  if (make_tmap_bf16_2d(&tm_qkv64, qkv, rows, 3ull * p.d, 3ull * p.d, 64, 64)) return -20;
  if (make_tmap_bf16_2d(&tm_do128, dout, rows, (uint64_t)p.d, (uint64_t)p.d, 64, 128)) return -20;
  if (make_tmap_bf16_2d(&tm_do64, dout, rows, (uint64_t)p.d, (uint64_t)p.d, 64, 64)) return -20;
  auto k1 = flash_dkdv_kernel<DH>;
  auto k2 = flash_dq_kernel<DH>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, DkDvSmem<DH>::TOTAL) != cudaSuccess) return -3;
    if (cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<DH>::TOTAL) != cudaSuccess) return -3;
    configured = true;
  }
  const int n_kblk = (p.seq + 127) / 128;
  // tracing (tuning aid): CTA c >= 0 selects the dQ kernel's CTA c, c < 0 the dK/dV kernel's CTA -c-1
  FlashBwdParams p1 = p, p2 = p;
  if (p.trace_cta == BWD_CTA_LOG) { }
  else if (p.trace_cta >= 0) p1.trace = nullptr;
  else { p2.trace = nullptr; p1.trace_cta = -p.trace_cta - 1; }
  k1<<<p.batch * p.heads * n_kblk, BWD_THREADS, DkDvSmem<DH>::TOTAL, stream>>>(tm_qkv128, tm_qkv64, tm_do64, p1);
  k2<<<p.batch * p.heads * n_kblk, BWD_THREADS, DqSmem<DH>::TOTAL, stream>>>(tm_qkv128, tm_do128, p2);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace b200

using namespace b200;

static long long* g_bwd_trace = nullptr;
static int g_bwd_trace_cta = 0;

// Tuning aid: record the timeline of CTA `cta` of the next backward launches into `buf`
// (device memory, 10 roles x 64 steps x 8 stamps of 8 bytes); null switches it off.
extern "C" void b200_flash_bwd_set_trace(long long* buf, int cta) {
  g_bwd_trace = buf;
  g_bwd_trace_cta = cta;
}

// qkv (rows, 3d), o / dout (rows, d) bf16; lse (batch, heads, seq) from the forward; delta: scratch of the
// same shape (fp32); dqkv (rows, 3d) bf16 receives dQ | dK | dV.  dh must be 64 or 128.
static int flash_bwd_impl(const void* qkv, const void* o, const void* dout, const float* lse, float* delta, void* dqkv,
                          int batch, int seq, int heads, int dh, float scale, const float* rope_cs, int rope_ctx,
                          uint32_t* status, cudaStream_t stream) {
  if (dh != 64 && dh != 128) return -10;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(dout) |
       reinterpret_cast<uintptr_t>(dqkv)) & 15)
    return -10;
  if (batch <= 0 || seq <= 0) return 0;
  const long long items = (long long)batch * seq * heads;   // (row, head) pairs; o and dout are (rows, heads*dh)
  {
    const int lpi = dh / 8;
    long long blocks = (items * lpi + 2 * 256 - 1) / (2 * 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    if (dh == 128)
      flash_delta_kernel<128><<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout,
                                                                    delta, items, seq, heads);
    else
      flash_delta_kernel<64><<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout,
                                                                   delta, items, seq, heads);
  }
  FlashBwdParams p;
  p.lse = lse; p.delta = delta; p.dqkv = (__nv_bfloat16*)dqkv;
  p.batch = batch; p.seq = seq; p.heads = heads; p.d = heads * dh;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.rope_cs = rope_cs; p.rope_ctx = rope_ctx;
  p.trace = g_bwd_trace; p.trace_cta = g_bwd_trace_cta;
  return dh == 64 ? launch_flash_bwd<64>(qkv, dout, p, stream) : launch_flash_bwd<128>(qkv, dout, p, stream);
}

extern "C" int b200_flash_bwd(const void* qkv, const void* o, const void* dout, const float* lse, float* delta,
                              void* dqkv, int batch, int seq, int heads, int dh, float scale, uint32_t* status,
                              cudaStream_t stream) {
  return flash_bwd_impl(qkv, o, dout, lse, delta, dqkv, batch, seq, heads, dh, scale, nullptr, 0, status, stream);
}

// As b200_flash_bwd, but `qkv` holds rotated Q and K (rotary embedding already applied) and the returned dQ / dK
// are gradients with respect to the projections before the rotation.  cos_sin: (2, ctx, dh/2) fp32, seq <= ctx.
extern "C" int b200_flash_bwd_rope(const void* qkv, const void* o, const void* dout, const float* lse, float* delta,
                                   void* dqkv, int batch, int seq, int heads, int dh, float scale,
                                   const float* cos_sin, int ctx, uint32_t* status, cudaStream_t stream) {
  if (cos_sin == nullptr || seq > ctx || (reinterpret_cast<uintptr_t>(cos_sin) & 15)) return -12;
  return flash_bwd_impl(qkv, o, dout, lse, delta, dqkv, batch, seq, heads, dh, scale, cos_sin, ctx, status, stream);
}
