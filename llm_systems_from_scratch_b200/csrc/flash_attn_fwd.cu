// Causal FlashAttention forward for sm_100a, reading Q, K and V directly out of the packed
// (batch*seq, 3*H*dh) QKV activation (no head transposes) and writing O as (batch*seq, H*dh).
// Replaces the library SDPA call of the reference (llm-core/llm_core/model.py:381-382) and its
// naive masked-softmax path (model.py:308-325).
//
// One CTA owns a 128-query tile of one (batch, head) and walks the key/value tiles up to the
// diagonal:
//   warp 0     TMA producer: Q once, then K_j / V_j into two-stage rings (128B swizzle)
//   warp 1     MMA issuer:   S_j = Q K_j^T (TMEM, double buffered)  and  O += P_j V_j (TMEM)
//   warps 2-9  softmax:      tcgen05.ld S_j -> online softmax in registers (two threads per row, 64 columns each)
//                            -> P_j as bf16 into swizzled smem; rescale O in TMEM only when the
//                            running max moved by more than 2^8 (vote per warp)
// S_{j+1} is issued before P_j V_j, so the tensor core computes the next scores while the softmax
// warps work on the current ones.
#include "ptx.cuh"

namespace b200 {

int make_tmap_bf16_2d(CUtensorMap* tm, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                      uint32_t box_rows);

__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr int FA_BQ = 128;   // queries per CTA
constexpr int FA_BK = 128;   // keys per step
constexpr int FA_THREADS = 64 + 256;   // TMA warp, MMA warp, 8 softmax warps

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

struct FlashFwdParams {
  __nv_bfloat16* o;      // (rows, d)
  float* lse;            // (batch, heads, seq)
  const int* cu_seqlens; // optional (batch+1) row offsets for packed variable-length sequences
  int batch, seq, heads, d;  // d = heads * dh; seq = max sequence length when cu_seqlens is given
  int n_qblk;
  float scale_log2;      // softmax scale * log2(e)
  uint32_t* status;
  long long* trace;      // optional timeline of CTA `trace_cta` (tuning aid); null = off
  int trace_cta;
};

// stamp[(role * 64 + step) * 8 + slot] = SM clock, written by one lane of the traced CTA
#define FWD_TRACE(role, step, slot)                                                          \
  do {                                                                                       \
    if (p.trace != nullptr && (int)blockIdx.x == p.trace_cta && lane == 0 && (step) < 64)    \
      p.trace[((role) * 64 + (step)) * 8 + (slot)] = clock64();                              \
  } while (0)

template <int DH>
struct FlashFwdSmem {
  static constexpr int PANELS = DH / 64;              // 64-column (128-byte) panels per tile
  static constexpr int TILE_BYTES = 128 * DH * 2;     // Q, K or V tile
  static constexpr int P_BYTES = 128 * FA_BK * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + TILE_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * TILE_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * TILE_BYTES;
  static constexpr int OFF_XCH = OFF_P + P_BYTES;        // row-max / row-sum exchange: 3 x 2 x 128 floats
  static constexpr int OFF_BAR = OFF_XCH + 3 * 2 * 128 * 4;   // two step buffers + one for the final sums
  static constexpr int NUM_BARS = 1 + 4 + 4 + 2 + 2 + 2;  // q, k full/empty, v full/empty, s full/empty, p full/empty
  static constexpr int TOTAL = OFF_BAR + NUM_BARS * 8 + 16 + 1024;
};

template <int DH>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const FlashFwdParams p) {
  using L = FlashFwdSmem<DH>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_empty = bars + 11;  // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* p_empty = bars + 14;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
  volatile uint32_t* abort_word = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Work assignment: longest-first over the whole grid (latest query tile = most key steps), so the tail of the
  // launch is made of short CTAs; the (b, h) index varies fastest.
  const int bh = blockIdx.x % (p.batch * p.heads);
  const int qblk = p.n_qblk - 1 - blockIdx.x / (p.batch * p.heads);
  const int b = bh / p.heads, h = bh % p.heads;
  int row_base, seq_len;
  if (p.cu_seqlens != nullptr) {
    row_base = p.cu_seqlens[b];
    seq_len = p.cu_seqlens[b + 1] - row_base;
  } else {
    row_base = b * p.seq;
    seq_len = p.seq;
  }
  const int q0 = qblk * FA_BQ;
  const bool active = q0 < seq_len;           // CTA-uniform
  const int n_kv = active ? (min(q0 + FA_BQ, seq_len) + FA_BK - 1) / FA_BK : 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 256);
    }
    mbar_init(p_full, 256);
    mbar_init(p_empty, 1);
    *abort_word = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_qkv);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base;            // 2 x 128 columns
  const uint32_t tmem_o = tmem_base + 256;      // DH columns

  const int col_q = h * DH, col_k = p.d + h * DH, col_v = 2 * p.d + h * DH;

  if (warp == 0) {
    if (active && elect_one()) {   // elect.sync keeps the issuing code warp-uniform (descriptors in uniform registers)
      const int lane = 0;   // the tracing macro stamps from the issuing thread
      (void)lane;
      mbar_expect_tx(q_full, L::TILE_BYTES);
#pragma unroll
      for (int pn = 0; pn < L::PANELS; ++pn)
        tma_load_2d(smem + L::OFF_Q + pn * 16384, &tm_qkv, q_full, col_q + pn * 64, row_base + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int krow = row_base + j * FA_BK;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_word)) { *abort_word = ERR_WAIT_EMPTY; break; }
        mbar_expect_tx(&k_full[st], L::TILE_BYTES);
#pragma unroll
        for (int pn = 0; pn < L::PANELS; ++pn)
          tma_load_2d(smem + L::OFF_K + st * L::TILE_BYTES + pn * 16384, &tm_qkv, &k_full[st], col_k + pn * 64, krow);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_word)) { *abort_word = ERR_WAIT_EMPTY; break; }
        mbar_expect_tx(&v_full[st], L::TILE_BYTES);
#pragma unroll
        for (int pn = 0; pn < L::PANELS; ++pn)
          tma_load_2d(smem + L::OFF_V + st * L::TILE_BYTES + pn * 16384, &tm_qkv, &v_full[st], col_v + pn * 64, krow);
      }
    }
  } else if (warp == 1) {
    if (active && elect_one()) {   // elect.sync keeps the issuing code warp-uniform (descriptors in uniform registers)
      const int lane = 0;   // the tracing macro stamps from the issuing thread
      (void)lane;
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, FA_BK, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, DH, false, true);
      const uint32_t q_addr = smem_u32(smem + L::OFF_Q);
      const uint32_t p_addr = smem_u32(smem + L::OFF_P);
      bool ok = mbar_wait(q_full, 0, abort_word);
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t k_addr = smem_u32(smem + L::OFF_K + st * L::TILE_BYTES);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t off = (k / 4) * 16384 + (k % 4) * 32;
          umma_f16_ss(tmem_s + st * 128, make_smem_desc(q_addr + off, 16, 1024), make_smem_desc(k_addr + off, 16, 1024),
                      idesc_qk, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
      };
      if (ok) {
        ok = mbar_wait(&k_full[0], 0, abort_word);
        if (ok) { tc_fence_after(); issue_s(0); }
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < n_kv) {
          const int st1 = (j + 1) & 1;
          const uint32_t ph1 = ((j + 1) >> 1) & 1;
          ok = mbar_wait(&k_full[st1], ph1, abort_word) && mbar_wait(&s_empty[st1], ph1 ^ 1, abort_word);
          if (!ok) break;
          tc_fence_after();
          FWD_TRACE(1, j, 0);
          issue_s(j + 1);
          FWD_TRACE(1, j, 1);
        }
        ok = mbar_wait(p_full, j & 1, abort_word) && mbar_wait(&v_full[st], ph, abort_word);
        if (!ok) break;
        tc_fence_after();
        FWD_TRACE(1, j, 2);
        const uint32_t v_addr = smem_u32(smem + L::OFF_V + st * L::TILE_BYTES);
#pragma unroll
        for (int k = 0; k < FA_BK / 16; ++k) {
          // A = P (K-major over keys): panel k/4, 32-byte step inside the panel.
          // B = V (MN-major: dh contiguous, keys are rows of 128 B): 16 keys = 2048 B; dh panels 16384 B apart.
          const uint64_t a_desc = make_smem_desc(p_addr + (k / 4) * 16384 + (k % 4) * 32, 16, 1024);
          const uint64_t b_desc = make_smem_desc(v_addr + k * 2048, 16384, 1024);
          umma_f16_ss(tmem_o, a_desc, b_desc, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(p_empty);
        umma_commit(&v_empty[st]);
        FWD_TRACE(1, j, 3);
      }
      if (!ok) *abort_word = ERR_WAIT_FULL;
    }
  } else if (active) {
    // ----------------------------------------------------------------- softmax warps
    // Two warpgroups share every row: warpgroup g owns score columns [64g, 64g+64) and output
    // columns [g*DH/2, (g+1)*DH/2).  They exchange the row maximum once per step through shared
    // memory; the row sum is kept as two partial sums and combined at the end.
    const int quarter = warp & 3;
    const int wg = (warp - 2) >> 2;             // 0 or 1
    const int r = quarter * 32 + lane;          // row inside the query tile
    const int q_idx = q0 + r;                   // position inside the sequence
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    float m_run = -INFINITY;                    // running max in scaled log2 units (identical in both halves)
    float l_run = 0.f;                          // this half's part of the row sum
    uint8_t* p_row = smem + L::OFF_P + wg * 16384 + r * 128;
    float* xch = reinterpret_cast<float*>(smem + L::OFF_XCH);   // [2 steps][2 halves][128 rows]
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      float mx = -INFINITY;
      uint32_t s[2][32];
      const int trole = warp;
      FWD_TRACE(trole, j, 0);
      if (ok && !mbar_wait(&s_full[st], ph, abort_word)) ok = false;
      if (ok) {
        tc_fence_after();
        FWD_TRACE(trole, j, 1);
#pragma unroll
        for (int c = 0; c < 2; ++c) tmem_ld_32x32(tmem_s + lane_addr + st * 128 + wg * 64 + c * 32, s[c]);
        tmem_ld_wait();
        FWD_TRACE(trole, j, 2);
        tc_fence_before();
        mbar_arrive(&s_empty[st]);
        const bool diag = (j == n_kv - 1);
        const int k0 = j * FA_BK + wg * 64;
        // row maximum over the raw scores (the softmax scale is positive, so it is applied afterwards)
        if (diag) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (k0 + c * 32 + i > q_idx) s[c][i] = 0xff800000u;   // -inf
              mx = fmaxf(mx, __uint_as_float(s[c][i]));
            }
        } else {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(s[c][i]));
        }
        mx *= p.scale_log2;
        xch[(st * 2 + wg) * 128 + r] = mx;
      }
      FWD_TRACE(trole, j, 3);
      named_barrier_sync(1, 256);               // reached by all 256 softmax threads every step
      if (!ok) continue;
      FWD_TRACE(trole, j, 4);
      mx = fmaxf(mx, xch[(st * 2 + (wg ^ 1)) * 128 + r]);
      // Lazy rescale: keep the old reference max unless it moved by more than 8 (a factor 256).
      float m_new = m_run;
      if (mx > m_run + 8.f) m_new = mx;
      const bool need = m_new != m_run;
      const float alpha = (m_run == -INFINITY) ? 0.f : fa_exp2(m_run - m_new);
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float e = fa_exp2(fmaf(__uint_as_float(s[c][i]), p.scale_log2, -m_new));   // exp2(-inf) = 0 for masked keys
          sum += e;
          s[c][i] = __float_as_uint(e);
        }
      l_run = l_run * (need ? alpha : 1.f) + sum;
      m_run = m_new;
      // P_{j-1} V_{j-1} must have finished before P is overwritten or O is rescaled.
      FWD_TRACE(trole, j, 5);
      if (j > 0) {
        if (!mbar_wait(p_empty, (j - 1) & 1, abort_word)) { ok = false; continue; }
        tc_fence_after();
        FWD_TRACE(trole, j, 6);
        if (__any_sync(0xffffffffu, need)) {
          const float f = need ? alpha : 1.f;
#pragma unroll 1
          for (int c = 0; c < DH / 32; ++c) {   // this warpgroup's half of the output columns
            uint32_t o[16];
            const uint32_t col = wg * (DH / 2) + c * 16;
            tmem_ld_32x16(tmem_o + lane_addr + col, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st_32x16(tmem_o + lane_addr + col, o);
          }
          tmem_st_wait();
        }
      }
      // P row -> swizzled smem (panel = warpgroup): 16-byte chunk c16 lands at chunk (c16 ^ (r & 7)).
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c16 = c * 4 + q;
          uint4 v = make_uint4(pack_bf16x2_alu(__uint_as_float(s[c][q * 8 + 0]), __uint_as_float(s[c][q * 8 + 1])),
                               pack_bf16x2_alu(__uint_as_float(s[c][q * 8 + 2]), __uint_as_float(s[c][q * 8 + 3])),
                               pack_bf16x2_alu(__uint_as_float(s[c][q * 8 + 4]), __uint_as_float(s[c][q * 8 + 5])),
                               pack_bf16x2_alu(__uint_as_float(s[c][q * 8 + 6]), __uint_as_float(s[c][q * 8 + 7])));
          *reinterpret_cast<uint4*>(p_row + ((c16 ^ (r & 7)) << 4)) = v;
        }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
      FWD_TRACE(trole, j, 7);
    }
    // ------------------------------------------------------------------- epilogue
    xch[512 + wg * 128 + r] = l_run;            // combine the two partial row sums (own buffer: no reuse hazard)
    named_barrier_sync(1, 256);
    const float l_tot = l_run + xch[512 + (wg ^ 1) * 128 + r];
    if (ok && n_kv > 0) ok = mbar_wait(p_empty, (n_kv - 1) & 1, abort_word);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l_tot;
      const bool valid = q_idx < seq_len;
      __nv_bfloat16* orow = p.o + (size_t)(row_base + q_idx) * p.d + h * DH + wg * (DH / 2);
#pragma unroll 1
      for (int c = 0; c < DH / 64; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + lane_addr + wg * (DH / 2) + c * 32, o);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v = make_uint4(pack_bf16x2(__uint_as_float(o[q * 8 + 0]) * inv_l, __uint_as_float(o[q * 8 + 1]) * inv_l),
                                 pack_bf16x2(__uint_as_float(o[q * 8 + 2]) * inv_l, __uint_as_float(o[q * 8 + 3]) * inv_l),
                                 pack_bf16x2(__uint_as_float(o[q * 8 + 4]) * inv_l, __uint_as_float(o[q * 8 + 5]) * inv_l),
                                 pack_bf16x2(__uint_as_float(o[q * 8 + 6]) * inv_l, __uint_as_float(o[q * 8 + 7]) * inv_l));
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = v;
          }
        }
      }
      if (wg == 0 && valid && p.lse != nullptr)
        p.lse[((size_t)b * p.heads + h) * p.seq + q_idx] = (m_run + log2f(l_tot)) * 0.6931471805599453f;
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
}

template <int DH>
static int launch_flash_fwd(const CUtensorMap& tm, const FlashFwdParams& p, cudaStream_t stream) {
  using L = FlashFwdSmem<DH>;
  auto kern = flash_fwd_kernel<DH>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess) return -3;
    configured = true;
  }
  const int grid = p.batch * p.heads * p.n_qblk;
  kern<<<grid, FA_THREADS, L::TOTAL, stream>>>(tm, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace b200

using namespace b200;

static long long* g_fwd_trace = nullptr;
static int g_fwd_trace_cta = 0;

// Tuning aid: record the timeline of CTA `cta` of the next forward launches into `buf`
// (device memory, 10 roles x 64 steps x 8 stamps of 8 bytes); null switches it off.
extern "C" void b200_flash_fwd_set_trace(long long* buf, int cta) {
  g_fwd_trace = buf;
  g_fwd_trace_cta = cta;
}

// qkv: (rows, 3*heads*dh) bf16 row-major, rows = batch*seq (or cu_seqlens[batch] when packed).
// o: (rows, heads*dh) bf16.  lse: (batch, heads, seq) fp32 or null.  dh must be 64 or 128.
extern "C" int b200_flash_fwd(const void* qkv, void* o, float* lse, int batch, int seq, int heads, int dh,
                              float scale, uint32_t* status, cudaStream_t stream) {
  if (dh != 64 && dh != 128) return -10;
  if (reinterpret_cast<uintptr_t>(qkv) & 15 || reinterpret_cast<uintptr_t>(o) & 15) return -10;
  if (batch <= 0 || seq <= 0) return 0;
  const int d = heads * dh;
  CUtensorMap tm;
  if (make_tmap_bf16_2d(&tm, qkv, (uint64_t)batch * seq, (uint64_t)3 * d, (uint64_t)3 * d, 64, 128)) return -20;
  FlashFwdParams p;
  p.o = (__nv_bfloat16*)o; p.lse = lse; p.cu_seqlens = nullptr;
  p.batch = batch; p.seq = seq; p.heads = heads; p.d = d;
  p.n_qblk = (seq + FA_BQ - 1) / FA_BQ;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.trace = g_fwd_trace; p.trace_cta = g_fwd_trace_cta;
  return dh == 64 ? launch_flash_fwd<64>(tm, p, stream) : launch_flash_fwd<128>(tm, p, stream);
}

// Packed variable-length sequences (serving prefill): cu_seqlens (batch+1) int32 on the device,
// total_rows = cu_seqlens[batch], max_seq = longest sequence.
extern "C" int b200_flash_varlen_fwd(const void* qkv, void* o, const int* cu_seqlens, int batch, int max_seq,
                                     int total_rows, int heads, int dh, float scale, uint32_t* status,
                                     cudaStream_t stream) {
  if (dh != 64 && dh != 128) return -10;
  if (reinterpret_cast<uintptr_t>(qkv) & 15 || reinterpret_cast<uintptr_t>(o) & 15) return -10;
  if (batch <= 0 || total_rows <= 0) return 0;
  const int d = heads * dh;
  CUtensorMap tm;
  if (make_tmap_bf16_2d(&tm, qkv, (uint64_t)total_rows, (uint64_t)3 * d, (uint64_t)3 * d, 64, 128)) return -20;
  FlashFwdParams p;
  p.o = (__nv_bfloat16*)o; p.lse = nullptr; p.cu_seqlens = cu_seqlens;
  p.batch = batch; p.seq = max_seq; p.heads = heads; p.d = d;
  p.n_qblk = (max_seq + FA_BQ - 1) / FA_BQ;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.trace = g_fwd_trace; p.trace_cta = g_fwd_trace_cta;
  return dh == 64 ? launch_flash_fwd<64>(tm, p, stream) : launch_flash_fwd<128>(tm, p, stream);
}
