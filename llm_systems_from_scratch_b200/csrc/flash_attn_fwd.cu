// Causal FlashAttention forward for sm_100a, reading Q, K and V directly out of the packed
// (batch*seq, 3*H*dh) QKV activation (no head transposes) and writing O as (batch*seq, H*dh).
// Replaces the library SDPA call of the reference (llm-core/llm_core/model.py:381-382) and its
// naive masked-softmax path (model.py:308-325).
//
// One CTA owns TWO 128-query tiles (A, B) of one (batch, head) and walks the key/value tiles up to the
// diagonal.  The two tiles take turns on the tensor pipe, so the softmax of one overlaps the MMAs of the other:
//   warp 0      TMA producer: Q_A, Q_B once, then K_j / V_j into two-stage rings (128B swizzle)
//   warp 1      MMA issuer:   S_X = Q_X K_j^T (TMEM, 128 fp32 columns per tile)  and  O_X += P_X V_j
//   warps 2-5   softmax of tile A, warps 6-9 softmax of tile B: one thread per query row, no exchange between
//               threads.  Two passes over the row in tensor memory (row max, then exp2 / sum / bf16 pack); P is
//               written back over the S columns it came from (tcgen05.st) and is the A operand of the P V MMA
//               straight from tensor memory.  O is rescaled in TMEM only when the running max moved by more
//               than 2^8 (vote per warp).
// Tensor-pipe order per key tile j: P_A V_j, S_A(j+1), P_B V_j, S_B(j+1).
#include "ptx.cuh"

namespace b200 {

int make_tmap_bf16_2d(CUtensorMap* tm, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                      uint32_t box_rows);

__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// 2^x on the FMA and integer pipes (no special-function unit): round x to the nearest integer n with the
// 1.5 * 2^23 trick, evaluate a cubic on the remainder in [-0.5, 0.5] (relative error 8e-5, far below bf16
// rounding of the result) and add n to the exponent field.  x must be <= 127; x below -126 gives 2^-126.
__device__ __forceinline__ float fa_exp2_poly(float x) {
  x = fmaxf(x, -126.f);
  const float t = x + 12582912.f;
  const float f = x - (t - 12582912.f);
  float pl = fmaf(f, 0.05508868f, 0.24260405f);
  pl = fmaf(pl, f, 0.69327624f);
  pl = fmaf(pl, f, 0.99992894f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(t) << 23));
}

// Packed fp32 pairs: one FMA-pipe instruction for two elements.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n\t"
      ".reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %4};\n\t"
      "mov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1) {   // (d0, d1) += (a0, a1)
  asm("{\n\t"
      ".reg .b64 ra, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rd, {%0, %1};\n\t"
      "add.rn.f32x2 rd, rd, ra;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1));
}

constexpr int FA_POLY_PER_8 = 0;   // of every 8 exponentials, this many are evaluated by fa_exp2_poly

constexpr int FA_BQ = 128;   // queries per tile (two tiles per CTA)
constexpr int FA_BK = 128;   // keys per step
constexpr int FA_THREADS = 64 + 256;   // TMA warp, MMA warp, 4 + 4 softmax warps

struct FlashFwdParams {
  __nv_bfloat16* o;      // (rows, d)
  float* lse;            // (batch, heads, seq)
  const int* cu_seqlens; // optional (batch+1) row offsets for packed variable-length sequences
  int batch, seq, heads, d;  // d = heads * dh; seq = max sequence length when cu_seqlens is given
  int n_qblk;            // 128-query tiles per sequence; a CTA takes two of them
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
  static constexpr int OFF_Q = 0;                     // Q_A, Q_B
  static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_V + 2 * TILE_BYTES;
  static constexpr int NUM_BARS = 1 + 4 + 4 + 2 + 4 + 2;  // q, k full/empty, v full/empty, s_full[2], p_full[2][2], o_full[2]
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
  uint64_t* k_empty = bars + 3;   // [2]  both tiles' S MMAs on this K stage have been issued and completed
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]  both tiles' P V MMAs on this V stage have completed
  uint64_t* s_full = bars + 9;    // [2]  per tile: S_X(j) is in tensor memory (and P_X V_{j-1} has completed)
  uint64_t* p_full = bars + 11;   // [2][2]  per tile and half of the key tile: P_X(j) is in tensor memory (128 arrivals)
  uint64_t* o_full = bars + 15;   // [2]  per tile: the last P V MMA has completed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
  volatile uint32_t* abort_word = tmem_holder + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Work assignment: longest-first over the whole grid (latest query tiles = most key steps), so the tail of the
  // launch is made of short CTAs; the (b, h) index varies fastest.
  const int n_pair = (p.n_qblk + 1) >> 1;
  const int bh = blockIdx.x % (p.batch * p.heads);
  const int pair = n_pair - 1 - blockIdx.x / (p.batch * p.heads);
  const int b = bh / p.heads, h = bh % p.heads;
  int row_base, seq_len;
  if (p.cu_seqlens != nullptr) {
    row_base = p.cu_seqlens[b];
    seq_len = p.cu_seqlens[b + 1] - row_base;
  } else {
    row_base = b * p.seq;
    seq_len = p.seq;
  }
  // CTA-uniform tile geometry: tile X covers queries [q0[X], q0[X] + 128) and key tiles 0 .. n_kv_t[X] - 1
  const int q0_t[2] = {pair * 2 * FA_BQ, pair * 2 * FA_BQ + FA_BQ};
  int n_kv_t[2];
#pragma unroll
  for (int x = 0; x < 2; ++x)
    n_kv_t[x] = q0_t[x] < seq_len ? (min(q0_t[x] + FA_BQ, seq_len) + FA_BK - 1) / FA_BK : 0;
  const int n_kv = max(n_kv_t[0], n_kv_t[1]);
  const bool active = n_kv > 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[2 * i], 128);
      mbar_init(&p_full[2 * i + 1], 128);
      mbar_init(&o_full[i], 1);
    }
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
  // columns: S_A [0,128)  S_B [128,256)  O_A [256,256+DH)  O_B [384,384+DH); P_X overlays the first 64 columns of S_X

  const int col_q = h * DH, col_k = p.d + h * DH, col_v = 2 * p.d + h * DH;

  if (warp == 0) {
    if (active && elect_one()) {   // elect.sync keeps the issuing code warp-uniform (descriptors in uniform registers)
      // rows past the end of the tensor are zero-filled by TMA; rows of a following packed sequence are masked or unused
      mbar_expect_tx(q_full, 2 * L::TILE_BYTES);
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int pn = 0; pn < L::PANELS; ++pn)
          tma_load_2d(smem + L::OFF_Q + x * L::TILE_BYTES + pn * 16384, &tm_qkv, q_full, col_q + pn * 64,
                      row_base + q0_t[x]);
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
    if (active && elect_one()) {
      const int lane = 0;   // the tracing macro stamps from the issuing thread
      (void)lane;
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, FA_BK, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, DH, false, true);
      auto issue_s = [&](int x, int j) {   // S_X(j) = Q_X K_j^T
        const uint64_t q_desc = make_smem_desc(smem_u32(smem + L::OFF_Q + x * L::TILE_BYTES), 16, 1024);
        const uint64_t k_desc = make_smem_desc(smem_u32(smem + L::OFF_K + (j & 1) * L::TILE_BYTES), 16, 1024);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t off = ((k / 4) * 16384 + (k % 4) * 32) >> 4;
          umma_f16_ss(tmem_base + x * 128, q_desc + off, k_desc + off, idesc_qk, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[x]);
      };
      // O_X += P_X(j) V_j, one half of the key tile at a time (the softmax warps publish P in two halves):
      // A = P from tensor memory (16 keys = 8 packed columns), B = V MN-major (dh contiguous, keys are rows of
      // 128 B): 16 keys = 2048 B; dh panels 16384 B apart.
      auto issue_pv = [&](int x, int j, int half) {
        const uint64_t v_desc = make_smem_desc(smem_u32(smem + L::OFF_V + (j & 1) * L::TILE_BYTES), 16384, 1024);
#pragma unroll
        for (int kk = 0; kk < FA_BK / 32; ++kk) {
          const int k = half * (FA_BK / 32) + kk;
          umma_f16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + k * 8, v_desc + ((k * 2048) >> 4), idesc_pv,
                      (j > 0 || k > 0) ? 1u : 0u);
        }
        if (half == 1 && j == n_kv_t[x] - 1) umma_commit(&o_full[x]);
      };
      bool ok = mbar_wait(q_full, 0, abort_word) && mbar_wait(&k_full[0], 0, abort_word);
      if (ok) {
        tc_fence_after();
        if (n_kv_t[0] > 0) issue_s(0, 0);
        if (n_kv_t[1] > 0) issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        bool v_ready = false, k_ready = false;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (j < n_kv_t[x]) {
            ok = mbar_wait(&p_full[2 * x], j & 1, abort_word) && (v_ready || mbar_wait(&v_full[st], ph, abort_word));
            if (!ok) break;
            v_ready = true;
            tc_fence_after();
            FWD_TRACE(1, j, x * 4 + 0);
            issue_pv(x, j, 0);
            ok = mbar_wait(&p_full[2 * x + 1], j & 1, abort_word);
            if (!ok) break;
            tc_fence_after();
            issue_pv(x, j, 1);
            FWD_TRACE(1, j, x * 4 + 1);
          }
          if (x == 1) umma_commit(&v_empty[st]);   // both tiles are done with V_j
          if (j + 1 < n_kv_t[x]) {
            ok = k_ready || mbar_wait(&k_full[st ^ 1], ((j + 1) >> 1) & 1, abort_word);
            if (!ok) break;
            k_ready = true;
            tc_fence_after();
            issue_s(x, j + 1);
            FWD_TRACE(1, j, x * 4 + 2);
          }
        }
        if (ok && j + 1 < n_kv) umma_commit(&k_empty[st ^ 1]);   // both tiles are done with K_{j+1}
      }
      if (!ok) *abort_word = ERR_WAIT_FULL;
    }
  } else if (active) {
    // ----------------------------------------------------------------- softmax warps: one thread per query row
    const int x = (warp - 2) >> 2;              // tile A (warps 2-5) or B (warps 6-9)
    const int quarter = warp & 3;               // TMEM lanes [32*quarter, 32*quarter+32) are visible to this warp
    const int r = quarter * 32 + lane;          // row inside the query tile
    const int q0 = (pair * 2 + x) * FA_BQ;
    const int n_kv_x = q0 < seq_len ? (min(q0 + FA_BQ, seq_len) + FA_BK - 1) / FA_BK : 0;
    const int q_idx = q0 + r;                   // position inside the sequence
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const uint32_t tm_s = tmem_base + x * 128 + lane_addr;
    const uint32_t tm_o = tmem_base + 256 + x * 128 + lane_addr;
    float m_run = -INFINITY;                    // running reference max in scaled log2 units
    float l_run = 0.f;                          // running row sum relative to m_run
    bool ok = true;
    for (int j = 0; j < n_kv_x; ++j) {
      const int trole = warp;
      FWD_TRACE(trole, j, 0);
      if (!mbar_wait(&s_full[x], j & 1, abort_word)) { ok = false; break; }
      tc_fence_after();
      FWD_TRACE(trole, j, 1);
      const int k0 = j * FA_BK;
      const bool diag = (k0 + FA_BK - 1 > q0);   // tile touches the diagonal (warp-uniform)
      // pass 1: row maximum over the raw scores (the softmax scale is positive, so it is applied afterwards).
      // The load of chunk c+1 is in flight while chunk c is reduced.
      float mx = -INFINITY;
      {
        uint32_t sa[32], sb[32];
        tmem_ld_32x32(tm_s, sa);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < FA_BK / 32; ++c) {
          uint32_t (&cur)[32] = (c & 1) ? sb : sa;
          uint32_t (&nxt)[32] = (c & 1) ? sa : sb;
          if (c + 1 < FA_BK / 32) tmem_ld_32x32(tm_s + (c + 1) * 32, nxt);
          if (diag) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (k0 + c * 32 + i > q_idx) cur[i] = 0xff800000u;   // -inf
          }
#pragma unroll
          for (int i = 0; i < 32; i += 2) mx = fmax3(mx, __uint_as_float(cur[i]), __uint_as_float(cur[i + 1]));
          if (c + 1 < FA_BK / 32) tmem_ld_wait();
        }
      }
      mx *= p.scale_log2;
      FWD_TRACE(trole, j, 2);
      // Lazy rescale: keep the old reference max unless it moved by more than 8 (a factor 256).
      float m_new = m_run;
      if (mx > m_run + 8.f) m_new = mx;
      const bool need = m_new != m_run;
      const float alpha = (m_run == -INFINITY) ? 0.f : fa_exp2(m_run - m_new);
      // S_X(j) was issued after P_X V_{j-1}, so that MMA has completed and O_X may be rescaled here.
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        const float f = need ? alpha : 1.f;
#pragma unroll 1
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tm_o + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tmem_st_32x32(tm_o + c * 32, o);
        }
      }
      FWD_TRACE(trole, j, 3);
      // pass 2: P = exp2(S * scale - m), row sum, bf16 pack; P chunk c (16 packed columns) lands on S columns
      // [16c, 16c+16), all of which this thread has already read.
      float sum = 0.f, sum1 = 0.f;
      {
        uint32_t sa[32], sb[32];
        tmem_ld_32x32(tm_s, sa);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < FA_BK / 32; ++c) {
          uint32_t (&s)[32] = (c & 1) ? sb : sa;
          uint32_t (&nxt)[32] = (c & 1) ? sa : sb;
          uint32_t pk[16];
          if (c + 1 < FA_BK / 32) tmem_ld_32x32(tm_s + (c + 1) * 32, nxt);   // in flight while this chunk is processed
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0, x1;
            fma2(x0, x1, __uint_as_float(s[i]), __uint_as_float(s[i + 1]), p.scale_log2, -m_new);
            float e0 = ((i & 7) < FA_POLY_PER_8) ? fa_exp2_poly(x0) : fa_exp2(x0);
            float e1 = (((i + 1) & 7) < FA_POLY_PER_8) ? fa_exp2_poly(x1) : fa_exp2(x1);
            if (diag) {
              e0 = (k0 + c * 32 + i > q_idx) ? 0.f : e0;
              e1 = (k0 + c * 32 + i + 1 > q_idx) ? 0.f : e1;
            }
            add2(sum, sum1, e0, e1);
            pk[i / 2] = pack_bf16x2(e0, e1);
          }
          if (c + 1 < FA_BK / 32) tmem_ld_wait();   // before the store below: wait::ld covers the prefetched chunk
          tmem_st_32x16(tm_s + c * 16, pk);
          if (c == 1 || c == 3) {   // publish this half of P
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&p_full[2 * x + (c >> 1)]);
          }
        }
      }
      l_run = l_run * (need ? alpha : 1.f) + (sum + sum1);
      m_run = m_new;
      FWD_TRACE(trole, j, 4);
    }
    // ------------------------------------------------------------------- epilogue
    if (ok && n_kv_x > 0) ok = mbar_wait(&o_full[x], 0, abort_word);
    if (ok && n_kv_x > 0) {
      tc_fence_after();
      const float inv_l = 1.f / l_run;
      const bool valid = q_idx < seq_len;
      __nv_bfloat16* orow = p.o + (size_t)(row_base + q_idx) * p.d + h * DH;
#pragma unroll 1
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tm_o + c * 32, o);
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
      if (valid && p.lse != nullptr)
        p.lse[((size_t)b * p.heads + h) * p.seq + q_idx] = (m_run + log2f(l_run)) * 0.6931471805599453f;
    } else if (!ok && lane == 0) {
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
  const int grid = p.batch * p.heads * ((p.n_qblk + 1) / 2);   // one CTA per pair of query tiles
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
