// Shared pieces of the tcgen05 GEMM kernels: problem description, tile order and the fused epilogue.
#pragma once
#include "comm_device.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;

enum GemmEpilogue : int {
  EPI_BF16 = 0,       // C = bf16(acc)
  EPI_F32 = 1,        // C = acc (fp32)
  EPI_BF16_RES = 2,   // C = bf16(acc + R)   (R bf16, may alias C)
  EPI_F32_ACC = 3,    // C += acc (fp32 read-modify-write)
  // Backward of h = silu(gate) * up fused into the GEMM that produces dh = acc (M x N): R holds gate | up
  // (M x 2N, bf16) and C (M x 2N, bf16) receives d(gate) | d(up).
  EPI_SWIGLU_BWD = 4,
  // Flag or-ed into the epilogue code by the caller (CTA-pair kernel): output columns from N up to the next 16-byte
  // boundary lie inside the row pitch and may be overwritten with zeros.
  EPI_PAD_WRITABLE = 0x100,
  // Flag or-ed into the epilogue code by the caller (single-CTA kernel): operand B is not written by the kernel
  // before this one on the stream (inference weights), so its first tiles may be requested before that kernel ends.
  EPI_B_STABLE = 0x200,
};

// Optional all-gather carried by a GEMM launch: while the MMA warps work, two copy warps per CTA pull
// the weight shards of the *next* FSDP unit from every peer GPU into a local buffer (plain 16-byte peer
// loads, no TMA, no multicast).  `done` is bumped once per CTA when its slice has landed, so a consumer
// on another stream can wait for `done >= expected` instead of a kernel boundary.
struct GatherTask {
  const uint4* src[16];          // shard base address of every rank as mapped on this GPU
  uint4* dst;                    // local buffer of world * shard_vec vectors; null = no gather
  unsigned long long shard_vec;  // 16-byte vectors per shard
  int world, rank;
  uint32_t* done;
};

struct GemmParams {
  GatherTask gather;
  // Optional reduce-scatter (+ scale + sum of squares, or + AdamW) of an earlier FSDP unit's gradient staging, run
  // by the same copy warps after the gather (CTA-pair kernel only); reduce.n == 0 = none.
  ReduceTask reduce;
  const uint32_t* wait_counter;  // optional: do not touch operand B before *wait_counter >= wait_value
  uint32_t wait_value;
  unsigned long long wait_limit_ns;   // how long the producer warp polls wait_counter before it gives up
  // Optional rotary embedding fused into the epilogue of the QKV projection: output columns [0, 2*rope_d)
  // (the Q and K thirds) are rotated pair-wise by the angle of position (row % rope_seq); the table is
  // (2, rope_ctx, rope_dh/2) fp32 (cos, then sin).  Null = off.
  const float* rope_cs;
  int rope_seq, rope_d, rope_dh, rope_ctx;
  // Optional SwiGLU fused into the epilogue of the merged gate|up projection (CTA-pair kernel only): B is
  // (2F, K) with gate rows first; a tile then holds 128 gate columns and the matching 128 up columns, C
  // receives both (they are needed by the backward pass) and H (M x F, bf16) receives silu(gate) * up.
  int swiglu_f;        // F, 0 = off
  void* H;
  long long ldh;
  int M, N, K;
  void* C;
  long long ldc;
  const void* R;
  long long ldr;
  int epi;
  int tma_store;       // CTA-pair kernel: the epilogue stages tiles in shared memory and writes them with TMA stores
  int num_m_tiles, num_n_tiles, group_m;
  uint32_t* status;
  // Split-K (single-CTA kernel, small M): `splits` CTAs share an output tile, each contracts a slice of K and leaves
  // an fp32 partial tile in `ws`; the epilogue warp that arrives last at the counter of its 32 rows adds their partials in
  // split order (so the result does not depend on which CTA that is) and runs the epilogue.  splits <= 1 = off.
  // B (the weights) does not depend on the kernel before this one: as a programmatic dependent the kernel requests
  // its first B tiles before it waits for that kernel, so the weights' DRAM latency overlaps the predecessor's tail.
  int b_early;
  int splits;
  float* ws;                  // splits * tiles partial tiles of BM x BN floats
  uint32_t* tile_counters;    // four per tile (one per 32-row quarter), zero between launches (the last warp resets its own)
};

__device__ __forceinline__ void tile_coords(int tile, const GemmParams& p, int& m_blk, int& n_blk) {
  const int per_group = p.group_m * p.num_n_tiles;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gm = min(p.group_m, p.num_m_tiles - first_m);
  const int r = tile - g * per_group;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

__device__ __forceinline__ void report(const GemmParams& p, volatile uint32_t* abort_word, uint32_t code) {
  *abort_word = code;
  if (p.status != nullptr) atomicCAS(p.status, 0u, code | (blockIdx.x << 8));
}

// Interleaved-pair rotation of a 32-column accumulator chunk (16 pairs, all inside one head).
__device__ __forceinline__ void epilogue_rope(const GemmParams& p, int row, int col0, uint32_t (&acc)[32]) {
  const int pos = row % p.rope_seq;
  const int e = col0 % p.rope_dh;                       // multiple of 32
  const float* cs = p.rope_cs + (size_t)pos * (p.rope_dh / 2) + e / 2;
  const float* sn = cs + (size_t)p.rope_ctx * (p.rope_dh / 2);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 c4 = *reinterpret_cast<const float4*>(cs + q * 4);
    const float4 s4 = *reinterpret_cast<const float4*>(sn + q * 4);
    const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float x0 = __uint_as_float(acc[q * 8 + 2 * t]), x1 = __uint_as_float(acc[q * 8 + 2 * t + 1]);
      acc[q * 8 + 2 * t] = __float_as_uint(cc[t] * x0 - ss[t] * x1);
      acc[q * 8 + 2 * t + 1] = __float_as_uint(ss[t] * x0 + cc[t] * x1);
    }
  }
}

// One 32-column chunk of one output row.
__device__ __forceinline__ void epilogue_store(const GemmParams& p, int row, int col0, uint32_t (&acc)[32]) {
  if (row >= p.M) return;
  const int ncols = min(32, p.N - col0);
  if (ncols <= 0) return;
  if (p.rope_cs != nullptr && col0 < 2 * p.rope_d && ncols == 32) epilogue_rope(p, row, col0, acc);
  if (p.epi == EPI_SWIGLU_BWD) {
    // as the stand-alone kernel (fast division apart): dh is rounded to bf16 first, gate and up are read as bf16
    const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(p.R) + (long long)row * p.ldr + col0;
    const __nv_bfloat16* up = gp + p.N;
    __nv_bfloat16* dgp = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
    __nv_bfloat16* dup = dgp + p.N;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j * 8 >= ncols) break;          // N, ldr and ldc are multiples of 8 (checked on the host)
      const uint4 gv = *reinterpret_cast<const uint4*>(gp + j * 8);
      const uint4 uv = *reinterpret_cast<const uint4*>(up + j * 8);
      const uint32_t gg[4] = {gv.x, gv.y, gv.z, gv.w}, uu[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t og[4], ou[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 g = unpack_bf16x2(gg[t]), u = unpack_bf16x2(uu[t]);
        const float2 d = unpack_bf16x2(pack_bf16x2(__uint_as_float(acc[j * 8 + 2 * t]), __uint_as_float(acc[j * 8 + 2 * t + 1])));
        const float s0 = __fdividef(1.f, 1.f + __expf(-g.x)), s1 = __fdividef(1.f, 1.f + __expf(-g.y));
        const float l0 = g.x * s0, l1 = g.y * s1;
        og[t] = pack_bf16x2(d.x * u.x * (s0 + l0 * (1.f - s0)), d.y * u.y * (s1 + l1 * (1.f - s1)));
        ou[t] = pack_bf16x2(d.x * l0, d.y * l1);
      }
      *reinterpret_cast<uint4*>(dgp + j * 8) = make_uint4(og[0], og[1], og[2], og[3]);
      *reinterpret_cast<uint4*>(dup + j * 8) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
    }
    return;
  }
  if (p.epi == EPI_BF16 || p.epi == EPI_BF16_RES) {
    __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
    const bool vec_ok = (ncols == 32) && ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    if (p.epi == EPI_BF16_RES) {
      const __nv_bfloat16* r = reinterpret_cast<const __nv_bfloat16*>(p.R) + (long long)row * p.ldr + col0;
      const bool rvec = vec_ok && ((p.ldr & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.R) & 15) == 0);
      if (rvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 rv = *reinterpret_cast<const uint4*>(r + j * 8);
          const uint32_t rr[4] = {rv.x, rv.y, rv.z, rv.w};
          uint32_t o[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            float2 f = unpack_bf16x2(rr[t]);
            o[t] = pack_bf16x2(__uint_as_float(acc[j * 8 + 2 * t]) + f.x,
                               __uint_as_float(acc[j * 8 + 2 * t + 1]) + f.y);
          }
          *reinterpret_cast<uint4*>(c + j * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)    // static register indices keep the accumulator chunk out of local memory
          if (j < ncols) c[j] = __float2bfloat16(__uint_as_float(acc[j]) + __bfloat162float(r[j]));
      }
    } else if (vec_ok) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t o[4];
#pragma unroll
        for (int t = 0; t < 4; ++t)
          o[t] = pack_bf16x2(__uint_as_float(acc[j * 8 + 2 * t]), __uint_as_float(acc[j * 8 + 2 * t + 1]));
        *reinterpret_cast<uint4*>(c + j * 8) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) c[j] = __float2bfloat16(__uint_as_float(acc[j]));
    }
  } else {
    float* c = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
    const bool vec_ok = (ncols == 32) && ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    if (p.epi == EPI_F32) {
      if (vec_ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(c + j * 4) = make_uint4(acc[j * 4], acc[j * 4 + 1], acc[j * 4 + 2], acc[j * 4 + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) c[j] = __uint_as_float(acc[j]);
      }
    } else {  // EPI_F32_ACC
      if (vec_ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 v = *reinterpret_cast<float4*>(c + j * 4);
          v.x += __uint_as_float(acc[j * 4]);
          v.y += __uint_as_float(acc[j * 4 + 1]);
          v.z += __uint_as_float(acc[j * 4 + 2]);
          v.w += __uint_as_float(acc[j * 4 + 3]);
          *reinterpret_cast<float4*>(c + j * 4) = v;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) c[j] += __uint_as_float(acc[j]);
      }
    }
  }
}

}  // namespace b200
