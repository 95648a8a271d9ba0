// Decode-time attention over a paged KV cache (16-token pages by default) for sm_100a, plus the kernel
// that appends the new K / V rows to the cache.  The reference has no KV cache at all: its generate()
// re-runs the full forward for every token (llm-core/llm_core/model.py:187-236).
//
// Cache layout per layer: (num_pages, page_size, H*dh) bf16 for K and for V.  A request's tokens live in
// the pages listed in its row of `block_tables`.
//
// Decode attention is bandwidth bound (every cached K and V byte is read once per step), so the kernel is
// organised around fully coalesced 16-byte loads: 16 lanes cover the 256 bytes of one token's head
// (dh = 128; 8 lanes for dh = 64), each warp streams two (four) tokens per iteration, scores are reduced
// with shuffles, and the softmax is kept online.  The context of one (request, head) is split over
// gridDim.y CTAs (flash-decoding); partial (max, sum, output) triples go to a scratch buffer and a
// second kernel merges them.
#include "ptx.cuh"

namespace b200 {

constexpr int PD_THREADS = 128;

template <int DH>
__global__ void __launch_bounds__(PD_THREADS)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q,        // (R, 3d) packed qkv or (R, d): row stride q_ld
                    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                    const int* __restrict__ block_tables, const int* __restrict__ context_lens,
                    float* __restrict__ part_o,                  // (R, H, splits, DH)
                    float* __restrict__ part_ml,                 // (R, H, splits, 2)
                    int q_ld, int heads, int page_size, int max_pages, int splits, float scale_log2, int num_pages,
                    uint32_t* __restrict__ status) {
  constexpr int LPT = DH / 8;            // lanes per token (16-byte loads)
  constexpr int TPW = 32 / LPT;          // tokens per warp iteration
  const int r = blockIdx.x / heads, h = blockIdx.x % heads;
  const int split = blockIdx.y;
  // The tables come from the host scheduler; a length beyond the table or a page id beyond the cache is reported
  // through the status word and skipped, never dereferenced.
  int ctx = context_lens[r];
  if (ctx < 0 || ctx > max_pages * page_size) {
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0u, ERR_BAD_ARG | (1u << 8));
    ctx = ctx < 0 ? 0 : max_pages * page_size;
  }
  const int d = heads * DH;
  const int per = (ctx + splits - 1) / splits;
  const int t0 = split * per;
  const int t1 = min(ctx, t0 + per);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPT;            // which token of the warp's group
  const int li = lane % LPT;             // which 8-element slice of the head

  float qv[8];
  {
    const uint4 u = *reinterpret_cast<const uint4*>(q + (size_t)r * q_ld + h * DH + li * 8);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
    qv[0] = a.x; qv[1] = a.y; qv[2] = b.x; qv[3] = b.y; qv[4] = c.x; qv[5] = c.y; qv[6] = e.x; qv[7] = e.y;
  }
  float m = -INFINITY, l = 0.f;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int* table = block_tables + (size_t)r * max_pages;
  // The loop bound is uniform across the warp so that the shuffles below are executed by all 32 lanes;
  // a token group whose index runs past the end of the split only skips its loads and its update.
  for (int tb = t0 + warp * TPW; tb < t1; tb += (PD_THREADS / 32) * TPW) {
    const int t = tb + sub;
    uint4 ku = make_uint4(0, 0, 0, 0), vu = make_uint4(0, 0, 0, 0);
    bool valid = t < t1;
    if (valid) {
      const int page = table[t / page_size];
      if ((unsigned)page >= (unsigned)num_pages) {
        if (status != nullptr) atomicCAS(status, 0u, ERR_BAD_ARG | (2u << 8));
        valid = false;
      } else {
        const size_t row = ((size_t)page * page_size + (t % page_size)) * d + h * DH + li * 8;
        ku = *reinterpret_cast<const uint4*>(k_cache + row);
        vu = *reinterpret_cast<const uint4*>(v_cache + row);
      }
    }
    const float2 k0 = unpack_bf16x2(ku.x), k1 = unpack_bf16x2(ku.y), k2 = unpack_bf16x2(ku.z), k3 = unpack_bf16x2(ku.w);
    float s = qv[0] * k0.x + qv[1] * k0.y + qv[2] * k1.x + qv[3] * k1.y + qv[4] * k2.x + qv[5] * k2.y + qv[6] * k3.x +
              qv[7] * k3.y;
#pragma unroll
    for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (valid) {
      s *= scale_log2;
      const float mn = fmaxf(m, s);
      const float corr = exp2f(m - mn);   // 0 when m == -inf
      const float p = exp2f(s - mn);
      l = l * corr + p;
      const float2 v0 = unpack_bf16x2(vu.x), v1 = unpack_bf16x2(vu.y), v2 = unpack_bf16x2(vu.z), v3 = unpack_bf16x2(vu.w);
      acc[0] = acc[0] * corr + p * v0.x; acc[1] = acc[1] * corr + p * v0.y;
      acc[2] = acc[2] * corr + p * v1.x; acc[3] = acc[3] * corr + p * v1.y;
      acc[4] = acc[4] * corr + p * v2.x; acc[5] = acc[5] * corr + p * v2.y;
      acc[6] = acc[6] * corr + p * v3.x; acc[7] = acc[7] * corr + p * v3.y;
      m = mn;
    }
  }
  // ---- combine the (PD_THREADS / LPT) token groups of the CTA through shared memory
  constexpr int GROUPS = PD_THREADS / LPT;
  __shared__ float sm_m[GROUPS], sm_l[GROUPS];
  __shared__ float sm_o[GROUPS][DH];
  const int grp = threadIdx.x / LPT;
  if (li == 0) { sm_m[grp] = m; sm_l[grp] = l; }
#pragma unroll
  for (int i = 0; i < 8; ++i) sm_o[grp][li * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < DH) {
    float gm = -INFINITY;
    for (int g = 0; g < GROUPS; ++g) gm = fmaxf(gm, sm_m[g]);
    float gl = 0.f, go = 0.f;
    for (int g = 0; g < GROUPS; ++g) {
      const float w = (sm_m[g] == -INFINITY) ? 0.f : exp2f(sm_m[g] - gm);
      gl += sm_l[g] * w;
      go += sm_o[g][threadIdx.x] * w;
    }
    const size_t idx = ((size_t)r * heads + h) * splits + split;
    part_o[idx * DH + threadIdx.x] = go;
    if (threadIdx.x == 0) { part_ml[idx * 2] = gm; part_ml[idx * 2 + 1] = gl; }
  }
}

template <int DH>
__global__ void paged_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          __nv_bfloat16* __restrict__ out, int heads, int splits) {
  const int r = blockIdx.x / heads, h = blockIdx.x % heads;
  const size_t base = ((size_t)r * heads + h) * splits;
  float gm = -INFINITY;
  for (int s = 0; s < splits; ++s) gm = fmaxf(gm, part_ml[(base + s) * 2]);
  float gl = 0.f, go = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - gm);
    gl += part_ml[(base + s) * 2 + 1] * w;
    go += part_o[(base + s) * DH + threadIdx.x] * w;
  }
  out[((size_t)r * heads + h) * DH + threadIdx.x] = __float2bfloat16(gl > 0.f ? go / gl : 0.f);
}

// cache[slot] = K (V) row of qkv for every request row; slot = page * page_size + offset (negative: skip).
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ k_cache,
                                 __nv_bfloat16* __restrict__ v_cache, const long long* __restrict__ slots, long long rows,
                                 int d, long long num_slots, uint32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const long long slot = slots[row];
  if (slot < 0) return;
  if (slot >= num_slots) {      // beyond the cache: report, do not write
    if (lane == 0 && status != nullptr) atomicCAS(status, 0u, ERR_BAD_ARG | (3u << 8));
    return;
  }
  const __nv_bfloat16* src = qkv + (size_t)row * 3 * d;
  for (int c = lane * 8; c < d; c += 256) {
    *reinterpret_cast<uint4*>(k_cache + (size_t)slot * d + c) = *reinterpret_cast<const uint4*>(src + d + c);
    *reinterpret_cast<uint4*>(v_cache + (size_t)slot * d + c) = *reinterpret_cast<const uint4*>(src + 2 * d + c);
  }
}

}  // namespace b200

using namespace b200;

// q: rows of stride q_ld elements whose first d entries are the queries (pass the packed qkv buffer with
// q_ld = 3d).  part_o: R*H*splits*dh floats, part_ml: R*H*splits*2 floats (caller-provided scratch).
extern "C" int b200_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                 const int* context_lens, void* out, float* part_o, float* part_ml, int rows, int q_ld,
                                 int heads, int dh, int page_size, int max_pages, int splits, float scale,
                                 int num_pages, uint32_t* status, cudaStream_t st) {
  if (dh != 64 && dh != 128) return -10;
  if (page_size <= 0 || max_pages <= 0 || num_pages <= 0) return -11;
  if (q_ld % 8 || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15))
    return -10;
  if (rows <= 0) return 0;
  if (splits < 1) splits = 1;
  const dim3 grid(rows * heads, splits);
  const float sl2 = scale * 1.4426950408889634f;
  if (dh == 128) {
    paged_decode_kernel<128><<<grid, PD_THREADS, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                                                          (const __nv_bfloat16*)v_cache, block_tables, context_lens,
                                                          part_o, part_ml, q_ld, heads, page_size, max_pages, splits, sl2,
                                                          num_pages, status);
    paged_decode_merge_kernel<128><<<rows * heads, 128, 0, st>>>(part_o, part_ml, (__nv_bfloat16*)out, heads, splits);
  } else {
    paged_decode_kernel<64><<<grid, PD_THREADS, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                                                         (const __nv_bfloat16*)v_cache, block_tables, context_lens,
                                                         part_o, part_ml, q_ld, heads, page_size, max_pages, splits, sl2,
                                                          num_pages, status);
    paged_decode_merge_kernel<64><<<rows * heads, 64, 0, st>>>(part_o, part_ml, (__nv_bfloat16*)out, heads, splits);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int b200_kv_append(const void* qkv, void* k_cache, void* v_cache, const long long* slots, long long rows,
                              int d, long long num_slots, uint32_t* status, cudaStream_t st) {
  if (d % 8 || (reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15))
    return -10;
  if (rows <= 0) return 0;
  kv_append_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)k_cache,
                                                               (__nv_bfloat16*)v_cache, slots, rows, d, num_slots, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
