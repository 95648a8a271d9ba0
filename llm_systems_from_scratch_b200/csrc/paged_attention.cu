// Decode-time attention over a paged KV cache (16-token pages by default) for sm_100a, plus the kernel
// that appends the new K / V rows to the cache.  The reference has no KV cache at all: its generate()
// re-runs the full forward for every token (llm-core/llm_core/model.py:187-236).
//
// Cache layout per layer: (num_pages, page_size, H*dh) bf16 for K and for V.  A request's tokens live in
// the pages listed in its row of `block_tables`.
//
// Decode attention is bandwidth bound (every cached K and V byte is read once per step), so the kernel is
// organised around reading whole token rows: one CTA serves one request (all its heads) over one split of the
// context, 16 lanes cover the 256 bytes of one head (dh = 128; 8 lanes for dh = 64), scores are reduced with
// shuffles, the softmax is kept online in registers and eight tokens' rows are in flight per thread.  The context
// of a request is split over gridDim.y CTAs (flash-decoding); partial (max, sum, output) triples go to a scratch
// buffer and a second kernel merges them.
#include "ptx.cuh"

namespace b200 {

constexpr int PD_UNROLL = 8;     // tokens whose K / V rows are in flight together, per CTA

// 16-byte load of cache data that is read exactly once per step: do not keep it in L1.
__device__ __forceinline__ uint4 ld_stream(const __nv_bfloat16* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// One CTA = one request x one split of its context; its threads cover ALL heads: thread i owns the 8 head-columns
// [8 i, 8 i + 8) of the token row, so the CTA reads every cached token as one contiguous row of H * DH elements (and
// the 16 tokens of a page as one contiguous 16-row block), which is the access pattern DRAM serves at full speed.
// A head's score is reduced over its DH / 8 neighbouring lanes with shuffles; each thread keeps the online-softmax
// state (max, sum) of its head and its 8 output columns for the whole split, so nothing is combined inside the CTA.
// The K and V rows of PD_UNROLL tokens are requested before the first score is computed.
template <int DH>
__global__ void __launch_bounds__(512)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q,        // (R, 3d) packed qkv or (R, d): row stride q_ld
                    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                    const int* __restrict__ block_tables, const int* __restrict__ context_lens,
                    float* __restrict__ part_o,                  // (R, H, splits, DH)
                    float* __restrict__ part_ml,                 // (R, H, splits, 2)
                    int q_ld, int heads, int page_size, int max_pages, int splits, float scale_log2, int num_pages,
                    uint32_t* __restrict__ status) {
  pdl_sync();
  constexpr int LPT = DH / 8;            // lanes per head (16-byte loads)
  const int r = blockIdx.x, split = blockIdx.y;
  const int d = heads * DH;
  const int col = threadIdx.x * 8;       // first of this thread's 8 columns of the token row
  const bool active = col < d;           // the block is rounded up to whole warps
  const int h = active ? col / DH : 0;
  const int li = (threadIdx.x % LPT);
  // The tables come from the host scheduler; a length beyond the table or a page id beyond the cache is reported
  // through the status word and skipped, never dereferenced.
  int ctx = context_lens[r];
  if (ctx < 0 || ctx > max_pages * page_size) {
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0u, ERR_BAD_ARG | (1u << 8));
    ctx = ctx < 0 ? 0 : max_pages * page_size;
  }
  // splits start on multiples of PD_UNROLL tokens so that a chunk of PD_UNROLL tokens never straddles a page whose
  // size is a multiple of PD_UNROLL: one table lookup (and one integer division) per chunk instead of one per token
  const int per = ((ctx + splits - 1) / splits + PD_UNROLL - 1) / PD_UNROLL * PD_UNROLL;
  const int t0 = split * per;
  const int t1 = min(ctx, t0 + per);

  float qv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (active) {
    const uint4 u = *reinterpret_cast<const uint4*>(q + (size_t)r * q_ld + col);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
    qv[0] = a.x; qv[1] = a.y; qv[2] = b.x; qv[3] = b.y; qv[4] = c.x; qv[5] = c.y; qv[6] = e.x; qv[7] = e.y;
  }
  float m = -INFINITY, l = 0.f;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int* table = block_tables + (size_t)r * max_pages;
  for (int tb = t0; tb < t1; tb += PD_UNROLL) {
    uint4 ku[PD_UNROLL], vu[PD_UNROLL];
    bool valid[PD_UNROLL];
    const int pg = tb / page_size, off = tb - pg * page_size;
    if (off + PD_UNROLL <= page_size) {
      // the whole chunk lies in one page: consecutive rows of the cache
      const int page = table[pg];
      const bool page_ok = (unsigned)page < (unsigned)num_pages;
      if (!page_ok && threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0u, ERR_BAD_ARG | (2u << 8));
      const size_t row0 = ((size_t)(page_ok ? page : 0) * page_size + off) * d + col;
#pragma unroll
      for (int u = 0; u < PD_UNROLL; ++u) {
        valid[u] = page_ok && tb + u < t1;
        ku[u] = make_uint4(0, 0, 0, 0);
        vu[u] = make_uint4(0, 0, 0, 0);
        if (valid[u] && active) {
          ku[u] = ld_stream(k_cache + row0 + (size_t)u * d);
          vu[u] = ld_stream(v_cache + row0 + (size_t)u * d);
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < PD_UNROLL; ++u) {
        const int t = tb + u;
        valid[u] = t < t1;
        ku[u] = make_uint4(0, 0, 0, 0);
        vu[u] = make_uint4(0, 0, 0, 0);
        if (valid[u]) {
          const int page = table[t / page_size];
          if ((unsigned)page >= (unsigned)num_pages) {
            if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0u, ERR_BAD_ARG | (2u << 8));
            valid[u] = false;
          } else if (active) {
            const size_t row = ((size_t)page * page_size + (t % page_size)) * d + col;
            ku[u] = ld_stream(k_cache + row);
            vu[u] = ld_stream(v_cache + row);
          }
        }
      }
    }
    // scores of the whole chunk first (independent of one another), then ONE running-max update for the chunk:
    // the serial chain of the online softmax is per chunk, not per token
    float sc[PD_UNROLL];
    float mc = m;
#pragma unroll
    for (int u = 0; u < PD_UNROLL; ++u) {
      const float2 k0 = unpack_bf16x2(ku[u].x), k1 = unpack_bf16x2(ku[u].y), k2 = unpack_bf16x2(ku[u].z),
                   k3 = unpack_bf16x2(ku[u].w);
      float s = qv[0] * k0.x + qv[1] * k0.y + qv[2] * k1.x + qv[3] * k1.y + qv[4] * k2.x + qv[5] * k2.y +
                qv[6] * k3.x + qv[7] * k3.y;
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      sc[u] = valid[u] ? s * scale_log2 : -INFINITY;
      mc = fmaxf(mc, sc[u]);
    }
    if (mc > -INFINITY) {
      const float corr = exp2f(m - mc);       // 0 when m == -inf
      l *= corr;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= corr;
#pragma unroll
      for (int u = 0; u < PD_UNROLL; ++u) {
        const float p = exp2f(sc[u] - mc);    // 0 for tokens beyond the split or on a bad page
        l += p;
        const float2 v0 = unpack_bf16x2(vu[u].x), v1 = unpack_bf16x2(vu[u].y), v2 = unpack_bf16x2(vu[u].z),
                     v3 = unpack_bf16x2(vu[u].w);
        acc[0] += p * v0.x; acc[1] += p * v0.y; acc[2] += p * v1.x; acc[3] += p * v1.y;
        acc[4] += p * v2.x; acc[5] += p * v2.y; acc[6] += p * v3.x; acc[7] += p * v3.y;
      }
      m = mc;
    }
  }
  if (active) {
    const size_t idx = ((size_t)r * heads + h) * splits + split;
    float4* o = reinterpret_cast<float4*>(part_o + idx * DH + li * 8);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (li == 0) { part_ml[idx * 2] = m; part_ml[idx * 2 + 1] = l; }
  }
}

template <int DH>
__global__ void paged_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          __nv_bfloat16* __restrict__ out, int heads, int splits) {
  pdl_sync();
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
  pdl_sync();
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

// Rotary embedding of the Q and K thirds of qkv (in place, interleaved pairs, angle of positions[row]) and the append
// of the rotated K row and the V row to their cache slot, in one pass over the row: what rope_kernel followed by
// kv_append_kernel do, with one launch and one read of K less.  slot < 0: rotate only.
__global__ void rope_kv_append_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_sin,
                                      const int* __restrict__ positions, __nv_bfloat16* __restrict__ k_cache,
                                      __nv_bfloat16* __restrict__ v_cache, const long long* __restrict__ slots,
                                      long long rows, int d, int dh, int ctx, long long num_slots,
                                      uint32_t* __restrict__ status) {
  pdl_sync();
  const int gpr = 3 * d / 8;             // groups of 8 elements per row
  const long long groups = rows * gpr;
  const float* cosb = cos_sin;
  const float* sinb = cos_sin + (size_t)ctx * (dh / 2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < groups;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / gpr;
    const int c = (int)(i - row * gpr) * 8;            // column within [0, 3d)
    long long slot = slots[row];
    if (slot >= num_slots) {                           // beyond the cache: report, do not write
      if (c == 0 && status != nullptr) atomicCAS(status, 0u, ERR_BAD_ARG | (3u << 8));
      slot = -1;
    }
    __nv_bfloat16* p = qkv + row * 3 * d + c;
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    if (c < 2 * d) {
      const int pos = positions[row];
      const int e = c % dh;                            // element offset inside the head (multiple of 8)
      const float4 cs = *reinterpret_cast<const float4*>(cosb + (size_t)pos * (dh / 2) + e / 2);
      const float4 sn = *reinterpret_cast<const float4*>(sinb + (size_t)pos * (dh / 2) + e / 2);
      const float cc[4] = {cs.x, cs.y, cs.z, cs.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
      const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 v = unpack_bf16x2(in[k]);
        o[k] = pack_bf16x2(cc[k] * v.x - ss[k] * v.y, ss[k] * v.x + cc[k] * v.y);
      }
      raw = make_uint4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<uint4*>(p) = raw;
    }
    if (slot >= 0 && c >= d) {
      __nv_bfloat16* dst = (c < 2 * d) ? k_cache + (size_t)slot * d + (c - d) : v_cache + (size_t)slot * d + (c - 2 * d);
      *reinterpret_cast<uint4*>(dst) = raw;
    }
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
  const int threads = (heads * (dh / 8) + 31) / 32 * 32;      // one thread per 8 columns of the token row, whole warps
  if (threads > 512) return -12;     // heads * dh <= 4096
  const dim3 grid(rows, splits);
  const float sl2 = scale * 1.4426950408889634f;
  if (dh == 128) {
    launch_dep(paged_decode_kernel<128>, grid, threads, 0, st, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
               (const __nv_bfloat16*)v_cache, block_tables, context_lens, part_o, part_ml, q_ld, heads, page_size,
               max_pages, splits, sl2, num_pages, status);
    launch_dep(paged_decode_merge_kernel<128>, rows * heads, 128, 0, st, part_o, part_ml, (__nv_bfloat16*)out, heads,
               splits);
  } else {
    launch_dep(paged_decode_kernel<64>, grid, threads, 0, st, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
               (const __nv_bfloat16*)v_cache, block_tables, context_lens, part_o, part_ml, q_ld, heads, page_size,
               max_pages, splits, sl2, num_pages, status);
    launch_dep(paged_decode_merge_kernel<64>, rows * heads, 64, 0, st, part_o, part_ml, (__nv_bfloat16*)out, heads,
               splits);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int b200_kv_append(const void* qkv, void* k_cache, void* v_cache, const long long* slots, long long rows,
                              int d, long long num_slots, uint32_t* status, cudaStream_t st) {
  if (d % 8 || (reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15))
    return -10;
  if (rows <= 0) return 0;
  launch_dep(kv_append_kernel, (unsigned)((rows + 7) / 8), 256, 0, st, (const __nv_bfloat16*)qkv,
             (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slots, rows, d, num_slots, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Rotary embedding of Q and K in place plus the append of K and V to their cache slots, one launch.
extern "C" int b200_rope_kv_append(void* qkv, const float* cos_sin, const int* positions, void* k_cache, void* v_cache,
                                   const long long* slots, long long rows, int d, int dh, int ctx, long long num_slots,
                                   uint32_t* status, cudaStream_t st) {
  if (dh % 8 || d % dh || positions == nullptr || slots == nullptr ||
      ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
        reinterpret_cast<uintptr_t>(cos_sin)) & 15))
    return -10;
  if (rows <= 0) return 0;
  const long long groups = rows * (3 * d / 8);
  long long blocks = (groups + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_dep(rope_kv_append_kernel, (unsigned)blocks, 256, 0, st, (__nv_bfloat16*)qkv, cos_sin, positions,
             (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slots, rows, d, dh, ctx, num_slots, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
