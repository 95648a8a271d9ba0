// Temperature / top-k sampling of one token per row of bf16 logits, one launch for the whole batch:
// the filter, the softmax and the draw of the reference's generation loop
// (llm-core/llm_core/model.py:213-231: divide by the temperature, keep the top-k logits, softmax,
// torch.multinomial) without materialising probabilities or sorting the vocabulary.
//
// One block per row:
//   1. top-k threshold by radix select on the order-preserving 16-bit key of the bf16 logit: a 256-bin
//      histogram of the high byte, then of the low byte inside the selected bin.  Every logit >= the k-th
//      largest is kept (ties included, like `logits < kth -> -inf`).
//   2. row maximum and sum of exp((x - max) / T) over the kept logits (fp32).
//   3. inverse-CDF draw with the caller's uniform u in [0, 1): each thread owns a contiguous slice of the
//      vocabulary, a block scan of the slice sums finds the slice, a serial walk finds the token.
#include "ptx.cuh"

namespace b200 {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ uint32_t bf16_key(uint16_t bits) {   // larger float <=> larger key
  return (bits & 0x8000u) ? (~bits & 0xffffu) : (bits | 0x8000u);
}

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, w) : v + w;
  }
  __syncthreads();            // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = lane < (SAMPLE_THREADS / 32) ? red[lane] : (is_max ? -INFINITY : 0.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, w) : v + w;
  }
  return v;                   // every thread of every warp holds the result
}

// Scans hist[255..0] for the bin where the running count reaches `need`; returns the bin and the count above it.
__device__ __forceinline__ void select_bin(const uint32_t* hist, uint32_t need, uint32_t* sel) {
  if (threadIdx.x == 0) {
    uint32_t above = 0;
    int b = 255;
    for (; b > 0; --b) {
      if (above + hist[b] >= need) break;
      above += hist[b];
    }
    sel[0] = (uint32_t)b;
    sel[1] = above;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_topk_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int vocab, const float* __restrict__ uniforms,
                   float inv_temperature, int top_k, long long* __restrict__ out) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t sel[2];
  __shared__ float red[32];
  __shared__ float warp_sums[32];
  __shared__ int result;
  const uint16_t* row = reinterpret_cast<const uint16_t*>(logits) + (long long)blockIdx.x * ld;
  const int tid = threadIdx.x;

  // ---- 1. threshold key: all logits with key >= thr are kept
  uint32_t thr = 0;
  if (top_k > 0 && top_k < vocab) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) atomicAdd(&hist[bf16_key(row[i]) >> 8], 1u);
    __syncthreads();
    select_bin(hist, (uint32_t)top_k, sel);
    const uint32_t hi = sel[0], need_lo = (uint32_t)top_k - sel[1];
    __syncthreads();
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
      const uint32_t key = bf16_key(row[i]);
      if ((key >> 8) == hi) atomicAdd(&hist[key & 0xff], 1u);
    }
    __syncthreads();
    select_bin(hist, need_lo, sel);
    thr = (hi << 8) | sel[0];
  }

  // ---- 2. maximum and normaliser over the kept logits; thread t owns tokens [t*per, (t+1)*per)
  const int per = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int i0 = min(tid * per, vocab), i1 = min(i0 + per, vocab);
  float mx = -INFINITY;
  for (int i = i0; i < i1; ++i) {
    const uint16_t b = row[i];
    if (bf16_key(b) >= thr) mx = fmaxf(mx, __uint_as_float((uint32_t)b << 16));
  }
  mx = block_reduce(mx, red, true);
  const float c = inv_temperature * 1.4426950408889634f;
  float part = 0.f;
  for (int i = i0; i < i1; ++i) {
    const uint16_t b = row[i];
    if (bf16_key(b) >= thr) part += exp2f((__uint_as_float((uint32_t)b << 16) - mx) * c);
  }
  const float total = block_reduce(part, red, false);

  // ---- 3. inverse-CDF draw
  const float target = uniforms[blockIdx.x] * total;
  const int lane = tid & 31, warp = tid >> 5;
  float incl = part;                                  // inclusive scan of the slice sums
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float w = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += w;
  }
  if (lane == 31) warp_sums[warp] = incl;
  if (tid == 0) result = -1;
  __syncthreads();
  float base = 0.f;
  for (int w = 0; w < warp; ++w) base += warp_sums[w];   // same order in every thread: consistent prefix sums
  const float after = base + incl;
  float before = __shfl_up_sync(0xffffffffu, after, 1);   // the neighbour's upper bound: the slices tile [0, total)
  if (lane == 0) before = base;
  if (part > 0.f && before <= target && target < after) {
    float run = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const uint16_t b = row[i];
      if (bf16_key(b) < thr) continue;
      run += exp2f((__uint_as_float((uint32_t)b << 16) - mx) * c);
      pick = i;
      if (target < run) break;
    }
    result = pick;                                    // at most one thread's interval contains the target
  }
  __syncthreads();
  if (result < 0) {
    // the target fell on or past the total through rounding: take the last kept token
    int last = -1;
    for (int i = i1 - 1; i >= i0; --i)
      if (bf16_key(row[i]) >= thr) { last = i; break; }
    if (last >= 0) atomicMax(&result, last);
    __syncthreads();
  }
  if (tid == 0) out[blockIdx.x] = result;
}

}  // namespace b200

using namespace b200;

// logits: (rows, ld) bf16 with `vocab` valid columns; uniforms: (rows) fp32 in [0, 1); out: (rows) int64.
// temperature > 0; top_k <= 0 or >= vocab keeps the whole vocabulary.
extern "C" int b200_sample_topk(const void* logits, long long rows, long long ld, int vocab, const float* uniforms,
                                float temperature, int top_k, long long* out, cudaStream_t st) {
  if (!(temperature > 0.f) || vocab <= 0 || ld < vocab) return -10;
  if (rows == 0) return 0;
  sample_topk_kernel<<<(unsigned)rows, SAMPLE_THREADS, 0, st>>>((const __nv_bfloat16*)logits, ld, vocab, uniforms,
                                                              1.f / temperature, top_k, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
