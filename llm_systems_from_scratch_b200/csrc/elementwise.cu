// Bandwidth-bound kernels of the training step, written for sm_100a: every kernel moves 16 bytes per
// thread per access, keeps reductions in fp32, and never synchronises with the host.
//
//   rmsnorm_fwd / rmsnorm_bwd    (reference: llm-systems/llm_systems/kernels/triton_rms_norm.py:30-149)
//   silu_mul_fwd / silu_mul_bwd  (reference: llm-systems/llm_systems/kernels/triton_swiglu.py:27-86)
//   rope (interleaved pairs)     (reference: llm-core/llm_core/model.py:93-104)
//   embedding gather / scatter   (reference: llm-core/llm_core/model.py:48-49)
//   cross-entropy fwd + in-place grad (reference: llm-systems/llm_systems/kernels/triton_cross_entropy.py:22-85)
//   flat AdamW with bf16 mirror  (reference: llm-systems/llm_systems/kernels/triton_adamw.py:40-101)
//   sum of squares / clip coefficient / scale / casts
#include "ptx.cuh"

namespace b200 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blockDim.x <= 1024; every thread receives the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(p) =
      make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ void load8f(const float* p, float (&f)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// ------------------------------------------------------------------------ RMSNorm fwd
// One warp per row; the row is read twice (the second read hits L1/L2).
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                          int rows, int d, float eps) {
  pdl_sync();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + (size_t)row * d;
  float ss = 0.f;
  for (int c = lane * 8; c < d; c += 256) {
    float f[8];
    load8(xr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)d + eps);
  if (lane == 0 && rstd != nullptr) rstd[row] = r;
  __nv_bfloat16* yr = y + (size_t)row * d;
  for (int c = lane * 8; c < d; c += 256) {
    float f[8], g[8];
    load8(xr + c, f);
    load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * r * g[i];
    store8(yr + c, f);
  }
}

// Persistent variant for d = NC * 256: a warp walks rows warp, warp + n_warps, ... with the whole row in
// registers (read once) and the next row's loads issued before the current row is reduced, so a warp always has
// a row in flight; the grid is a few blocks per SM instead of one short-lived block per eight rows.
__device__ __forceinline__ uint4 ld_stream16(const __nv_bfloat16* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

template <int NC>
__global__ void __launch_bounds__(256, 2) rmsnorm_fwd_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ y,
                                                               float* __restrict__ rstd, int rows, float eps) {
  pdl_sync();
  constexpr int D = NC * 256;
  const int lane = threadIdx.x & 31;
  const int n_warps = gridDim.x * (blockDim.x >> 5);
  int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  uint4 cur[NC], nxt[NC];
  if (row < rows) {
#pragma unroll
    for (int j = 0; j < NC; ++j) cur[j] = ld_stream16(x + (size_t)row * D + j * 256 + lane * 8);
  }
  for (; row < rows; row += n_warps) {
    const int nrow = row + n_warps;
    if (nrow < rows) {
#pragma unroll
      for (int j = 0; j < NC; ++j) nxt[j] = ld_stream16(x + (size_t)nrow * D + j * 256 + lane * 8);
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      float f[8];
      unpack8(cur[j], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)D + eps);
    if (lane == 0 && rstd != nullptr) rstd[row] = r;
    __nv_bfloat16* yr = y + (size_t)row * D;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      float f[8], g[8];
      unpack8(cur[j], f);
      load8(w + j * 256 + lane * 8, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * r * g[i];
      store8(yr + j * 256 + lane * 8, f);
    }
#pragma unroll
    for (int j = 0; j < NC; ++j) cur[j] = nxt[j];
  }
}

// ------------------------------------------------------------------------ RMSNorm bwd
// dx = [dres +] rstd * (dy*w) - rstd^3/d * sum(dy*w*x) * x ;  dw += dy * x * rstd.
// Each block walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; a thread owns up to MAXC groups of
// 8 columns and keeps the weight-gradient partial for them in registers.  Partials go to
// `dw_partial` (gridDim.x, d) fp32 and are summed in a fixed order by rmsnorm_dw_reduce_kernel.
constexpr int RMS_BWD_THREADS = 256;
constexpr int RMS_BWD_MAXC_LIMIT = 4;  // d <= 256 * 8 * 4 = 8192

// RMS_BWD_MAXC is a template parameter so that narrow rows (d <= 2048 needs one group per thread) use
// few registers and several blocks fit on an SM; with the widest instance only one block fits.
template <int RMS_BWD_MAXC>
__global__ void __launch_bounds__(RMS_BWD_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int d) {
  __shared__ float red[32];
  float wreg[RMS_BWD_MAXC][8];
  float dwacc[RMS_BWD_MAXC][8];
#pragma unroll
  for (int j = 0; j < RMS_BWD_MAXC; ++j) {
    const int c = (j * RMS_BWD_THREADS + threadIdx.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
    if (c < d) load8(w + c, wreg[j]);
  }
  // The next row's dy, x and residual gradient are requested before the current row's block-wide reduction, so
  // the memory system always has a row per block in flight.
  uint4 cdy[RMS_BWD_MAXC], cx[RMS_BWD_MAXC], ce[RMS_BWD_MAXC];
  uint4 ndy[RMS_BWD_MAXC], nx[RMS_BWD_MAXC], ne[RMS_BWD_MAXC];
  auto request = [&](int row, uint4 (&qdy)[RMS_BWD_MAXC], uint4 (&qx)[RMS_BWD_MAXC], uint4 (&qe)[RMS_BWD_MAXC]) {
#pragma unroll
    for (int j = 0; j < RMS_BWD_MAXC; ++j) {
      const int c = (j * RMS_BWD_THREADS + threadIdx.x) * 8;
      if (c < d) {
        qdy[j] = ld_stream16(dy + (size_t)row * d + c);
        qx[j] = ld_stream16(x + (size_t)row * d + c);
        if (dres != nullptr) qe[j] = ld_stream16(dres + (size_t)row * d + c);
      }
    }
  };
  int row = blockIdx.x;
  float r = 0.f, rn = 0.f;
  if (row < rows) {
    request(row, cdy, cx, ce);
    r = rstd[row];
  }
  for (; row < rows; row += gridDim.x) {
    const int nrow = row + gridDim.x;
    if (nrow < rows) {
      request(nrow, ndy, nx, ne);
      rn = rstd[nrow];
    }
    float g[RMS_BWD_MAXC][8], xv[RMS_BWD_MAXC][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < RMS_BWD_MAXC; ++j) {
      const int c = (j * RMS_BWD_THREADS + threadIdx.x) * 8;
      if (c < d) {
        float dyv[8];
        unpack8(cdy[j], dyv);
        unpack8(cx[j], xv[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dwacc[j][i] += dyv[i] * xv[j][i] * r;
          g[j][i] = dyv[i] * wreg[j][i];
          dot += g[j][i] * xv[j][i];
        }
      }
    }
    dot = block_sum(dot, red);
    const float coef = r * r * r * dot / (float)d;
    __nv_bfloat16* dxr = dx + (size_t)row * d;
#pragma unroll
    for (int j = 0; j < RMS_BWD_MAXC; ++j) {
      const int c = (j * RMS_BWD_THREADS + threadIdx.x) * 8;
      if (c < d) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = r * g[j][i] - coef * xv[j][i];
        if (dres != nullptr) {  // gradient arriving through the residual branch
          float ev[8];
          unpack8(ce[j], ev);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += ev[i];
        }
        store8(dxr + c, o);
      }
    }
#pragma unroll
    for (int j = 0; j < RMS_BWD_MAXC; ++j) {
      cdy[j] = ndy[j];
      cx[j] = nx[j];
      ce[j] = ne[j];
    }
    r = rn;
  }
  float* part = dw_partial + (size_t)blockIdx.x * d;
#pragma unroll
  for (int j = 0; j < RMS_BWD_MAXC; ++j) {
    const int c = (j * RMS_BWD_THREADS + threadIdx.x) * 8;
    if (c < d) {
      *reinterpret_cast<float4*>(part + c) = make_float4(dwacc[j][0], dwacc[j][1], dwacc[j][2], dwacc[j][3]);
      *reinterpret_cast<float4*>(part + c + 4) = make_float4(dwacc[j][4], dwacc[j][5], dwacc[j][6], dwacc[j][7]);
    }
  }
}

// Variant for d = NC * 256 and enough rows to fill the GPU: one warp per row, no block-wide barrier inside the row
// loop.  A lane owns 8 * NC columns; a row's dy, x and residual gradient (3 * NC 16-byte loads per lane) are all
// requested before the first is used, and with eight independent warps per SM a row's latency is covered by the
// other warps.  The weight-gradient partial of a lane's columns stays in registers over all rows of the warp; at the
// end the eight warps of a block add theirs in warp order through shared memory, so a launch leaves gridDim.x
// partial rows (148 instead of 592) for rmsnorm_dw_reduce_kernel.
template <int NC>
__global__ void __launch_bounds__(256, 1)
rmsnorm_bwd_rows_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                        const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                        float* __restrict__ dw_partial, int rows) {
  constexpr int D = NC * 256;
  __shared__ float dw_s[D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = gridDim.x * 8;
  // the weight row (4 KB at most) is re-read from L1 where it is used: keeping it in registers as well would spill
  const __nv_bfloat16* wl = w + lane * 8;
  float dwacc[NC][8];
#pragma unroll
  for (int j = 0; j < NC; ++j) {
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
  }
  for (int row = blockIdx.x * 8 + warp; row < rows; row += n_warps) {
    const size_t base = (size_t)row * D + lane * 8;
    uint4 qdy[NC], qx[NC], qe[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      qdy[j] = ld_stream16(dy + base + j * 256);
      qx[j] = ld_stream16(x + base + j * 256);
      if (dres != nullptr) qe[j] = ld_stream16(dres + base + j * 256);
    }
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      float dyv[8], xv[8], wv[8];
      unpack8(qdy[j], dyv);
      unpack8(qx[j], xv);
      load8(wl + j * 256, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dwacc[j][i] += dyv[i] * xv[i] * r;
        dot += dyv[i] * wv[i] * xv[i];
      }
    }
    dot = warp_sum(dot);
    const float coef = r * r * r * dot / (float)D;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      float dyv[8], xv[8], wv[8], o[8];
      unpack8(qdy[j], dyv);
      unpack8(qx[j], xv);
      load8(wl + j * 256, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = r * (dyv[i] * wv[i]) - coef * xv[i];
      if (dres != nullptr) {
        float ev[8];
        unpack8(qe[j], ev);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += ev[i];
      }
      store8(dx + base + j * 256, o);
    }
  }
  // block partial: warps add in warp order (fixed), one barrier per warp
  for (int wi = 0; wi < 8; ++wi) {
    if (warp == wi) {
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        float* dst = dw_s + j * 256 + lane * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = (wi == 0) ? dwacc[j][i] : dst[i] + dwacc[j][i];
      }
    }
    __syncthreads();
  }
  float* part = dw_partial + (size_t)blockIdx.x * D;
  for (int c = threadIdx.x * 4; c < D; c += 256 * 4)
    *reinterpret_cast<float4*>(part + c) = *reinterpret_cast<const float4*>(dw_s + c);
}

// dw[c] (=|+=) sum_p partial[p][c], fixed summation order => bitwise reproducible.
// A block of 1024 threads owns 32 columns: thread (g, x) sums partial rows g, g+32, ... of column x (four
// independent loads in flight at a time), then the 32 row groups are combined in a fixed order through shared
// memory.  With 592 partial rows a thread adds 18 or 19 of them, so the kernel takes a few microseconds.
constexpr int RMS_DW_GROUPS = 32;
__global__ void __launch_bounds__(32 * RMS_DW_GROUPS)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nparts, int d, int accumulate) {
  __shared__ float sm[RMS_DW_GROUPS][33];
  const int x = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + x;
  float s = 0.f;
  if (c < d) {
    int p = g;
    for (; p + 3 * RMS_DW_GROUPS < nparts; p += 4 * RMS_DW_GROUPS) {
      const float a0 = partial[(size_t)p * d + c];
      const float a1 = partial[(size_t)(p + RMS_DW_GROUPS) * d + c];
      const float a2 = partial[(size_t)(p + 2 * RMS_DW_GROUPS) * d + c];
      const float a3 = partial[(size_t)(p + 3 * RMS_DW_GROUPS) * d + c];
      s += a0; s += a1; s += a2; s += a3;
    }
    for (; p < nparts; p += RMS_DW_GROUPS) s += partial[(size_t)p * d + c];
  }
  sm[g][x] = s;
  __syncthreads();
  if (g == 0 && c < d) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < RMS_DW_GROUPS; ++k) t += sm[k][x];
    dw[c] = accumulate ? dw[c] + t : t;
  }
}

// --------------------------------------------------------------------------- SwiGLU
// gu is (rows, 2F): gate columns [0,F), up columns [F,2F).
__global__ void silu_mul_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h,
                                    long long rows, int F) {
  pdl_sync();
  const long long groups = rows * (F / 8);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < groups;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / (F / 8);
    const int c = (int)(i - row * (F / 8)) * 8;
    float g[8], u[8], o[8];
    load8(gu + row * 2 * F + c, g);
    load8(gu + row * 2 * F + F + c, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    store8(h + row * F + c, o);
  }
}

__global__ void silu_mul_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gu,
                                    __nv_bfloat16* __restrict__ dgu, long long rows, int F) {
  const long long groups = rows * (F / 8);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < groups;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / (F / 8);
    const int c = (int)(i - row * (F / 8)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + row * 2 * F + c, g);
    load8(gu + row * 2 * F + F + c, u);
    load8(dh + row * F + c, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = 1.f / (1.f + __expf(-g[k]));
      const float silu = g[k] * s;
      dg[k] = d[k] * u[k] * (s + silu * (1.f - s));
      du[k] = d[k] * silu;
    }
    store8(dgu + row * 2 * F + c, dg);
    store8(dgu + row * 2 * F + F + c, du);
  }
}

// ----------------------------------------------------------------------------- RoPE
// In-place rotation of the Q and K thirds of qkv (rows, 3*d), d = H*dh.  cos_sin is (2, ctx, dh/2) fp32.
// Position of a row: positions[row] when given, else row % seq.  sign = -1 applies the inverse rotation.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_sin,
                            const int* __restrict__ positions, long long rows, int seq, int d, int dh, int ctx,
                            float sign) {
  pdl_sync();
  const int gpr = 2 * d / 8;  // groups of 8 elements per row over the Q and K parts
  const long long groups = rows * gpr;
  const float* cosb = cos_sin;
  const float* sinb = cos_sin + (size_t)ctx * (dh / 2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < groups;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / gpr;
    const int c = (int)(i - row * gpr) * 8;  // column within [0, 2d)
    const int pos = positions ? positions[row] : (int)(row % seq);
    const int e = c % dh;                    // element offset inside the head (multiple of 8)
    float v[8];
    __nv_bfloat16* p = qkv + row * 3 * d + c;
    load8(p, v);
    const float4 cs = *reinterpret_cast<const float4*>(cosb + (size_t)pos * (dh / 2) + e / 2);
    const float4 sn = *reinterpret_cast<const float4*>(sinb + (size_t)pos * (dh / 2) + e / 2);
    const float cc[4] = {cs.x, cs.y, cs.z, cs.w};
    const float ss[4] = {sn.x * sign, sn.y * sign, sn.z * sign, sn.w * sign};
    float o[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      o[2 * k] = cc[k] * v[2 * k] - ss[k] * v[2 * k + 1];
      o[2 * k + 1] = ss[k] * v[2 * k] + cc[k] * v[2 * k + 1];
    }
    store8(p, o);
  }
}

// ------------------------------------------------------------------------ Embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long rows, int d, int vocab) {
  pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  long long t = tokens[row];
  if (t < 0 || t >= vocab) t = 0;  // out-of-range ids are clamped rather than read out of bounds
  const __nv_bfloat16* src = table + (size_t)t * d;
  __nv_bfloat16* dst = out + (size_t)row * d;
  for (int c = lane * 8; c < d; c += 256) *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
}

// grad_table (V, d) fp32 += dx rows; one warp per token row, 16-byte vector reductions.
__global__ void embedding_bwd_kernel(const long long* __restrict__ tokens, const __nv_bfloat16* __restrict__ dx,
                                     float* __restrict__ grad_table, long long rows, int d, int vocab) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const long long t = tokens[row];
  if (t < 0 || t >= vocab) return;
  const __nv_bfloat16* src = dx + (size_t)row * d;
  float* dst = grad_table + (size_t)t * d;
  for (int c = lane * 8; c < d; c += 256) {
    float f[8];
    load8(src + c, f);
    atomicAdd(reinterpret_cast<float4*>(dst + c), make_float4(f[0], f[1], f[2], f[3]));
    atomicAdd(reinterpret_cast<float4*>(dst + c + 4), make_float4(f[4], f[5], f[6], f[7]));
  }
}

// Deterministic variant: `order` lists the token rows sorted by token id (stable), `sorted_tokens` the ids in that
// order.  The warp at the first position of every run of equal ids adds the run's dx rows in order in fp32
// registers and writes (or accumulates into) the table row once: no atomics, bitwise reproducible.
// OUT = float: the fp32 gradient table; OUT = __nv_bfloat16: a bf16 staging table (multi-GPU gradient staging),
// written once per row from the fp32 sum of the run (accumulate is not offered there).
template <int CHUNKS, typename OUT>   // 256-column chunks per launch: columns [col0, col0 + 256 * CHUNKS) of every row
__global__ void embedding_bwd_sorted_kernel(const long long* __restrict__ sorted_tokens,
                                            const long long* __restrict__ order,
                                            const __nv_bfloat16* __restrict__ dx, OUT* __restrict__ grad_table,
                                            long long rows, int d, int vocab, int accumulate, int col0) {
  const int lane = threadIdx.x & 31;
  const long long j0 = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (j0 >= rows) return;
  const long long t = sorted_tokens[j0];
  if (t < 0 || t >= vocab) return;
  if (j0 > 0 && sorted_tokens[j0 - 1] == t) return;   // not the head of its run
  float acc[CHUNKS][8];
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[k][e] = 0.f;
  for (long long j = j0; j < rows && sorted_tokens[j] == t; ++j) {
    const __nv_bfloat16* src = dx + (size_t)order[j] * d;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = col0 + lane * 8 + k * 256;
      if (c < d) {
        float f[8];
        load8(src + c, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[k][e] += f[e];
      }
    }
  }
  OUT* dst = grad_table + (size_t)t * d;
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    const int c = col0 + lane * 8 + k * 256;
    if (c < d) {
      if constexpr (sizeof(OUT) == 2) {
        *reinterpret_cast<uint4*>(dst + c) = make_uint4(pack_bf16x2(acc[k][0], acc[k][1]), pack_bf16x2(acc[k][2], acc[k][3]),
                                                        pack_bf16x2(acc[k][4], acc[k][5]), pack_bf16x2(acc[k][6], acc[k][7]));
        continue;
      }
      float4* o = reinterpret_cast<float4*>(dst + c);
      float4 a = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
      float4 b = make_float4(acc[k][4], acc[k][5], acc[k][6], acc[k][7]);
      if (accumulate) {
        const float4 pa = o[0], pb = o[1];
        a.x += pa.x; a.y += pa.y; a.z += pa.z; a.w += pa.w;
        b.x += pb.x; b.y += pb.y; b.z += pb.z; b.w += pb.w;
      }
      o[0] = a;
      o[1] = b;
    }
  }
}

// -------------------------------------------------------------------- Cross entropy
// One block per row of logits (rows, ld) bf16 with `vocab` valid columns.  Pass 1: online max / sum.
// Pass 2: overwrite the row with (softmax - onehot) * grad_scale / n_valid.  Row losses go to
// `row_loss` (fp32); `n_valid` is a device float computed by count_valid_kernel (no host sync).
constexpr int XENT_THREADS = 512;

__global__ void count_valid_kernel(const long long* __restrict__ targets, long long rows, int ignore_index,
                                   float* __restrict__ n_valid) {
  __shared__ float red[32];
  float c = 0.f;
  for (long long i = threadIdx.x; i < rows; i += blockDim.x) c += (targets[i] != ignore_index) ? 1.f : 0.f;
  c = block_sum(c, red);
  if (threadIdx.x == 0) *n_valid = fmaxf(c, 1.f);
}

__global__ void __launch_bounds__(XENT_THREADS)
xent_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ row_loss,
            const float* __restrict__ n_valid, long long ld, int vocab, int ignore_index, float grad_scale,
            int write_grad) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long tgt = targets[row];
  const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= vocab;
  const int nvec = vocab / 8;
  float m = -INFINITY, s = 0.f;
  for (int g = threadIdx.x; g < nvec; g += XENT_THREADS) {
    float f[8];
    load8(lr + g * 8, f);
    float lm = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) lm = fmaxf(lm, f[i]);
    const float nm = fmaxf(m, lm);
    float add = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) add += __expf(f[i] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  for (int c = nvec * 8 + threadIdx.x; c < vocab; c += XENT_THREADS) {
    const float f = __bfloat162float(lr[c]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  const float lse = gm + logf(gs);
  const float nv = *n_valid;
  if (threadIdx.x == 0) row_loss[row] = ignored ? 0.f : (lse - __bfloat162float(lr[tgt])) / nv;
  if (!write_grad) return;
  __syncthreads();  // the target logit has been read before anyone overwrites it
  const float k = ignored ? 0.f : grad_scale / nv;
  for (int g = threadIdx.x; g < nvec; g += XENT_THREADS) {
    float f[8];
    load8(lr + g * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = g * 8 + i;
      f[i] = (__expf(f[i] - lse) - ((c == tgt) ? 1.f : 0.f)) * k;
    }
    store8(lr + g * 8, f);
  }
  for (int c = nvec * 8 + threadIdx.x; c < vocab; c += XENT_THREADS)   // columns past `vocab` are never touched
    lr[c] = __float2bfloat16((__expf(__bfloat162float(lr[c]) - lse) - ((c == tgt) ? 1.f : 0.f)) * k);
}

// loss (=|+=) sum(row_loss) in a fixed order (single block).
__global__ void sum_rows_kernel(const float* __restrict__ v, long long n, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) s += v[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) *out = accumulate ? *out + s : s;
}

// argmax over the first `vocab` columns of each row of bf16 logits; ties -> lowest index.
__global__ void argmax_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int vocab,
                              long long* __restrict__ out) {
  pdl_sync();
  __shared__ float sv[32];
  __shared__ int si[32];
  const __nv_bfloat16* lr = logits + (long long)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
    const float f = __bfloat162float(lr[c]);
    if (f > best || (f == best && c < bi)) { best = f; bi = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = bi;
  }
}

// ---------------------------------------------------------------------------- AdamW
// One pass over flat fp32 state: 4 B grad (or 2 B bf16) + 12 B state in, 12 B state + 2 B mirror out.
//   m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 ; p -= alpha_t m / (sqrt(v)+eps) ; p -= lr wd p
// `gscale` (device float, may be null) is multiplied into g: the clip coefficient stays on the device.
template <typename GradT>
__global__ void adamw_kernel(float* __restrict__ p, const GradT* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ mirror, long long n,
                             const float* __restrict__ gscale, float lr, float b1, float b2, float eps, float wd,
                             float alpha_t) {
  const float gs = gscale ? *gscale : 1.f;
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float gg[4];
    if constexpr (sizeof(GradT) == 4) {
      float4 t = reinterpret_cast<const float4*>(g)[i];
      gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
    } else {
      uint2 t = reinterpret_cast<const uint2*>(g)[i];
      float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y);
      gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
    }
    float pp[4] = {pv.x, pv.y, pv.z, pv.w}, mm[4] = {mv.x, mv.y, mv.z, mv.w}, vq[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = gg[k] * gs;
      mm[k] = b1 * mm[k] + (1.f - b1) * gk;
      vq[k] = b2 * vq[k] + (1.f - b2) * gk * gk;
      pp[k] -= alpha_t * mm[k] / (sqrtf(vq[k]) + eps);
      pp[k] -= lr * wd * pp[k];
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vq[0], vq[1], vq[2], vq[3]);
    if (mirror) reinterpret_cast<uint2*>(mirror)[i] = make_uint2(pack_bf16x2(pp[0], pp[1]), pack_bf16x2(pp[2], pp[3]));
  }
  // tail (n % 4 elements)
  const long long tail0 = nvec * 4;
  const long long t = tail0 + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < n) {
    float gk;
    if constexpr (sizeof(GradT) == 4) gk = g[t] * gs; else gk = __bfloat162float(g[t]) * gs;
    float mk = b1 * m[t] + (1.f - b1) * gk;
    float vk = b2 * v[t] + (1.f - b2) * gk * gk;
    float pk = p[t] - alpha_t * mk / (sqrtf(vk) + eps);
    pk -= lr * wd * pk;
    p[t] = pk; m[t] = mk; v[t] = vk;
    if (mirror) mirror[t] = __float2bfloat16(pk);
  }
}

// Deterministic two-step variant: per-block partials to `partials[blockIdx.x]`, then one block adds them in index
// order (fixed summation order => bitwise reproducible gradient norm).
template <typename T>
__global__ void sumsq_partials_kernel(const T* __restrict__ x, long long n, float* __restrict__ partials) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 4) f = x[i]; else f = __bfloat162float(x[i]);
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

__global__ void sumsq_finish_kernel(const float* __restrict__ partials, int n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];   // fixed assignment of partials to threads
  s = block_sum(s, red);
  if (threadIdx.x == 0) *out += s;
}

// out += sum(x^2).  fp32 or bf16 input.  Per-block partials are combined with one atomic per block.
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 4) f = x[i]; else f = __bfloat162float(x[i]);
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// coef = min(1, max_norm / (sqrt(sumsq) + 1e-6)); also stores the norm.
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float* __restrict__ coef,
                                 float* __restrict__ norm_out) {
  const float nrm = sqrtf(*sumsq);
  if (norm_out) *norm_out = nrm;
  *coef = fminf(1.f, max_norm / (nrm + 1e-6f));
}

template <typename T>
__global__ void scale_kernel(T* __restrict__ x, long long n, const float* __restrict__ coef) {
  // 16-byte accesses over the aligned body, scalar head and tail
  const float c = *coef;
  constexpr int V = 16 / sizeof(T);
  const long long head = min(n, (long long)(((16 - (reinterpret_cast<uintptr_t>(x) & 15)) & 15) / sizeof(T)));
  const long long nvec = (n - head) / V;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  uint4* xv = reinterpret_cast<uint4*>(x + head);
  for (long long i = tid; i < nvec; i += nth) {
    uint4 v = xv[i];
    if constexpr (sizeof(T) == 4) {
      v.x = __float_as_uint(__uint_as_float(v.x) * c); v.y = __float_as_uint(__uint_as_float(v.y) * c);
      v.z = __float_as_uint(__uint_as_float(v.z) * c); v.w = __float_as_uint(__uint_as_float(v.w) * c);
    } else {
      float2 f;
      f = unpack_bf16x2(v.x); v.x = pack_bf16x2(f.x * c, f.y * c);
      f = unpack_bf16x2(v.y); v.y = pack_bf16x2(f.x * c, f.y * c);
      f = unpack_bf16x2(v.z); v.z = pack_bf16x2(f.x * c, f.y * c);
      f = unpack_bf16x2(v.w); v.w = pack_bf16x2(f.x * c, f.y * c);
    }
    xv[i] = v;
  }
  const long long rest = n - head - nvec * V;
  if (tid < head + rest) {
    const long long i = tid < head ? tid : head + nvec * V + (tid - head);
    if constexpr (sizeof(T) == 4) x[i] = x[i] * c; else x[i] = __float2bfloat16(__bfloat162float(x[i]) * c);
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 v = reinterpret_cast<const float4*>(src)[i];
    reinterpret_cast<uint2*>(dst)[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
  const long long t = nvec * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < n) dst[t] = __float2bfloat16(src[t]);
}

__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __bfloat162float(src[i]);
}

static int grid_for(long long work_items, int threads, int max_blocks = 148 * 16) {
  long long b = (work_items + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return (int)b;
}

}  // namespace b200

using namespace b200;
#define CHECK_LAUNCH() return (cudaGetLastError() == cudaSuccess) ? 0 : -4
#define ALIGNED16(p) ((reinterpret_cast<uintptr_t>(p) & 15) == 0)

namespace b200 {
int g_pdl_enabled = 0;
}
// 1 = kernels of the decode path (norm, GEMM, rotary embedding, KV append, paged attention, SiLU, embedding, argmax)
// are launched as programmatic dependents of the kernel before them; returns the previous setting.
extern "C" int b200_set_pdl(int on) {
  const int old = b200::g_pdl_enabled;
  b200::g_pdl_enabled = on ? 1 : 0;
  return old;
}

static int g_rmsnorm_fwd_rows = 1;
// 0: the general-width kernel (a block per row); 1: one warp per row where the width allows it
static int g_rmsnorm_bwd_rows = 1;
extern "C" int b200_rmsnorm_set_bwd_rows(int variant) {
  const int old = g_rmsnorm_bwd_rows;
  g_rmsnorm_bwd_rows = variant;
  return old;
}

// 0 = always the one-block-per-eight-rows kernel (kept for A/B timing and as the general-width path)
extern "C" void b200_rmsnorm_set_fwd_rows(int on) { g_rmsnorm_fwd_rows = on; }

extern "C" int b200_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int d, float eps,
                                cudaStream_t st) {
  if (d % 8 || !ALIGNED16(x) || !ALIGNED16(w) || !ALIGNED16(y)) return -10;
  if (rows == 0) return 0;
  // widths that are a multiple of 256 up to 2048 with enough rows to fill the GPU: the row-pipelined kernel
  const int nc = d / 256;
  if (g_rmsnorm_fwd_rows && d % 256 == 0 && nc <= 8 && rows >= 148 * 8 * 2 * 2) {
    const int grid = 148 * 2;      // two resident blocks per SM at the widest instance (128 registers)
#define RMS_FWD_ROWS(NC)                                                                                  \
  case NC:                                                                                                \
    launch_dep(rmsnorm_fwd_rows_kernel<NC>, grid, 256, 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, \
               (__nv_bfloat16*)y, rstd, rows, eps);                                                       \
    break
    switch (nc) {
      RMS_FWD_ROWS(1); RMS_FWD_ROWS(2); RMS_FWD_ROWS(3); RMS_FWD_ROWS(4);
      RMS_FWD_ROWS(5); RMS_FWD_ROWS(6); RMS_FWD_ROWS(7); RMS_FWD_ROWS(8);
    }
#undef RMS_FWD_ROWS
    CHECK_LAUNCH();
  }
  launch_dep(rmsnorm_fwd_kernel, (rows + 7) / 8, 256, 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
             (__nv_bfloat16*)y, rstd, rows, d, eps);
  CHECK_LAUNCH();
}

// Number of partial rows rmsnorm_bwd needs in its scratch buffer for a given row count.
extern "C" int b200_rmsnorm_bwd_parts(int rows) { return rows < 148 * 4 ? (rows > 0 ? rows : 1) : 148 * 4; }

// dw_partial: scratch of b200_rmsnorm_bwd_parts(rows) * d floats.  dw (d floats) is overwritten or accumulated.
// dres (bf16, same shape as dx, may be null) is added to dx.
extern "C" int b200_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                void* dx, float* dw, float* dw_partial, int rows, int d, int accumulate_dw,
                                cudaStream_t st) {
  if (d % 8 || d > RMS_BWD_THREADS * 8 * RMS_BWD_MAXC_LIMIT) return -10;
  if (!ALIGNED16(dy) || !ALIGNED16(x) || !ALIGNED16(w) || !ALIGNED16(dx) || !ALIGNED16(dw_partial) ||
      !ALIGNED16(dres))
    return -10;
  if (rows == 0) return 0;
  const int nc = d / 256;
  if (g_rmsnorm_bwd_rows && d % 256 == 0 && nc <= 8 && rows >= 148 * 8) {
    const int parts = 148;        // <= b200_rmsnorm_bwd_parts(rows) partial rows of the scratch are used
#define RMS_BWD_ROWS(NC)                                                                                     \
  case NC:                                                                                                   \
    rmsnorm_bwd_rows_kernel<NC><<<parts, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,    \
                                                       (const __nv_bfloat16*)w, rstd,                        \
                                                       (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx,       \
                                                       dw_partial, rows);                                    \
    break
    switch (nc) {
      RMS_BWD_ROWS(1); RMS_BWD_ROWS(2); RMS_BWD_ROWS(3); RMS_BWD_ROWS(4);
      RMS_BWD_ROWS(5); RMS_BWD_ROWS(6); RMS_BWD_ROWS(7); RMS_BWD_ROWS(8);
    }
#undef RMS_BWD_ROWS
    rmsnorm_dw_reduce_kernel<<<(d + 31) / 32, 32 * RMS_DW_GROUPS, 0, st>>>(dw_partial, dw, parts, d, accumulate_dw);
    CHECK_LAUNCH();
  }
  const int parts = b200_rmsnorm_bwd_parts(rows);
#define RMS_BWD_LAUNCH(C)                                                                                   \
  rmsnorm_bwd_kernel<C><<<parts, RMS_BWD_THREADS, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, \
                                                           (const __nv_bfloat16*)w, rstd,                     \
                                                           (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx,    \
                                                           dw_partial, rows, d)
  if (d <= 2048) RMS_BWD_LAUNCH(1);
  else if (d <= 4096) RMS_BWD_LAUNCH(2);
  else RMS_BWD_LAUNCH(4);
#undef RMS_BWD_LAUNCH
  rmsnorm_dw_reduce_kernel<<<(d + 31) / 32, 32 * RMS_DW_GROUPS, 0, st>>>(dw_partial, dw, parts, d, accumulate_dw);
  CHECK_LAUNCH();
}

extern "C" int b200_silu_mul_fwd(const void* gu, void* h, long long rows, int F, cudaStream_t st) {
  if (F % 8 || !ALIGNED16(gu) || !ALIGNED16(h)) return -10;
  if (rows == 0) return 0;
  launch_dep(silu_mul_fwd_kernel, grid_for(rows * (F / 8), 256), 256, 0, st, (const __nv_bfloat16*)gu, (__nv_bfloat16*)h,
             rows, F);
  CHECK_LAUNCH();
}

extern "C" int b200_silu_mul_bwd(const void* dh, const void* gu, void* dgu, long long rows, int F, cudaStream_t st) {
  if (F % 8 || !ALIGNED16(gu) || !ALIGNED16(dh) || !ALIGNED16(dgu)) return -10;
  if (rows == 0) return 0;
  silu_mul_bwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)dh, (const __nv_bfloat16*)gu,
                                                                     (__nv_bfloat16*)dgu, rows, F);
  CHECK_LAUNCH();
}

extern "C" int b200_rope(void* qkv, const float* cos_sin, const int* positions, long long rows, int seq, int d, int dh,
                         int ctx, int inverse, cudaStream_t st) {
  if (dh % 8 || d % dh || !ALIGNED16(qkv) || !ALIGNED16(cos_sin) || seq <= 0) return -10;
  if (positions == nullptr && seq > ctx) return -11;
  if (rows == 0) return 0;
  launch_dep(rope_kernel, grid_for(rows * (2 * d / 8), 256), 256, 0, st, (__nv_bfloat16*)qkv, cos_sin, positions, rows,
             seq, d, dh, ctx, inverse ? -1.f : 1.f);
  CHECK_LAUNCH();
}

extern "C" int b200_embedding_fwd(const long long* tokens, const void* table, void* out, long long rows, int d,
                                  int vocab, cudaStream_t st) {
  if (d % 8 || !ALIGNED16(table) || !ALIGNED16(out)) return -10;
  if (rows == 0) return 0;
  launch_dep(embedding_fwd_kernel, (unsigned)((rows + 7) / 8), 256, 0, st, tokens, (const __nv_bfloat16*)table,
             (__nv_bfloat16*)out, rows, d, vocab);
  CHECK_LAUNCH();
}

extern "C" int b200_embedding_bwd(const long long* tokens, const void* dx, float* grad_table, long long rows, int d,
                                  int vocab, cudaStream_t st) {
  if (d % 8 || !ALIGNED16(dx) || !ALIGNED16(grad_table)) return -10;
  if (rows == 0) return 0;
  embedding_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(tokens, (const __nv_bfloat16*)dx, grad_table, rows, d,
                                                                   vocab);
  CHECK_LAUNCH();
}

// Deterministic embedding backward.  sorted_tokens / order: the token ids sorted ascending (stable) and the row
// index of each; the table rows of tokens that occur are overwritten (accumulate = 0: the caller zeroes the rest)
// or added to (accumulate = 1).  d must be a multiple of 8.
extern "C" int b200_embedding_bwd_sorted(const long long* sorted_tokens, const long long* order, const void* dx,
                                         float* grad_table, long long rows, int d, int vocab, int accumulate,
                                         cudaStream_t st) {
  if (d % 8 || !ALIGNED16(dx) || !ALIGNED16(grad_table)) return -10;
  if (rows == 0) return 0;
  const unsigned grid = (unsigned)((rows + 7) / 8);
#define EMB_LAUNCH(C_, COL0_)                                                                                    \
  embedding_bwd_sorted_kernel<C_, float><<<grid, 256, 0, st>>>(sorted_tokens, order, (const __nv_bfloat16*)dx,        \
                                                              grad_table, rows, d, vocab, accumulate, COL0_)
  if (d <= 1024) EMB_LAUNCH(4, 0);
  else if (d <= 2048) EMB_LAUNCH(8, 0);
  else
    for (int col0 = 0; col0 < d; col0 += 4096) EMB_LAUNCH(16, col0);   // wide rows: one launch per 4096 columns
#undef EMB_LAUNCH
  CHECK_LAUNCH();
}

// The same with a bf16 table (gradient staging that a reduce-scatter reads): rows of tokens that occur are
// overwritten with the rounded fp32 sum of their run; the caller zeroes the table first.
extern "C" int b200_embedding_bwd_sorted_bf16(const long long* sorted_tokens, const long long* order, const void* dx,
                                              void* grad_table, long long rows, int d, int vocab, cudaStream_t st) {
  if (d % 8 || !ALIGNED16(dx) || !ALIGNED16(grad_table)) return -10;
  if (rows == 0) return 0;
  const unsigned grid = (unsigned)((rows + 7) / 8);
#define EMB_LAUNCH(C_, COL0_)                                                                                          \
  embedding_bwd_sorted_kernel<C_, __nv_bfloat16><<<grid, 256, 0, st>>>(sorted_tokens, order, (const __nv_bfloat16*)dx, \
                                                                      (__nv_bfloat16*)grad_table, rows, d, vocab, 0, COL0_)
  if (d <= 1024) EMB_LAUNCH(4, 0);
  else if (d <= 2048) EMB_LAUNCH(8, 0);
  else
    for (int col0 = 0; col0 < d; col0 += 4096) EMB_LAUNCH(16, col0);
#undef EMB_LAUNCH
  CHECK_LAUNCH();
}

// scratch: rows + 1 floats (row losses, then n_valid).  loss (device float) is overwritten or accumulated.
// n_valid_in (device float, may be null): normalise by this count instead of the number of non-ignored
// targets among these rows, so that a caller processing the rows in chunks gets the global mean directly.
extern "C" int b200_xent(void* logits, const long long* targets, float* loss, float* scratch, long long rows,
                         long long ld, int vocab, int ignore_index, float grad_scale, int write_grad,
                         int accumulate_loss, const float* n_valid_in, cudaStream_t st) {
  if (!ALIGNED16(logits) || ld % 8 || vocab > ld) return -10;
  if (rows == 0) return 0;
  const float* n_valid = n_valid_in;
  if (n_valid == nullptr) {
    count_valid_kernel<<<1, 1024, 0, st>>>(targets, rows, ignore_index, scratch + rows);
    n_valid = scratch + rows;
  }
  xent_kernel<<<(unsigned)rows, XENT_THREADS, 0, st>>>((__nv_bfloat16*)logits, targets, scratch, n_valid, ld, vocab,
                                                       ignore_index, grad_scale, write_grad);
  sum_rows_kernel<<<1, 1024, 0, st>>>(scratch, rows, loss, accumulate_loss);
  CHECK_LAUNCH();
}

extern "C" int b200_argmax(const void* logits, long long rows, long long ld, int vocab, long long* out, cudaStream_t st) {
  if (rows == 0) return 0;
  launch_dep(argmax_kernel, (unsigned)rows, 256, 0, st, (const __nv_bfloat16*)logits, ld, vocab, out);
  CHECK_LAUNCH();
}

extern "C" int b200_adamw(float* p, const void* g, int grad_is_bf16, float* m, float* v, void* mirror, long long n,
                          const float* gscale, float lr, float b1, float b2, float eps, float wd, float alpha_t,
                          cudaStream_t st) {
  if (!ALIGNED16(p) || !ALIGNED16(g) || !ALIGNED16(m) || !ALIGNED16(v) || (mirror && (reinterpret_cast<uintptr_t>(mirror) & 7)))
    return -10;
  if (n == 0) return 0;
  const int grid = grid_for(n / 4 + 4, 256, 148 * 8);
  if (grad_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, (const __nv_bfloat16*)g, m, v, (__nv_bfloat16*)mirror, n, gscale,
                                                      lr, b1, b2, eps, wd, alpha_t);
  else
    adamw_kernel<float><<<grid, 256, 0, st>>>(p, (const float*)g, m, v, (__nv_bfloat16*)mirror, n, gscale, lr, b1, b2, eps,
                                              wd, alpha_t);
  CHECK_LAUNCH();
}

// Number of floats of scratch that b200_sumsq_det needs.
extern "C" int b200_sumsq_scratch() { return 148 * 4; }

// out += sum(x^2) with a fixed summation order (scratch: b200_sumsq_scratch() floats, used only by this call's stream).
extern "C" int b200_sumsq_det(const void* x, int is_bf16, long long n, float* out, float* scratch, cudaStream_t st) {
  if (n == 0) return 0;
  if (scratch == nullptr) return -10;
  const int grid = grid_for(n, 512, 148 * 4);
  if (is_bf16) sumsq_partials_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>((const __nv_bfloat16*)x, n, scratch);
  else sumsq_partials_kernel<float><<<grid, 512, 0, st>>>((const float*)x, n, scratch);
  sumsq_finish_kernel<<<1, 256, 0, st>>>(scratch, grid, out);
  CHECK_LAUNCH();
}

extern "C" int b200_sumsq(const void* x, int is_bf16, long long n, float* out, cudaStream_t st) {
  if (n == 0) return 0;
  const int grid = grid_for(n, 512, 148 * 4);
  if (is_bf16) sumsq_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>((const __nv_bfloat16*)x, n, out);
  else sumsq_kernel<float><<<grid, 512, 0, st>>>((const float*)x, n, out);
  CHECK_LAUNCH();
}

extern "C" int b200_clip_coef(const float* sumsq, float max_norm, float* coef, float* norm_out, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(sumsq, max_norm, coef, norm_out);
  CHECK_LAUNCH();
}

extern "C" int b200_scale(void* x, int is_bf16, long long n, const float* coef, cudaStream_t st) {
  if (n == 0) return 0;
  const int grid = grid_for(n, 256, 148 * 8);
  if (is_bf16) scale_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)x, n, coef);
  else scale_kernel<float><<<grid, 256, 0, st>>>((float*)x, n, coef);
  CHECK_LAUNCH();
}

extern "C" int b200_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t st) {
  if (!ALIGNED16(src) || (reinterpret_cast<uintptr_t>(dst) & 7)) return -10;
  if (n == 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n / 4 + 4, 256, 148 * 8), 256, 0, st>>>(src, (__nv_bfloat16*)dst, n);
  CHECK_LAUNCH();
}

extern "C" int b200_cast_bf16_f32(const void* src, float* dst, long long n, cudaStream_t st) {
  if (n == 0) return 0;
  cast_bf16_to_f32_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, st>>>((const __nv_bfloat16*)src, dst, n);
  CHECK_LAUNCH();
}

// ------------------------------------------------------------------ allocation-free RMSNorm backward
#include "no_alloc.h"

namespace b200 {
// Weight-gradient partials for b200_rmsnorm_bwd_noalloc.  In host code this name is only a stand-in:
// the device address is obtained with cudaGetSymbolAddress below and passed to the kernels.
static __device__ __align__(256) float g_noalloc_dw_partials[B200_NOALLOC_MAX_PARTS * B200_NOALLOC_MAX_D];

constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};

// Resolve (once per device, with that device current) where the scratch array lives on this GPU.
static float* noalloc_scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return nullptr;
  if (g_noalloc_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_noalloc_dw_partials) != cudaSuccess) return nullptr;
    g_noalloc_ptr[dev] = ptr;
  }
  return g_noalloc_ptr[dev];
}
}  // namespace b200

extern "C" int b200_rmsnorm_bwd_noalloc_max_d(void) { return B200_NOALLOC_MAX_D; }

extern "C" int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                        const void* dres, void* dx, float* dw, int rows, int d, int accumulate_dw,
                                        cudaStream_t st) {
  if (d > B200_NOALLOC_MAX_D) return B200_ERR_NOALLOC_TOO_LARGE;
  if (d <= 0 || d % 8 || rows < 0) return -10;
  if (dw == nullptr || (reinterpret_cast<uintptr_t>(dw) & 3)) return -10;
  if (rows > 0 && (dy == nullptr || x == nullptr || w == nullptr || rstd == nullptr || dx == nullptr)) return -10;
  if (!ALIGNED16(dy) || !ALIGNED16(x) || !ALIGNED16(w) || !ALIGNED16(dx) || !ALIGNED16(dres) ||
      (reinterpret_cast<uintptr_t>(rstd) & 3))
    return -10;
  float* scratch = noalloc_scratch_for_current_device();
  if (scratch == nullptr) return B200_ERR_NOALLOC_SETUP;
  if (rows == 0) {
    // no rows: the weight gradient of this call is zero (dw is cleared, or left as it is when accumulating)
    rmsnorm_dw_reduce_kernel<<<(d + 31) / 32, 32 * RMS_DW_GROUPS, 0, st>>>(scratch, dw, 0, d, accumulate_dw);
    CHECK_LAUNCH();
  }
  const int parts = rows < B200_NOALLOC_MAX_PARTS ? rows : B200_NOALLOC_MAX_PARTS;
  // Every partial row [0, parts) x [0, d) is written by the first kernel before the second reads it,
  // so nothing in the shared array has to be cleared between calls.
  rmsnorm_bwd_kernel<RMS_BWD_MAXC_LIMIT><<<parts, RMS_BWD_THREADS, 0, st>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
      (__nv_bfloat16*)dx, scratch, rows, d);
  rmsnorm_dw_reduce_kernel<<<(d + 31) / 32, 32 * RMS_DW_GROUPS, 0, st>>>(scratch, dw, parts, d, accumulate_dw);
  CHECK_LAUNCH();
}
