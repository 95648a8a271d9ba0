// Collectives written as ordinary kernels over NVLink peer memory (every GPU maps every peer's
// communication buffers through CUDA IPC), each fused with the compute that neighbours it:
//
//   peer_barrier          flag exchange, bounded wait
//   peer_allgather        pull: every GPU copies the 7 remote shards into its own buffer
//                         (replaces dist.all_gather, reference fsdp_zero3.py:131-134)
//   peer_reduce_scatter   each GPU sums its slice of all peers' bf16 gradient staging in fp32, applies
//                         the 1/world scale and either stores the fp32 shard gradient (+ its sum of
//                         squares for global clipping) or runs the AdamW update on the fp32 master /
//                         m / v shard and rewrites the bf16 weight shard - the reduced gradient then
//                         never touches HBM (replaces fsdp_zero3.py:172-231 + triton_adamw.py)
//   peer_allreduce        two-shot in place: reduce my chunk from all peers, scale, push it to all
//                         peers (replaces flatten + divide + dist.all_reduce + unflatten, ddp.py:20-24)
//
// Synchronisation is by epoch-numbered flags in peer memory: rank p writes flags[slot][p] on every
// peer with a system-scope release store; waiters poll their local copy with acquire loads.  Every
// wait is bounded: when the limit runs out the kernel records ERR_WAIT_FLAG in the status word and
// returns without touching the data, leaving the context usable.  Loads from peers are plain
// vector loads (no TMA, no multicast).
#include "ptx.cuh"
#include <string.h>

namespace b200 {

constexpr int MAX_WORLD = 16;

struct PeerPtrs {
  void* p[MAX_WORLD];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Wait until flags[i] >= epoch for every i < world (wrap-safe comparison).  One thread polls each flag.
// Returns false when the time limit ran out.
__device__ __forceinline__ bool wait_flags(const uint32_t* flags, int world, uint32_t epoch, uint64_t limit_ns) {
  bool ok = true;
  if (threadIdx.x < world) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > limit_ns) {
        ok = false;
        break;
      }
      __nanosleep(64);
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// rank `rank` announces `epoch` in slot row `flag_row` (an array of `world` words) on every peer.
__device__ __forceinline__ void signal_peers(const PeerPtrs& flag_bases, size_t row_offset, int world, int rank,
                                             uint32_t epoch) {
  if (threadIdx.x < world) {
    __threadfence_system();
    uint32_t* dst = reinterpret_cast<uint32_t*>(flag_bases.p[threadIdx.x]) + row_offset + rank;
    st_release_sys(dst, epoch);
  }
}

__global__ void peer_barrier_kernel(PeerPtrs flag_bases, size_t row_offset, int world, int rank, uint32_t epoch,
                                    uint64_t limit_ns, uint32_t* status) {
  signal_peers(flag_bases, row_offset, world, rank, epoch);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flag_bases.p[rank]) + row_offset;
  if (!wait_flags(mine, world, epoch, limit_ns) && threadIdx.x == 0 && status) atomicCAS(status, 0u, ERR_WAIT_FLAG);
}

// dst[p * n_vec + i] = src_p[i] for every peer p (16-byte vectors); the local shard is copied too.
// A thread keeps WORLD x U loads in flight, one from every peer for U consecutive strides, so that all
// NVLink ports are busy at once and the round-trip latency is covered.
template <int WORLD, int U>
__device__ __forceinline__ void gather_body(const PeerPtrs& src, uint4* __restrict__ dst, size_t n_vec, int rank,
                                            size_t first, size_t stride) {
  size_t i = first;
  for (; i + (U - 1) * stride < n_vec; i += U * stride) {
    uint4 v[WORLD][U];
#pragma unroll
    for (int k = 0; k < WORLD; ++k) {
      const uint4* s = reinterpret_cast<const uint4*>(src.p[(rank + k) % WORLD]);
#pragma unroll
      for (int u = 0; u < U; ++u) v[k][u] = s[i + u * stride];
    }
#pragma unroll
    for (int k = 0; k < WORLD; ++k) {
      uint4* d = dst + (size_t)((rank + k) % WORLD) * n_vec;
#pragma unroll
      for (int u = 0; u < U; ++u) d[i + u * stride] = v[k][u];
    }
  }
  for (; i < n_vec; i += stride)
#pragma unroll
    for (int k = 0; k < WORLD; ++k) {
      const int p = (rank + k) % WORLD;
      dst[(size_t)p * n_vec + i] = reinterpret_cast<const uint4*>(src.p[p])[i];
    }
}

__device__ __forceinline__ void gather_any(const PeerPtrs& src, uint4* __restrict__ dst, size_t n_vec, int world,
                                           int rank, size_t first, size_t stride) {
  switch (world) {
    case 2: gather_body<2, 4>(src, dst, n_vec, rank, first, stride); break;
    case 4: gather_body<4, 2>(src, dst, n_vec, rank, first, stride); break;
    case 8: gather_body<8, 1>(src, dst, n_vec, rank, first, stride); break;
    default:
      for (int k = 0; k < world; ++k) {
        const int p = (rank + k) % world;
        for (size_t i = first; i < n_vec; i += stride) dst[(size_t)p * n_vec + i] = reinterpret_cast<const uint4*>(src.p[p])[i];
      }
  }
}

__global__ void peer_allgather_kernel(PeerPtrs src, uint4* __restrict__ dst, size_t n_vec, int world, int rank) {
  gather_any(src, dst, n_vec, world, rank, blockIdx.x * (size_t)blockDim.x + threadIdx.x,
             (size_t)gridDim.x * blockDim.x);
}

struct AdamArgs {
  float* master;
  float* m;
  float* v;
  __nv_bfloat16* mirror;
  const float* gscale;   // device clip coefficient or null
  float lr, b1, b2, eps, wd, alpha_t;
};

// Per-CTA partial sums of squares of one reduce-scatter launch.  Launches that share the array must be ordered on
// one stream (FSDP issues all of them on its communication stream).
constexpr int RS_MAX_CTAS = 1024;
__device__ float g_rs_sumsq_partials[RS_MAX_CTAS];

// mode 0: grad_out[i] = mean_p staging_p[rank*n + i]  (fp32), sumsq += sum(grad^2) when sumsq != null
// mode 1: the same mean feeds AdamW directly (grad_out may be null)
template <int MODE, int WORLD>
__global__ void __launch_bounds__(512)
peer_reduce_scatter_kernel(PeerPtrs staging, PeerPtrs flag_bases, size_t ready_row, size_t done_row, float* grad_out,
                           float* sumsq, AdamArgs adam, size_t n, int world, int rank, uint32_t epoch,
                           uint64_t limit_ns, uint32_t* counter, uint32_t* status) {
  __shared__ float red[32];
  // "my staging for this unit is complete" (this kernel is stream-ordered after the unit's backward)
  if (blockIdx.x == 0) signal_peers(flag_bases, ready_row, world, rank, epoch);
  const uint32_t* ready = reinterpret_cast<const uint32_t*>(flag_bases.p[rank]) + ready_row;
  if (!wait_flags(ready, world, epoch, limit_ns)) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0u, ERR_WAIT_FLAG | (1u << 8));
    return;
  }
  const float inv = 1.f / (float)world;
  const float gs = (MODE == 1 && adam.gscale) ? *adam.gscale : 1.f;
  const size_t n_vec = n / 8;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  float ss = 0.f;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 in[WORLD > 0 ? WORLD : 1];
    if (WORLD > 0) {                    // all peer loads are issued before the first one is consumed
#pragma unroll
      for (int p = 0; p < WORLD; ++p) in[p] = reinterpret_cast<const uint4*>(staging.p[p])[(size_t)rank * n_vec + i];
    }
#pragma unroll
    for (int p = 0; p < (WORLD > 0 ? WORLD : world); ++p) {   // fixed order: bitwise reproducible
      const uint4 u = WORLD > 0 ? in[p] : reinterpret_cast<const uint4*>(staging.p[p])[(size_t)rank * n_vec + i];
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] *= inv;
    if (MODE == 0) {
      float4* g = reinterpret_cast<float4*>(grad_out) + 2 * i;
      g[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      g[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += acc[k] * acc[k];
    } else {
      float4* pm = reinterpret_cast<float4*>(adam.master) + 2 * i;
      float4* mm = reinterpret_cast<float4*>(adam.m) + 2 * i;
      float4* vv = reinterpret_cast<float4*>(adam.v) + 2 * i;
      float pw[8], mw[8], vw[8];
      *reinterpret_cast<float4*>(pw) = pm[0]; *reinterpret_cast<float4*>(pw + 4) = pm[1];
      *reinterpret_cast<float4*>(mw) = mm[0]; *reinterpret_cast<float4*>(mw + 4) = mm[1];
      *reinterpret_cast<float4*>(vw) = vv[0]; *reinterpret_cast<float4*>(vw + 4) = vv[1];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float g = acc[k] * gs;
        mw[k] = adam.b1 * mw[k] + (1.f - adam.b1) * g;
        vw[k] = adam.b2 * vw[k] + (1.f - adam.b2) * g * g;
        pw[k] -= adam.alpha_t * mw[k] / (sqrtf(vw[k]) + adam.eps);
        pw[k] -= adam.lr * adam.wd * pw[k];
        ss += acc[k] * acc[k];
      }
      pm[0] = *reinterpret_cast<float4*>(pw); pm[1] = *reinterpret_cast<float4*>(pw + 4);
      mm[0] = *reinterpret_cast<float4*>(mw); mm[1] = *reinterpret_cast<float4*>(mw + 4);
      vv[0] = *reinterpret_cast<float4*>(vw); vv[1] = *reinterpret_cast<float4*>(vw + 4);
      if (adam.mirror)
        reinterpret_cast<uint4*>(adam.mirror)[i] = make_uint4(pack_bf16x2(pw[0], pw[1]), pack_bf16x2(pw[2], pw[3]),
                                                             pack_bf16x2(pw[4], pw[5]), pack_bf16x2(pw[6], pw[7]));
      if (grad_out) {
        float4* g = reinterpret_cast<float4*>(grad_out) + 2 * i;
        g[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        g[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    }
  }
  if (sumsq != nullptr) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
      ss = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) g_rs_sumsq_partials[blockIdx.x] = ss;   // added up in block order by the last CTA (below)
    }
  }
  // last CTA to finish tells every peer that this rank no longer reads their staging for this unit
  __syncthreads();
  __shared__ uint32_t last;
  if (threadIdx.x == 0) {
    __threadfence();
    last = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (last) {
    if (threadIdx.x == 0) {
      *counter = 0;
      if (sumsq != nullptr) {   // fixed summation order: the gradient norm is bitwise reproducible
        float t = 0.f;
        for (unsigned b = 0; b < gridDim.x; ++b) t += __ldcg(&g_rs_sumsq_partials[b]);
        *sumsq += t;
      }
    }
    signal_peers(flag_bases, done_row, world, rank, epoch);
  }
}

// Wait for a row of flags (used before a staging buffer is overwritten).
__global__ void peer_wait_kernel(const uint32_t* flags, int world, uint32_t epoch, uint64_t limit_ns, uint32_t* status) {
  if (!wait_flags(flags, world, epoch, limit_ns) && threadIdx.x == 0 && status)
    atomicCAS(status, 0u, ERR_WAIT_FLAG | (2u << 8));
}

// In-place mean all-reduce of fp32 buffers that live at the same offset on every peer.
__global__ void __launch_bounds__(512)
peer_allreduce_kernel(PeerPtrs bufs, PeerPtrs flag_bases, size_t ready_row, size_t done_row, size_t n, int world,
                      int rank, uint32_t epoch, uint64_t limit_ns, uint32_t* counter, uint32_t* status) {
  if (blockIdx.x == 0) signal_peers(flag_bases, ready_row, world, rank, epoch);
  const uint32_t* ready = reinterpret_cast<const uint32_t*>(flag_bases.p[rank]) + ready_row;
  if (!wait_flags(ready, world, epoch, limit_ns)) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0u, ERR_WAIT_FLAG | (3u << 8));
    return;
  }
  const size_t n_vec = n / 4;
  const size_t chunk = (n_vec + world - 1) / world;
  const size_t lo = (size_t)rank * chunk;
  const size_t hi = lo + chunk < n_vec ? lo + chunk : n_vec;
  const float inv = 1.f / (float)world;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = lo + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < hi; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 in[MAX_WORLD];
#pragma unroll
    for (int p = 0; p < MAX_WORLD; ++p)
      if (p < world) in[p] = reinterpret_cast<const float4*>(bufs.p[p])[i];   // all loads in flight together
#pragma unroll
    for (int p = 0; p < MAX_WORLD; ++p) {
      if (p >= world) break;
      const float4 u = in[p];
      acc.x += u.x; acc.y += u.y; acc.z += u.z; acc.w += u.w;
    }
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    for (int k = 0; k < world; ++k) reinterpret_cast<float4*>(bufs.p[(rank + k) % world])[i] = acc;
  }
  __syncthreads();
  __shared__ uint32_t last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (last) {
    if (threadIdx.x == 0) *counter = 0;
    signal_peers(flag_bases, done_row, world, rank, epoch);   // my chunk has been pushed everywhere
    const uint32_t* done = reinterpret_cast<const uint32_t*>(flag_bases.p[rank]) + done_row;
    if (!wait_flags(done, world, epoch, limit_ns) && threadIdx.x == 0 && status)
      atomicCAS(status, 0u, ERR_WAIT_FLAG | (4u << 8));
  }
}

}  // namespace b200

using namespace b200;

static PeerPtrs make_ptrs(const unsigned long long* host_ptrs, int world) {
  PeerPtrs p;
  for (int i = 0; i < MAX_WORLD; ++i) p.p[i] = i < world ? reinterpret_cast<void*>(host_ptrs[i]) : nullptr;
  return p;
}
#define COMM_CHECK() return (cudaGetLastError() == cudaSuccess) ? 0 : -4

// ---- peer memory plumbing (host): plain cudaMalloc regions shared through CUDA IPC handles
extern "C" int b200_ipc_alloc(unsigned long long bytes, unsigned long long* out_ptr) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return -1;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) return -2;
  *out_ptr = reinterpret_cast<unsigned long long>(p);
  return 0;
}
extern "C" int b200_ipc_free(unsigned long long ptr) {
  return cudaFree(reinterpret_cast<void*>(ptr)) == cudaSuccess ? 0 : -1;
}
extern "C" int b200_ipc_get_handle(unsigned long long ptr, unsigned char* out64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr)) != cudaSuccess) return -1;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out64, &h, 64);
  return 0;
}
extern "C" int b200_ipc_open(const unsigned char* in64, unsigned long long* out_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { cudaGetLastError(); return -(int)e; }
  *out_ptr = reinterpret_cast<unsigned long long>(p);
  return 0;
}
extern "C" int b200_ipc_close(unsigned long long ptr) {
  return cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)) == cudaSuccess ? 0 : -1;
}

// ---- launchers.  `flag_bases` / pointer tables are host arrays of `world` device addresses.
extern "C" int b200_peer_barrier(const unsigned long long* flag_bases, unsigned long long row_offset, int world,
                                 int rank, unsigned int epoch, unsigned long long limit_ns, uint32_t* status,
                                 cudaStream_t st) {
  if (world > MAX_WORLD) return -10;
  peer_barrier_kernel<<<1, 32, 0, st>>>(make_ptrs(flag_bases, world), row_offset, world, rank, epoch, limit_ns, status);
  COMM_CHECK();
}

extern "C" int b200_peer_allgather(const unsigned long long* src_ptrs, void* dst, unsigned long long shard_bytes,
                                   int world, int rank, int ctas, cudaStream_t st) {
  if (world > MAX_WORLD || shard_bytes % 16 || (reinterpret_cast<uintptr_t>(dst) & 15)) return -10;
  if (shard_bytes == 0) return 0;
  peer_allgather_kernel<<<ctas > 0 ? ctas : 128, 512, 0, st>>>(make_ptrs(src_ptrs, world), (uint4*)dst, shard_bytes / 16,
                                                               world, rank);
  COMM_CHECK();
}

// mode 0: reduce into grad_out (+ sumsq).  mode 1: fused AdamW on master/m/v/mirror (grad_out, sumsq optional).
extern "C" int b200_peer_reduce_scatter(const unsigned long long* staging_ptrs, const unsigned long long* flag_bases,
                                        unsigned long long ready_row, unsigned long long done_row, float* grad_out,
                                        float* sumsq, unsigned long long n, int world, int rank, unsigned int epoch,
                                        int mode, float* master, float* m, float* v, void* mirror, const float* gscale,
                                        float lr, float b1, float b2, float eps, float wd, float alpha_t,
                                        unsigned long long limit_ns, uint32_t* counter, uint32_t* status, int ctas,
                                        cudaStream_t st) {
  if (world > MAX_WORLD || n % 8) return -10;
  if (mode == 0 && grad_out == nullptr) return -11;
  if (mode == 1 && (master == nullptr || m == nullptr || v == nullptr)) return -11;
  AdamArgs a{master, m, v, (__nv_bfloat16*)mirror, gscale, lr, b1, b2, eps, wd, alpha_t};
  const int grid = ctas > 0 ? (ctas > RS_MAX_CTAS ? RS_MAX_CTAS : ctas) : 96;
#define RS_LAUNCH(MODE_, WORLD_)                                                                                  \
  peer_reduce_scatter_kernel<MODE_, WORLD_><<<grid, 512, 0, st>>>(make_ptrs(staging_ptrs, world),                 \
                                                                  make_ptrs(flag_bases, world), ready_row, done_row, \
                                                                  grad_out, sumsq, a, n, world, rank, epoch, limit_ns, \
                                                                  counter, status)
#define RS_WORLD(MODE_)                        \
  switch (world) {                             \
    case 2: RS_LAUNCH(MODE_, 2); break;        \
    case 4: RS_LAUNCH(MODE_, 4); break;        \
    case 8: RS_LAUNCH(MODE_, 8); break;        \
    default: RS_LAUNCH(MODE_, 0); break;       \
  }
  if (mode == 0) { RS_WORLD(0) } else { RS_WORLD(1) }
#undef RS_WORLD
#undef RS_LAUNCH
  COMM_CHECK();
}

// Plain pull copy (init-time broadcast: every rank reads the source rank's buffer through its peer mapping).
__global__ void __launch_bounds__(512) peer_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                                        size_t n_vec, unsigned char* __restrict__ dst_tail,
                                                        const unsigned char* __restrict__ src_tail, int tail) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_vec; i += stride) dst[i] = src[i];
  if (blockIdx.x == 0 && (int)threadIdx.x < tail) dst_tail[threadIdx.x] = src_tail[threadIdx.x];
}

// dst (local) <- src (any address this process can read, e.g. a peer's IPC-mapped buffer); both 16-byte aligned.
extern "C" int b200_peer_copy(void* dst, const void* src, unsigned long long nbytes, int ctas, cudaStream_t st) {
  if ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) return -10;
  if (nbytes == 0) return 0;
  const size_t n_vec = nbytes / 16;
  const int tail = (int)(nbytes % 16);
  peer_copy_kernel<<<ctas > 0 ? ctas : 128, 512, 0, st>>>(reinterpret_cast<uint4*>(dst), reinterpret_cast<const uint4*>(src),
                                                          n_vec, reinterpret_cast<unsigned char*>(dst) + n_vec * 16,
                                                          reinterpret_cast<const unsigned char*>(src) + n_vec * 16, tail);
  COMM_CHECK();
}

extern "C" int b200_peer_wait(const uint32_t* flags, int world, unsigned int epoch, unsigned long long limit_ns,
                              uint32_t* status, cudaStream_t st) {
  if (world > MAX_WORLD) return -10;
  peer_wait_kernel<<<1, 32, 0, st>>>(flags, world, epoch, limit_ns, status);
  COMM_CHECK();
}

extern "C" int b200_peer_allreduce(const unsigned long long* buf_ptrs, const unsigned long long* flag_bases,
                                   unsigned long long ready_row, unsigned long long done_row, unsigned long long n,
                                   int world, int rank, unsigned int epoch, unsigned long long limit_ns,
                                   uint32_t* counter, uint32_t* status, int ctas, cudaStream_t st) {
  if (world > MAX_WORLD || n % 4) return -10;
  peer_allreduce_kernel<<<ctas > 0 ? ctas : 96, 512, 0, st>>>(make_ptrs(buf_ptrs, world), make_ptrs(flag_bases, world),
                                                              ready_row, done_row, n, world, rank, epoch, limit_ns,
                                                              counter, status);
  COMM_CHECK();
}
