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
#include "comm_device.cuh"
#include <string.h>

namespace b200 {

// Block-wide forms of the flag helpers (all threads of the CTA call them).
__device__ __forceinline__ bool wait_flags(const uint32_t* flags, int world, uint32_t epoch, uint64_t limit_ns,
                                           const uint32_t* status = nullptr) {
  const bool ok = poll_flag(flags, world, epoch, limit_ns, threadIdx.x, status);
  return __syncthreads_and(ok ? 1 : 0) != 0;
}
__device__ __forceinline__ void signal_peers(const PeerPtrs& flag_bases, size_t row_offset, int world, int rank,
                                             uint32_t epoch) {
  signal_row(flag_bases, row_offset, world, rank, epoch, threadIdx.x);
}

__global__ void peer_barrier_kernel(PeerPtrs flag_bases, size_t row_offset, int world, int rank, uint32_t epoch,
                                    uint64_t limit_ns, uint32_t* status) {
  signal_peers(flag_bases, row_offset, world, rank, epoch);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flag_bases.p[rank]) + row_offset;
  if (!wait_flags(mine, world, epoch, limit_ns, status) && threadIdx.x == 0 && status) atomicCAS(status, 0u, ERR_WAIT_FLAG);
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

// Per-group partial sums of squares of one reduce-scatter launch.  Launches that share an array must be ordered
// on one stream: stand-alone launches (FSDP issues them on its communication stream) use the first array,
// reduce-scatters carried by a GEMM (compute stream) the second.
constexpr int RS_MAX_CTAS = 1024;
__device__ float g_rs_sumsq_partials[2][RS_MAX_CTAS];

// The AdamW variant keeps the optimizer state of two strides in registers next to the peers' copies: 256 threads
// per CTA (and twice the CTAs) give it the registers for that without spilling.
template <int MODE>
__global__ void __launch_bounds__(MODE == 1 ? 256 : 512) peer_reduce_scatter_kernel(const ReduceTask t) {
  __shared__ ReduceSmem sm;
  reduce_scatter_any<MODE>(t, threadIdx.x, blockDim.x, blockIdx.x, gridDim.x, 1, &sm);
}

// Rank `rank` publishes `epoch` in one flag row on every peer and returns (no wait).
__global__ void peer_signal_kernel(PeerPtrs flag_bases, size_t row_offset, int world, int rank, uint32_t epoch) {
  signal_peers(flag_bases, row_offset, world, rank, epoch);
}

// Wait for a row of flags (used before a staging buffer is overwritten).
__global__ void peer_wait_kernel(const uint32_t* flags, int world, uint32_t epoch, uint64_t limit_ns, uint32_t* status) {
  if (!wait_flags(flags, world, epoch, limit_ns, status) && threadIdx.x == 0 && status)
    atomicCAS(status, 0u, ERR_WAIT_FLAG | (2u << 8));
}

// In-place mean all-reduce of fp32 buffers that live at the same offset on every peer.
__global__ void __launch_bounds__(512)
peer_allreduce_kernel(PeerPtrs bufs, PeerPtrs flag_bases, size_t ready_row, size_t done_row, size_t n, int world,
                      int rank, uint32_t epoch, uint64_t limit_ns, uint32_t* counter, uint32_t* status) {
  if (blockIdx.x == 0) signal_peers(flag_bases, ready_row, world, rank, epoch);
  const uint32_t* ready = reinterpret_cast<const uint32_t*>(flag_bases.p[rank]) + ready_row;
  // A CTA whose wait ran out reports, skips the data and still takes part in the CTA count below, so that the
  // counter is back at zero for the next launch.
  const bool ok = wait_flags(ready, world, epoch, limit_ns, status);
  if (!ok && threadIdx.x == 0 && status) atomicCAS(status, 0u, ERR_WAIT_FLAG | (3u << 8));
  const size_t n_vec = ok ? n / 4 : 0;
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
    if (!wait_flags(done, world, epoch, limit_ns, status) && threadIdx.x == 0 && status)
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

float* b200_rs_partials(int which) {
  float* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rs_sumsq_partials) != cudaSuccess) return nullptr;
  return p + (which ? RS_MAX_CTAS : 0);
}

extern "C" int b200_peer_signal(const unsigned long long* flag_bases, unsigned long long row_offset, int world,
                                int rank, unsigned int epoch, cudaStream_t st) {
  if (world > MAX_WORLD) return -10;
  peer_signal_kernel<<<1, 32, 0, st>>>(make_ptrs(flag_bases, world), row_offset, world, rank, epoch);
  COMM_CHECK();
}

// Validates a description and turns it into the device-side task.  `carried`: the task will run on the copy warps
// of a GEMM (it then uses the second array of partial sums).
int b200_make_reduce_task(const B200ReduceDesc* d, uint32_t* status, bool carried, ReduceTask* out) {
  if (d->world > MAX_WORLD || d->world < 1 || d->n % 8 || d->counter == nullptr) return -10;
  if (d->mode == 0 && d->grad_out == nullptr) return -11;
  if (d->mode == 1 && (d->master == nullptr || d->m == nullptr || d->v == nullptr)) return -11;
  ReduceTask t;
  t.staging = make_ptrs(d->staging, d->world);
  // the multicast address covers the same buffer; this rank's slice starts rank * n elements in
  t.mc_slice = d->mc_staging
                   ? reinterpret_cast<const uint4*>(d->mc_staging + (unsigned long long)d->rank * d->n * 2ull)
                   : nullptr;
  if (d->mc_staging & 15) return -10;
  t.flag_bases = make_ptrs(d->flag_bases, d->world);
  t.ready_row = d->ready_row; t.done_row = d->done_row;
  t.grad_out = d->grad_out; t.sumsq = d->sumsq;
  t.adam = AdamArgs{d->master, d->m, d->v, (__nv_bfloat16*)d->mirror, d->gscale, d->lr, d->b1, d->b2, d->eps, d->wd,
                    d->alpha_t};
  t.n = d->n; t.world = d->world; t.rank = d->rank; t.mode = d->mode; t.epoch = d->epoch;
  t.limit_ns = d->limit_ns; t.counter = d->counter; t.status = status;
  t.partials = b200_rs_partials(carried ? 1 : 0);
  if (t.partials == nullptr) return -12;
  *out = t;
  return 0;
}

// Stand-alone launch.  mode 0: reduce into grad_out (+ sumsq).  mode 1: fused AdamW on master/m/v/mirror.
extern "C" int b200_peer_reduce_scatter_desc(const B200ReduceDesc* d, uint32_t* status, int ctas, cudaStream_t st) {
  ReduceTask t;
  const int rc = b200_make_reduce_task(d, status, false, &t);
  if (rc) return rc;
  const int grid = ctas > 0 ? (ctas > RS_MAX_CTAS ? RS_MAX_CTAS : ctas) : 96;
  if (d->mode == 0) peer_reduce_scatter_kernel<0><<<grid, 512, 0, st>>>(t);
  else peer_reduce_scatter_kernel<1><<<(2 * grid > RS_MAX_CTAS ? RS_MAX_CTAS : 2 * grid), 256, 0, st>>>(t);
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
