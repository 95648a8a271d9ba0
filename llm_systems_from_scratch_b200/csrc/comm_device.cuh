// Device-side pieces of the peer-memory collectives that more than one kernel uses: the epoch-flag handshake and the
// reduce-scatter (+ scale + sum of squares + optional AdamW) body.  The body runs either as a kernel of its own
// (comm_kernels.cu) or on the two copy warps of every CTA of the CTA-pair GEMM (gemm_tcgen05_2cta.cu), where it
// overlaps the tensor-core work of the same kernel tile by tile.  Peer data is read with plain vector loads: no TMA,
// no multicast.  Every wait is bounded and reports through the status word instead of hanging.
#pragma once
#include "ptx.cuh"

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
// Sum over all GPUs bound to the multicast object of the 16 bytes (8 bf16) at `mc_addr`, added up in fp32 inside the
// switch and returned as 8 bf16.  `mc_addr` must be a multicast address; it is only ever used by this instruction.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const uint4* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

// Barrier among `nthreads` threads of a CTA (a multiple of 32) on hardware barrier `id` (1..15; 0 is __syncthreads).
__device__ __forceinline__ void group_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

struct AdamArgs {
  float* master;
  float* m;
  float* v;
  __nv_bfloat16* mirror;
  const float* gscale;   // device clip coefficient or null
  float lr, b1, b2, eps, wd, alpha_t;
};

// One reduce-scatter of a unit's gradient staging.  Every rank holds `world * n` bf16 values in its own staging
// buffer (peer-mapped: staging.p[r] is rank r's buffer as seen from this GPU); this rank reduces slice `rank`.
//   mode 0: grad_out[i] = mean_r staging_r[rank * n + i] (fp32); *sumsq += sum(grad^2) when sumsq != null
//   mode 1: the same mean feeds the AdamW update of (master, m, v) and the bf16 weight shard; grad_out optional
// Handshake: `ready` row - rank r's staging is complete; `done` row - rank r no longer reads anybody's staging.
struct ReduceTask {
  PeerPtrs staging;
  // Optional NVLS path: the multicast address of this rank's slice of the staging (an NVLink multicast object bound
  // to every rank's staging buffer).  When set, one `multimem.ld_reduce` per 16 bytes lets the NVSwitch read the
  // eight copies and return their sum, instead of eight peer loads per thread.  Null = plain peer loads.
  const uint4* mc_slice;
  PeerPtrs flag_bases;
  unsigned long long ready_row, done_row;   // element offsets of the two flag rows (world words each)
  float* grad_out;
  float* sumsq;
  AdamArgs adam;
  unsigned long long n;     // elements of this rank's slice (multiple of 8); 0 = no task
  int world, rank, mode;
  uint32_t epoch;
  unsigned long long limit_ns;
  uint32_t* counter;        // zero before the launch; the last participating group resets it
  float* partials;          // one float per participating group (fixed-order sum of squares)
  uint32_t* status;
};

// Host description of a reduce-scatter (mirrors ReduceTask; filled by the Python side through ctypes).
struct B200ReduceDesc {
  unsigned long long staging[16];
  unsigned long long mc_staging;       // multicast address of the staging buffer (same offset as staging[]), 0 = none
  unsigned long long flag_bases[16];
  unsigned long long ready_row, done_row;
  float* grad_out;
  float* sumsq;
  float* master;
  float* m;
  float* v;
  void* mirror;
  const float* gscale;
  float lr, b1, b2, eps, wd, alpha_t;
  unsigned long long n;
  int world, rank, mode;
  unsigned int epoch;
  unsigned long long limit_ns;
  uint32_t* counter;
};

// Shared-memory words the body needs (per participating thread group).
struct ReduceSmem {
  float red[32];
  uint32_t flag;
};

// rank `rank` announces `epoch` in a flag row (an array of `world` words at element offset `row`) on every peer.
__device__ __forceinline__ void signal_row(const PeerPtrs& flag_bases, unsigned long long row, int world, int rank,
                                           uint32_t epoch, int tid) {
  if (tid < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flag_bases.p[tid]) + row + rank, epoch);
  }
}

// Thread `tid` < world polls flags[tid] until it reaches `epoch` (wrap-safe) or the limit runs out.  Once the device
// status word is set (some wait of this step has already given up) later waits give up at once: the step is lost
// anyway, and a rank whose peer is gone then unwinds in one limit instead of one limit per collective.
__device__ __forceinline__ bool poll_flag(const uint32_t* flags, int world, uint32_t epoch, unsigned long long limit_ns,
                                          int tid, const uint32_t* status = nullptr) {
  if (tid >= world) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_sys(flags + tid) - epoch) < 0) {
    if ((++spins & 0xff) == 1) {
      if (status != nullptr && *reinterpret_cast<const volatile uint32_t*>(status) != 0) return false;
      if (globaltimer_ns() - t0 > limit_ns) return false;
    }
    __nanosleep(64);
  }
  return true;
}

// The body.  `tid` in [0, nthreads) within the group, `part` in [0, nparts) is the group's index among all
// participating groups of the launch (one group per CTA).  bar_id: hardware barrier reserved for the group.
template <int MODE, int WORLD, int U>
__device__ __forceinline__ void reduce_scatter_body(const ReduceTask& t, int tid, int nthreads, int part, int nparts,
                                                    int bar_id, ReduceSmem* sm) {
  // "my staging for this unit is complete" (this launch is stream-ordered after the unit's backward)
  if (part == 0) signal_row(t.flag_bases, t.ready_row, t.world, t.rank, t.epoch, tid);
  if (tid == 0) sm->flag = 0;
  group_sync(bar_id, nthreads);
  const uint32_t* ready = reinterpret_cast<const uint32_t*>(t.flag_bases.p[t.rank]) + t.ready_row;
  if (!poll_flag(ready, t.world, t.epoch, t.limit_ns, tid, t.status)) sm->flag = 1;
  group_sync(bar_id, nthreads);
  const bool ok = sm->flag == 0;
  float ss = 0.f;
  if (ok) {
    const float inv = 1.f / (float)t.world;
    const float gs = (MODE == 1 && t.adam.gscale) ? *t.adam.gscale : 1.f;
    const size_t n_vec = t.n / 8;
    const size_t stride = (size_t)nparts * nthreads;
    constexpr int NW = WORLD > 0 ? WORLD : 1;
    const int world = WORLD > 0 ? WORLD : t.world;
    // One 16-byte piece of this rank's slice: the `world` copies are summed in rank order (bitwise reproducible) by
    // `consume`, or by the switch on the NVLS path; `apply` scales and stores the gradient or runs the AdamW update.
    // `acc` holds the sum over ranks of 8 consecutive gradient elements: scale, then store or update.
    struct AdamState {
      float pw[8], mw[8], vw[8];
    };
    // The optimizer state of a piece is requested together with the peers' copies of the gradient, not after they
    // have arrived: the two latencies overlap instead of adding up.
    auto load_state = [&](size_t i, AdamState& st) {
      if (MODE == 1) {
        const float4* pm = reinterpret_cast<const float4*>(t.adam.master) + 2 * i;
        const float4* mm = reinterpret_cast<const float4*>(t.adam.m) + 2 * i;
        const float4* vv = reinterpret_cast<const float4*>(t.adam.v) + 2 * i;
        *reinterpret_cast<float4*>(st.pw) = pm[0]; *reinterpret_cast<float4*>(st.pw + 4) = pm[1];
        *reinterpret_cast<float4*>(st.mw) = mm[0]; *reinterpret_cast<float4*>(st.mw + 4) = mm[1];
        *reinterpret_cast<float4*>(st.vw) = vv[0]; *reinterpret_cast<float4*>(st.vw + 4) = vv[1];
      }
    };
    auto apply = [&](size_t i, float (&acc)[8], AdamState& st) {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] *= inv;
      if (MODE == 0) {
        float4* g = reinterpret_cast<float4*>(t.grad_out) + 2 * i;
        g[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        g[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += acc[k] * acc[k];
      } else {
        float4* pm = reinterpret_cast<float4*>(t.adam.master) + 2 * i;
        float4* mm = reinterpret_cast<float4*>(t.adam.m) + 2 * i;
        float4* vv = reinterpret_cast<float4*>(t.adam.v) + 2 * i;
        float (&pw)[8] = st.pw, (&mw)[8] = st.mw, (&vw)[8] = st.vw;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float g = acc[k] * gs;
          mw[k] = t.adam.b1 * mw[k] + (1.f - t.adam.b1) * g;
          vw[k] = t.adam.b2 * vw[k] + (1.f - t.adam.b2) * g * g;
          pw[k] -= t.adam.alpha_t * mw[k] / (sqrtf(vw[k]) + t.adam.eps);
          pw[k] -= t.adam.lr * t.adam.wd * pw[k];
          ss += acc[k] * acc[k];
        }
        pm[0] = *reinterpret_cast<float4*>(pw); pm[1] = *reinterpret_cast<float4*>(pw + 4);
        mm[0] = *reinterpret_cast<float4*>(mw); mm[1] = *reinterpret_cast<float4*>(mw + 4);
        vv[0] = *reinterpret_cast<float4*>(vw); vv[1] = *reinterpret_cast<float4*>(vw + 4);
        if (t.adam.mirror)
          reinterpret_cast<uint4*>(t.adam.mirror)[i] = make_uint4(pack_bf16x2(pw[0], pw[1]), pack_bf16x2(pw[2], pw[3]),
                                                                 pack_bf16x2(pw[4], pw[5]), pack_bf16x2(pw[6], pw[7]));
        if (t.grad_out) {
          float4* g = reinterpret_cast<float4*>(t.grad_out) + 2 * i;
          g[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
          g[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
      }
    };
    auto add8 = [](float (&acc)[8], const uint4& u) {
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    };
    auto consume = [&](size_t i, const uint4 (&in)[NW], AdamState& st) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int p = 0; p < NW; ++p) add8(acc, in[p]);
      if (WORLD == 0)        // world sizes without a specialisation: one peer at a time
        for (int p = 1; p < world; ++p) add8(acc, reinterpret_cast<const uint4*>(t.staging.p[p])[(size_t)t.rank * n_vec + i]);
      apply(i, acc, st);
    };
    // strides in flight per thread: U for the plain reduction; with the AdamW state travelling along (24 more floats
    // per stride) two, or four at two ranks
    constexpr int UA = MODE == 1 ? (U > 2 ? (WORLD == 2 ? 4 : 2) : U) : U;
    // every peer's copy of U consecutive strides is requested before the first one is consumed: WORLD x U 16-byte
    // loads in flight per thread keep all NVLink ports busy and cover the round trip
    size_t i = (size_t)part * nthreads + tid;
    const size_t base = (size_t)t.rank * n_vec;
    if (t.mc_slice != nullptr) {
      // NVLS: the switch adds the copies (fp32 accumulation, bf16 result); 4 reduced pieces in flight per thread
      constexpr int UM = MODE == 1 ? 2 : 4;
      auto from_sum = [&](size_t idx, const uint4& sum, AdamState& st) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        add8(acc, sum);
        apply(idx, acc, st);
      };
      for (; i + (UM - 1) * stride < n_vec; i += UM * stride) {
        uint4 sum[UM];
        AdamState st[UM];
#pragma unroll
        for (int u = 0; u < UM; ++u) sum[u] = multimem_ld_reduce_bf16x8(t.mc_slice + i + u * stride);
#pragma unroll
        for (int u = 0; u < UM; ++u) load_state(i + u * stride, st[u]);
#pragma unroll
        for (int u = 0; u < UM; ++u) from_sum(i + u * stride, sum[u], st[u]);
      }
      for (; i < n_vec; i += stride) {
        AdamState st;
        const uint4 sum = multimem_ld_reduce_bf16x8(t.mc_slice + i);
        load_state(i, st);
        from_sum(i, sum, st);
      }
    } else if (UA > 1) {
      for (; i + (UA - 1) * stride < n_vec; i += UA * stride) {
        uint4 in[UA][NW];
        AdamState st[UA];
#pragma unroll
        for (int u = 0; u < UA; ++u)
#pragma unroll
          for (int p = 0; p < NW; ++p) in[u][p] = reinterpret_cast<const uint4*>(t.staging.p[p])[base + i + u * stride];
#pragma unroll
        for (int u = 0; u < UA; ++u) load_state(i + u * stride, st[u]);
#pragma unroll
        for (int u = 0; u < UA; ++u) consume(i + u * stride, in[u], st[u]);
      }
    }
    for (; i < n_vec; i += stride) {
      uint4 in[NW];
      AdamState st;
#pragma unroll
      for (int p = 0; p < NW; ++p) in[p] = reinterpret_cast<const uint4*>(t.staging.p[p])[base + i];
      load_state(i, st);
      consume(i, in, st);
    }
  } else if (tid == 0 && t.status != nullptr) {
    atomicCAS(t.status, 0u, ERR_WAIT_FLAG | (1u << 8));
  }
  // per-group partial sum of squares, added up in group order by the last group: bitwise reproducible
  if (t.sumsq != nullptr) {
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) sm->red[warp] = ss;
    group_sync(bar_id, nthreads);
    if (warp == 0) {
      ss = lane < (nthreads >> 5) ? sm->red[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) t.partials[part] = ss;
    }
  }
  // the last group to finish tells every peer that this rank no longer reads their staging for this unit; a group
  // whose wait ran out still counts itself, so the counter returns to zero and the next launch starts clean
  group_sync(bar_id, nthreads);
  if (tid == 0) {
    __threadfence();
    sm->flag = (atomicAdd(t.counter, 1u) == (uint32_t)nparts - 1) ? 2u : (ok ? 0u : 1u);
  }
  group_sync(bar_id, nthreads);
  if (sm->flag == 2u) {
    if (tid == 0) {
      *t.counter = 0;
      if (t.sumsq != nullptr) {
        float s = 0.f;
        for (int b = 0; b < nparts; ++b) s += __ldcg(&t.partials[b]);
        *t.sumsq += s;
      }
    }
    signal_row(t.flag_bases, t.done_row, t.world, t.rank, t.epoch, tid);
  }
}

// Loads in flight per thread: 8 x 2 at eight ranks, 4 x 4 at four, 2 x 8 at two (16 pieces of 16 bytes each).
template <int MODE>
__device__ __forceinline__ void reduce_scatter_any(const ReduceTask& t, int tid, int nthreads, int part, int nparts,
                                                   int bar_id, ReduceSmem* sm) {
  switch (t.world) {
    case 2: reduce_scatter_body<MODE, 2, 8>(t, tid, nthreads, part, nparts, bar_id, sm); break;
    case 4: reduce_scatter_body<MODE, 4, 4>(t, tid, nthreads, part, nparts, bar_id, sm); break;
    case 8: reduce_scatter_body<MODE, 8, 2>(t, tid, nthreads, part, nparts, bar_id, sm); break;
    default: reduce_scatter_body<MODE, 0, 1>(t, tid, nthreads, part, nparts, bar_id, sm); break;
  }
}

}  // namespace b200
