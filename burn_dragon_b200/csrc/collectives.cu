// In-kernel NVLink collectives over symmetric memory (every rank holds a mapping of every other
// rank's buffer, plus - when the fabric supports it - one NVSwitch multicast address).
//
//   allreduce_scale      grad <- scale * sum_ranks grad        (data-parallel gradient reduction)
//   rs_adamw_ag          reduce-scatter of gradients fused with the AdamW update of the locally
//                        owned shard and the all-gather of the refreshed bf16 parameters
//
// Both are two-shot: rank r reduces slice r (peer loads, or one multimem.ld_reduce through the
// switch) and writes its result to every rank (peer stores, or one multimem.st). The reference has
// no multi-device path at all (src/bin/train.rs:395 is single-device), so nothing here has a
// counterpart there.
//
// Cross-rank ordering uses flag words in a symmetric flag buffer, one slot per (CTA, peer). Values
// only grow (the host passes a new epoch each call). Every wait is bounded by BDH_WAIT_LIMIT_NS;
// a wait that runs out writes STATUS_TIMEOUT_PEER_FLAG to the status word and the kernel returns.
#include "bdh_kernels.h"
#include "flag_protocol.h"
#include "sm100_ptx.cuh"

namespace bdh {

constexpr int COLL_MAX_RANKS = 8;
constexpr int COLL_THREADS = 512;

struct CollPeers {
  void* buf[COLL_MAX_RANKS];        // peer mappings of the data buffer
  uint32_t* flags[COLL_MAX_RANKS];  // peer mappings of the flag buffer
  void* mc;                         // multicast mapping of the data buffer (nullptr: peer loads/stores)
  int rank, world;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier between the CTAs with the same blockIdx on every rank. Slot layout of a rank's flag
// buffer: flags[cta * world + writer]. Returns false on timeout.
__device__ bool cta_barrier_all_ranks(const CollPeers& p, uint32_t value, int* status) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  __threadfence_system();
  if (threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    st_release_sys(p.flags[peer] + flag_slot(blockIdx.x, p.world, p.rank), value);
    const uint32_t* mine = p.flags[p.rank] + flag_slot(blockIdx.x, p.world, peer);
    const uint64_t t0 = global_timer_ns();
    uint32_t it = 0;
    while (!flag_reached(ld_acquire_sys(mine), value)) {
      if ((++it & 255u) == 0 && global_timer_ns() - t0 > BDH_WAIT_LIMIT_NS) {
        atomicCAS(status, STATUS_OK, STATUS_TIMEOUT_PEER_FLAG);
        failed = 1;
        break;
      }
    }
  }
  __syncthreads();
  return failed == 0;
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f32x4(void* mc_addr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x),
               "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_st_b32x4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

// Sum of float4 element i over all ranks' buffers.
__device__ __forceinline__ float4 reduce_f32x4(const CollPeers& p, long long i) {
  if (p.mc) return multimem_ld_reduce_f32x4(static_cast<const float4*>(p.mc) + i);
  float4 v[COLL_MAX_RANKS];
#pragma unroll
  for (int r = 0; r < COLL_MAX_RANKS; ++r)
    if (r < p.world) v[r] = static_cast<const float4*>(p.buf[r])[i];
  float4 s = v[0];
#pragma unroll
  for (int r = 1; r < COLL_MAX_RANKS; ++r)
    if (r < p.world) {
      s.x += v[r].x; s.y += v[r].y; s.z += v[r].z; s.w += v[r].w;
    }
  return s;
}

// n4 = number of float4 elements (the buffer is padded to a multiple of 4 * world floats).
__global__ void __launch_bounds__(COLL_THREADS)
allreduce_scale_kernel(CollPeers p, long long n4, float scale, uint32_t epoch, int* status) {
  if (!cta_barrier_all_ranks(p, flag_value(epoch, 1), status)) return;
  const long long per = n4 / p.world;
  const long long lo = per * p.rank;
  const long long hi = (p.rank == p.world - 1) ? n4 : lo + per;
  for (long long i = lo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 s = reduce_f32x4(p, i);
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    if (p.mc) {
      multimem_st_f32x4(static_cast<float4*>(p.mc) + i, s);
    } else {
#pragma unroll
      for (int r = 0; r < COLL_MAX_RANKS; ++r)
        if (r < p.world) static_cast<float4*>(p.buf[r])[i] = s;
    }
  }
  cta_barrier_all_ranks(p, flag_value(epoch, 2), status);
}

struct AdamArgs {
  float lr, b1, b2, eps, wd, bc1, bc2, gscale;
};

// Gradient buffer `p` (fp32, symmetric). Parameter shadow `q` (bf16, symmetric). master / m / v
// hold only this rank's slice [lo, hi) (indexed from 0).
__global__ void __launch_bounds__(COLL_THREADS)
rs_adamw_ag_kernel(CollPeers p, CollPeers q, float* master, float* m, float* v, long long n4, AdamArgs a,
                   uint32_t epoch, int* status) {
  if (!cta_barrier_all_ranks(p, flag_value(epoch, 1), status)) return;
  const long long per = n4 / p.world;
  const long long lo = per * p.rank;
  const long long hi = (p.rank == p.world - 1) ? n4 : lo + per;
  for (long long i = lo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 g = reduce_f32x4(p, i);
    const long long j = i - lo;
    float4 w = reinterpret_cast<float4*>(master)[j];
    float4 mm = reinterpret_cast<float4*>(m)[j];
    float4 vv = reinterpret_cast<float4*>(v)[j];
    float* gp = &g.x; float* wp = &w.x; float* mp = &mm.x; float* vp = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float gk = gp[k] * a.gscale;
      mp[k] = a.b1 * mp[k] + (1.f - a.b1) * gk;
      vp[k] = a.b2 * vp[k] + (1.f - a.b2) * gk * gk;
      wp[k] = wp[k] * (1.f - a.lr * a.wd) - a.lr * (mp[k] / a.bc1) / (sqrtf(vp[k] / a.bc2) + a.eps);
    }
    reinterpret_cast<float4*>(master)[j] = w;
    reinterpret_cast<float4*>(m)[j] = mm;
    reinterpret_cast<float4*>(v)[j] = vv;
    // refreshed bf16 parameters go to every rank (4 values = 8 bytes)
    uint2 u;
    u.x = pack_bf16x2(w.x, w.y);
    u.y = pack_bf16x2(w.z, w.w);
#pragma unroll
    for (int r = 0; r < COLL_MAX_RANKS; ++r)
      if (r < q.world) static_cast<uint2*>(q.buf[r])[i] = u;
  }
  cta_barrier_all_ranks(p, flag_value(epoch, 2), status);
}

// Fully sharded update: this rank's gradient accumulator `gacc` (fp32, the 1/world slice every rank's
// weight-gradient epilogues added into over NVLink) feeds AdamW on the matching slices of master / m / v,
// the refreshed bf16 parameters go to every rank's working copy, and the accumulator is cleared for the
// next step. The slice is a list of segments (one per sharded parameter): segment s covers local elements
// [seg_lo[s], seg_lo[s+1]) and lands at bf16 element seg_dst[s] of the working copy. The barrier in front
// makes every rank's additions visible, the one behind makes every rank's parameter stores complete.
struct ShardSegs {
  long long lo4[5];     // local float4 offsets of the segments (n + 1 entries)
  long long dst4[4];    // destination offset in the working copy, in units of 4 bf16
  int n;
};

__global__ void __launch_bounds__(COLL_THREADS)
shard_adamw_ag_kernel(CollPeers f, CollPeers q, float* gacc, float* master, float* m, float* v, ShardSegs segs,
                      AdamArgs a, uint32_t epoch, int* status) {
  if (!cta_barrier_all_ranks(f, flag_value(epoch, 1), status)) return;
  const long long n4 = segs.lo4[segs.n];
  for (long long j = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; j < n4;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    int sgi = 0;
#pragma unroll
    for (int k = 1; k < 4; ++k)
      if (k < segs.n && j >= segs.lo4[k]) sgi = k;
    float4 g = reinterpret_cast<float4*>(gacc)[j];
    reinterpret_cast<float4*>(gacc)[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 w = reinterpret_cast<float4*>(master)[j];
    float4 mm = reinterpret_cast<float4*>(m)[j];
    float4 vv = reinterpret_cast<float4*>(v)[j];
    float* gp = &g.x; float* wp = &w.x; float* mp = &mm.x; float* vp = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float gk = gp[k] * a.gscale;
      mp[k] = a.b1 * mp[k] + (1.f - a.b1) * gk;
      vp[k] = a.b2 * vp[k] + (1.f - a.b2) * gk * gk;
      wp[k] = wp[k] * (1.f - a.lr * a.wd) - a.lr * (mp[k] / a.bc1) / (sqrtf(vp[k] / a.bc2) + a.eps);
    }
    reinterpret_cast<float4*>(master)[j] = w;
    reinterpret_cast<float4*>(m)[j] = mm;
    reinterpret_cast<float4*>(v)[j] = vv;
    uint2 u;
    u.x = pack_bf16x2(w.x, w.y);
    u.y = pack_bf16x2(w.z, w.w);
    const long long dst = segs.dst4[sgi] + (j - segs.lo4[sgi]);
#pragma unroll
    for (int r = 0; r < COLL_MAX_RANKS; ++r)
      if (r < q.world) static_cast<uint2*>(q.buf[r])[dst] = u;
  }
  cta_barrier_all_ranks(f, flag_value(epoch, 2), status);
}

// Data-parallel counterpart of the fully sharded update: the gradient slice this rank owns (`gacc`, complete
// once every rank's weight-gradient epilogues have added into it) is scaled and sent to its place in EVERY
// rank's full gradient buffer (one multimem.st through the switch, or one store per peer), then cleared. The
// reduce-scatter half of the gradient all-reduce has then happened inside the backward pass, tile by tile;
// this kernel is the all-gather half, fused with the 1/world scale.
__global__ void __launch_bounds__(COLL_THREADS)
shard_bcast_kernel(CollPeers f, CollPeers q, float* gacc, ShardSegs segs, float scale, uint32_t epoch, int* status) {
  if (!cta_barrier_all_ranks(f, flag_value(epoch, 1), status)) return;
  const long long n4 = segs.lo4[segs.n];
  for (long long j = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; j < n4;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    int sgi = 0;
#pragma unroll
    for (int k = 1; k < 4; ++k)
      if (k < segs.n && j >= segs.lo4[k]) sgi = k;
    float4 g = reinterpret_cast<float4*>(gacc)[j];
    reinterpret_cast<float4*>(gacc)[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    g.x *= scale; g.y *= scale; g.z *= scale; g.w *= scale;
    const long long dst = segs.dst4[sgi] + (j - segs.lo4[sgi]);
    if (q.mc) {
      multimem_st_f32x4(static_cast<float4*>(q.mc) + dst, g);
    } else {
#pragma unroll
      for (int r = 0; r < COLL_MAX_RANKS; ++r)
        if (r < q.world) static_cast<float4*>(q.buf[r])[dst] = g;
    }
  }
  cta_barrier_all_ranks(f, flag_value(epoch, 2), status);
}

// Second half of a reduce-scatter done by GEMM epilogues (EPI_F_PEER_RS): slot s of this rank's
// buffer `p` holds rank s's partial sums for the block of rows this rank owns (per4 float4 each).
// The owner adds the slots up (local reads, fixed order: the result does not depend on timing) and
// sends its block to position rank*per4 of every rank's output buffer `q`: as fp32, or rounded to
// bf16 (half the NVLink bytes, and the consumer's conversion pass disappears). One multimem.st
// through the switch when the output has a multicast mapping, else one store per peer.
template <bool OUT_BF16>
__global__ void __launch_bounds__(COLL_THREADS)
gather_blocks_kernel(CollPeers p, CollPeers q, long long per4, uint32_t epoch, int* status) {
  if (!cta_barrier_all_ranks(p, flag_value(epoch, 1), status)) return;
  const float4* src = static_cast<const float4*>(p.buf[p.rank]);
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nth = static_cast<long long>(gridDim.x) * blockDim.x;
  auto slot_sum = [&](long long j) {
    float4 v[COLL_MAX_RANKS];
#pragma unroll
    for (int r = 0; r < COLL_MAX_RANKS; ++r)
      if (r < p.world) v[r] = __ldcs(src + r * per4 + j);
    float4 s = v[0];
#pragma unroll
    for (int r = 1; r < COLL_MAX_RANKS; ++r)
      if (r < p.world) {
        s.x += v[r].x; s.y += v[r].y; s.z += v[r].z; s.w += v[r].w;
      }
    return s;
  };
  if constexpr (OUT_BF16) {
    // two float4 -> 8 bf16 = one 16-byte store (per4 is even: the host checks)
    const long long base = p.rank * (per4 / 2);
    for (long long i = tid; i < per4 / 2; i += nth) {
      const float4 a = slot_sum(2 * i), b = slot_sum(2 * i + 1);
      uint4 u;
      u.x = pack_bf16x2(a.x, a.y); u.y = pack_bf16x2(a.z, a.w);
      u.z = pack_bf16x2(b.x, b.y); u.w = pack_bf16x2(b.z, b.w);
      if (q.mc) {
        multimem_st_b32x4(static_cast<uint4*>(q.mc) + base + i, u);
      } else {
#pragma unroll
        for (int r = 0; r < COLL_MAX_RANKS; ++r)
          if (r < q.world) static_cast<uint4*>(q.buf[r])[base + i] = u;
      }
    }
  } else {
    const long long base = p.rank * per4;
    for (long long i = tid; i < per4; i += nth) {
      const float4 a = slot_sum(i);
      if (q.mc) {
        multimem_st_f32x4(static_cast<float4*>(q.mc) + base + i, a);
      } else {
#pragma unroll
        for (int r = 0; r < COLL_MAX_RANKS; ++r)
          if (r < q.world) static_cast<float4*>(q.buf[r])[base + i] = a;
      }
    }
  }
  cta_barrier_all_ranks(p, flag_value(epoch, 2), status);
}

// All ranks meet here (one CTA per rank): everything each rank launched before it on the stream is
// complete and visible to the others when it returns.
__global__ void rank_barrier_kernel(CollPeers p, uint32_t epoch, int* status) {
  cta_barrier_all_ranks(p, flag_value(epoch, 1), status);
}

// Test hook for the bounded wait: waits on a flag slot that nothing writes, with a short limit,
// and reports the timeout through the status word. Touches no peer memory.
__global__ void wait_timeout_probe_kernel(const uint32_t* flag, uint32_t value, unsigned long long limit_ns,
                                          int* status) {
  const uint64_t t0 = global_timer_ns();
  while (!flag_reached(ld_acquire_sys(flag), value)) {
    if (global_timer_ns() - t0 > limit_ns) {
      atomicCAS(status, STATUS_OK, STATUS_TIMEOUT_PEER_FLAG);
      return;
    }
  }
}

static void fill_peers(CollPeers& p, const long long* bufs, const long long* flags, long long mc, int rank,
                       int world) {
  for (int r = 0; r < COLL_MAX_RANKS; ++r) {
    p.buf[r] = r < world ? reinterpret_cast<void*>(bufs[r]) : nullptr;
    p.flags[r] = (r < world && flags) ? reinterpret_cast<uint32_t*>(flags[r]) : nullptr;
  }
  p.mc = reinterpret_cast<void*>(mc);
  p.rank = rank;
  p.world = world;
}

}  // namespace bdh

using namespace bdh;

extern "C" int bdh_allreduce_scale(const long long* buf_ptrs, const long long* flag_ptrs, long long mc_ptr,
                                   int rank, int world, long long n_floats, float scale, unsigned epoch,
                                   int ctas, int* status, cudaStream_t s) {
  if (world < 1 || world > COLL_MAX_RANKS || (n_floats % (4LL * world)) || ctas < 1) return BDH_ERR_ARGUMENT;
  CollPeers p;
  fill_peers(p, buf_ptrs, flag_ptrs, mc_ptr, rank, world);
  allreduce_scale_kernel<<<ctas, COLL_THREADS, 0, s>>>(p, n_floats / 4, scale, epoch, status);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_rs_adamw_ag(const long long* grad_ptrs, const long long* flag_ptrs, long long grad_mc,
                               const long long* shadow_ptrs, int rank, int world, long long n_floats,
                               float* master, float* m, float* v, float lr, float beta1, float beta2, float eps,
                               float wd, int step, float grad_scale, unsigned epoch, int ctas, int* status,
                               cudaStream_t s) {
  if (world < 1 || world > COLL_MAX_RANKS || (n_floats % (4LL * world)) || ctas < 1 || step < 1)
    return BDH_ERR_ARGUMENT;
  CollPeers p, q;
  fill_peers(p, grad_ptrs, flag_ptrs, grad_mc, rank, world);
  fill_peers(q, shadow_ptrs, nullptr, 0, rank, world);
  AdamArgs a{lr, beta1, beta2, eps, wd, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
             grad_scale};
  rs_adamw_ag_kernel<<<ctas, COLL_THREADS, 0, s>>>(p, q, master, m, v, n_floats / 4, a, epoch, status);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_shard_adamw_ag(const long long* flag_ptrs, const long long* shadow_ptrs, int rank, int world,
                                  float* gacc, float* master, float* m, float* v, int n_segs, const long long* seg_lo,
                                  const long long* seg_dst, float lr, float beta1, float beta2, float eps, float wd,
                                  int step, float grad_scale, unsigned epoch, int ctas, int* status, cudaStream_t s) {
  if (world < 1 || world > COLL_MAX_RANKS || ctas < 1 || step < 1 || n_segs < 1 || n_segs > 4) return BDH_ERR_ARGUMENT;
  ShardSegs segs;
  segs.n = n_segs;
  for (int i = 0; i <= n_segs; ++i) {
    if (seg_lo[i] % 4) return BDH_ERR_ALIGNMENT;
    segs.lo4[i] = seg_lo[i] / 4;
  }
  for (int i = 0; i < n_segs; ++i) {
    if (seg_dst[i] % 4) return BDH_ERR_ALIGNMENT;
    segs.dst4[i] = seg_dst[i] / 4;
  }
  CollPeers f, q;
  fill_peers(f, flag_ptrs, flag_ptrs, 0, rank, world);
  fill_peers(q, shadow_ptrs, nullptr, 0, rank, world);
  AdamArgs a{lr, beta1, beta2, eps, wd, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step), grad_scale};
  shard_adamw_ag_kernel<<<ctas, COLL_THREADS, 0, s>>>(f, q, gacc, master, m, v, segs, a, epoch, status);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_shard_bcast(const long long* flag_ptrs, const long long* out_ptrs, long long out_mc, int rank, int world,
                               float* gacc, int n_segs, const long long* seg_lo, const long long* seg_dst, float scale,
                               unsigned epoch, int ctas, int* status, cudaStream_t s) {
  if (world < 1 || world > COLL_MAX_RANKS || ctas < 1 || n_segs < 1 || n_segs > 4) return BDH_ERR_ARGUMENT;
  ShardSegs segs;
  segs.n = n_segs;
  for (int i = 0; i <= n_segs; ++i) {
    if (seg_lo[i] % 4) return BDH_ERR_ALIGNMENT;
    segs.lo4[i] = seg_lo[i] / 4;
  }
  for (int i = 0; i < n_segs; ++i) {
    if (seg_dst[i] % 4) return BDH_ERR_ALIGNMENT;
    segs.dst4[i] = seg_dst[i] / 4;
  }
  CollPeers f, q;
  fill_peers(f, flag_ptrs, flag_ptrs, 0, rank, world);
  fill_peers(q, out_ptrs, nullptr, out_mc, rank, world);
  shard_bcast_kernel<<<ctas, COLL_THREADS, 0, s>>>(f, q, gacc, segs, scale, epoch, status);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_gather_blocks(const long long* slot_ptrs, const long long* flag_ptrs, const long long* out_ptrs,
                                 long long out_mc, int out_bf16, int rank, int world, long long block_floats,
                                 unsigned epoch, int ctas, int* status, cudaStream_t s) {
  if (world < 1 || world > COLL_MAX_RANKS || (block_floats % 8) || block_floats < 8 || ctas < 1 || !out_ptrs)
    return BDH_ERR_ARGUMENT;
  CollPeers p, q;
  fill_peers(p, slot_ptrs, flag_ptrs, 0, rank, world);
  fill_peers(q, out_ptrs, nullptr, out_mc, rank, world);
  if (out_bf16)
    gather_blocks_kernel<true><<<ctas, COLL_THREADS, 0, s>>>(p, q, block_floats / 4, epoch, status);
  else
    gather_blocks_kernel<false><<<ctas, COLL_THREADS, 0, s>>>(p, q, block_floats / 4, epoch, status);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_rank_barrier(const long long* flag_ptrs, int rank, int world, unsigned epoch, int* status,
                                cudaStream_t s) {
  if (world < 1 || world > COLL_MAX_RANKS) return BDH_ERR_ARGUMENT;
  CollPeers p;
  fill_peers(p, flag_ptrs, flag_ptrs, 0, rank, world);
  rank_barrier_kernel<<<1, 32, 0, s>>>(p, epoch, status);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_wait_timeout_probe(const unsigned* flag, unsigned value, unsigned long long limit_ns,
                                      int* status, cudaStream_t s) {
  wait_timeout_probe_kernel<<<1, 1, 0, s>>>(flag, value, limit_ns, status);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}
