// Cached-decode kernels: the recurrent state update of BDH's linear attention for one new token
// per stream, batched next-token sampling, and the activation-image encoder.
//
// State update (reference: src/model/bdh.rs:288-302, one iteration of its per-timestep loop):
//     a[b,h,:]   = sum_n q[b,h,n] * rho[b,h,n,:]          (read before write: no self term)
//     rho[b,h,n,:] = (rho[b,h,n,:] + q[b,h,n] * v[b,:]) * gamma_h
// The state is fp32 [B, H, N', D] and is the only large thing a decode step touches, so the kernel
// is written around its traffic: rows whose query entry is zero (the ReLU-sparse majority) are
// neither read nor written when there is no decay (RoPE / PoPE). With ALiBi decay every row is
// scaled every step - unless the decay is applied lazily: `last[b,h,n]` holds the step up to which
// row n is current, a row is brought up to date (times gamma^(step - last)) only when its query entry
// touches it, and rows with a zero query entry are skipped as in the decay-free case. Whoever takes
// the state out of the engine first brings every row up to date (engine/decode_engine.py). One CTA
// owns a slab of rows of one (stream, head); partial outputs are combined with fp32 atomics into a
// zero-initialised `a`.
#include "bdh_kernels.h"
#include "sm100_ptx.cuh"

#include <cuda_fp16.h>
#include <math.h>

namespace bdh {

constexpr int DEC_ROWS_PER_CTA = 128;
constexpr int DEC_THREADS = 256;

// q: bf16 [B, H*Np] (row b, column h*Np + n); v: bf16 [B, D]; rho: fp32 [B,H,Np,D]; a: fp32 [H*B, D]
// written at row h*B + b (head-major, the layout the following GEMM consumes).
__device__ __forceinline__ int n0_of(int slab) { return slab * DEC_ROWS_PER_CTA; }

template <int VEC>  // D = VEC * 4 * lanes_per_row ... each thread owns 4*VEC consecutive floats
__global__ void __launch_bounds__(DEC_THREADS)
decode_state_update_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ v,
                           float* __restrict__ rho, float* __restrict__ a, const float* __restrict__ slopes,
                           int* __restrict__ last, const int* __restrict__ step_dev, int B, int H, int Np, int D) {
  const int slab = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int threads_per_row = D / (4 * VEC);              // threads that cover one row of D floats
  const int rows_in_flight = DEC_THREADS / threads_per_row;
  const int tr = threadIdx.x / threads_per_row;           // which row of the group
  const int tc = threadIdx.x % threads_per_row;           // which 4*VEC-float segment of the row
  const float slope = slopes ? slopes[h] : 0.f;
  const float gamma = slopes ? __expf(-slope) : 1.f;
  const bool lazy = slopes != nullptr && last != nullptr;
  const bool dense = slopes != nullptr && !lazy;
  const int step = lazy ? *step_dev : 0;
  int* last_row = lazy ? last + (static_cast<long long>(b) * H + h) * Np + n0_of(slab) : nullptr;

  __shared__ float qs[DEC_ROWS_PER_CTA];
  __shared__ int active[DEC_ROWS_PER_CTA];
  __shared__ int n_active;
  __shared__ float catch_up_s[DEC_ROWS_PER_CTA];
  const int n0 = slab * DEC_ROWS_PER_CTA;
  const __nv_bfloat16* qrow = q + static_cast<long long>(b) * H * Np + static_cast<long long>(h) * Np;
  if (threadIdx.x == 0) n_active = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < DEC_ROWS_PER_CTA; i += DEC_THREADS) {
    const int n = n0 + i;
    const float qv = (n < Np) ? __bfloat162float(qrow[n]) : 0.f;
    qs[i] = qv;
    const bool live = n < Np && (dense || qv != 0.f);
    if (live) active[atomicAdd(&n_active, 1)] = i;
    if (lazy && live) {
      // one thread per row reads how many steps the row sat out and marks it current (through this step's decay)
      catch_up_s[i] = __expf(-slope * static_cast<float>(step - last_row[i]));
      last_row[i] = step + 1;
    }
  }
  __syncthreads();
  const int na = n_active;
  if (na == 0) return;

  float vv[4 * VEC], acc[4 * VEC];
  const __nv_bfloat16* vrow = v + static_cast<long long>(b) * D + tc * 4 * VEC;
#pragma unroll
  for (int i = 0; i < 4 * VEC; ++i) {
    vv[i] = __bfloat162float(vrow[i]);
    acc[i] = 0.f;
  }
  float* base = rho + ((static_cast<long long>(b) * H + h) * Np) * D + tc * 4 * VEC;
  // UNROLL active rows per thread group are loaded before any of them is updated: the kernel is a pure stream
  // over the state, and what it sustains is set by the bytes each SM keeps in flight
  constexpr int UNROLL = (VEC >= 4) ? 1 : (VEC == 2 ? 2 : 4);
  for (int j0 = tr; j0 < na; j0 += rows_in_flight * UNROLL) {
    float4 r[UNROLL][VEC];
    float4* p[UNROLL];
    float qv[UNROLL], catch_up[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int j = j0 + u * rows_in_flight;
      const int i = (j < na) ? active[j] : 0;
      qv[u] = (j < na) ? qs[i] : 0.f;
      catch_up[u] = 1.f;
      p[u] = reinterpret_cast<float4*>(base + static_cast<long long>(n0 + i) * D);
      if (j < na) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) r[u][k] = __ldcs(p[u] + k);
        if (lazy) catch_up[u] = catch_up_s[i];
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (j0 + u * rows_in_flight >= na) break;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        float4 t = r[u][k];
        t.x *= catch_up[u]; t.y *= catch_up[u]; t.z *= catch_up[u]; t.w *= catch_up[u];
        acc[4 * k + 0] += qv[u] * t.x; acc[4 * k + 1] += qv[u] * t.y;
        acc[4 * k + 2] += qv[u] * t.z; acc[4 * k + 3] += qv[u] * t.w;
        t.x = (t.x + qv[u] * vv[4 * k + 0]) * gamma; t.y = (t.y + qv[u] * vv[4 * k + 1]) * gamma;
        t.z = (t.z + qv[u] * vv[4 * k + 2]) * gamma; t.w = (t.w + qv[u] * vv[4 * k + 3]) * gamma;
        __stcs(p[u] + k, t);
      }
    }
  }
  // combine the row groups of this CTA in shared memory, then one atomic per output element
  __shared__ float red[DEC_THREADS * 4];   // enough for VEC <= 1 per pass; larger VEC loops
  float* out = a + (static_cast<long long>(h) * B + b) * D + tc * 4 * VEC;
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) red[threadIdx.x * 4 + i] = acc[4 * k + i];
    __syncthreads();
    if (tr == 0) {
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      for (int g = 0; g < rows_in_flight; ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i] += red[(g * threads_per_row + tc) * 4 + i];
#pragma unroll
      for (int i = 0; i < 4; ++i) atomicAdd(out + 4 * k + i, s[i]);
    }
  }
}

// ---- sampling --------------------------------------------------------------------------------------
// One warp per stream, V <= 1024. Temperature, top-k with ties kept (values below the k-th largest
// are removed), softmax in fp32, uniform fallback for a degenerate row, inverse-CDF draw with a
// counter-based generator; `greedy` takes the arg-max. (reference: src/generation.rs:26-72)
__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}

__global__ void __launch_bounds__(128)
sample_tokens_kernel(const float* __restrict__ logits, long long* __restrict__ out, int B, int V,
                     float temperature, int top_k, int greedy, uint32_t seed, const int* __restrict__ step_ptr,
                     int step_host) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= B) return;
  const float* p = logits + static_cast<long long>(warp) * V;
  float x[32];
  const float inv_t = 1.f / fmaxf(temperature, 1e-8f);
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    int c = j * 32 + lane;
    x[j] = (c < V) ? p[c] * (greedy ? 1.f : inv_t) : -INFINITY;
  }
  // arg-max (lowest index wins ties)
  float best = -INFINITY;
  int best_i = 0x7fffffff;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    int c = j * 32 + lane;
    if (c < V && (x[j] > best || (x[j] == best && c < best_i))) { best = x[j]; best_i = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
  }
  if (greedy) {
    if (lane == 0) out[warp] = best_i == 0x7fffffff ? 0 : best_i;
    return;
  }
  // top-k threshold: k-th largest value, found by bisection on the count of values >= t
  if (top_k > 0 && top_k < V) {
    float lo = INFINITY, hi = best;
#pragma unroll
    for (int j = 0; j < 32; ++j) if (isfinite(x[j])) lo = fminf(lo, x[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    // invariant: count(x >= lo) >= k ; find the largest threshold that still keeps >= k values
    for (int it = 0; it < 40 && hi > lo; ++it) {
      float mid = lo + 0.5f * (hi - lo);
      if (mid <= lo || mid >= hi) break;
      int cnt = 0;
#pragma unroll
      for (int j = 0; j < 32; ++j) cnt += (x[j] >= mid) ? 1 : 0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
      if (cnt >= top_k) lo = mid; else hi = mid;
    }
    // the k-th largest value is the smallest element >= lo
    float kth = INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j) if (x[j] >= lo) kth = fminf(kth, x[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) kth = fminf(kth, __shfl_xor_sync(0xffffffffu, kth, o));
#pragma unroll
    for (int j = 0; j < 32; ++j) if (x[j] < kth) x[j] = -INFINITY;
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    x[j] = (x[j] == -INFINITY) ? 0.f : __expf(x[j] - best);
    s += x[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const bool degenerate = !(s > 0.f) || !isfinite(s);
  const int step = step_ptr ? *step_ptr : step_host;
  const uint32_t r = hash_u32(hash_u32(seed ^ (0x9E3779B9u * static_cast<uint32_t>(warp + 1))) ^
                              (0x85EBCA6Bu * static_cast<uint32_t>(step + 1)));
  const float u = (static_cast<float>(r >> 8) + 0.5f) * (1.f / 16777216.f);
  if (degenerate) {
    if (lane == 0) out[warp] = min(V - 1, static_cast<int>(u * V));
    return;
  }
  // inverse CDF over columns in index order: column c = j*32 + lane
  const float target = u * s;
  float run = 0.f;
  int pick = -1;
  for (int j = 0; j < 32 && pick < 0; ++j) {
    // inclusive prefix over lanes for this group of 32 columns
    float pre = x[j];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float t = __shfl_up_sync(0xffffffffu, pre, o);
      if (lane >= o) pre += t;
    }
    const float total = __shfl_sync(0xffffffffu, pre, 31);
    const unsigned hit = __ballot_sync(0xffffffffu, x[j] > 0.f && run + pre >= target);
    if (hit) pick = j * 32 + (__ffs(hit) - 1);
    run += total;
  }
  if (pick < 0) pick = best_i;     // rounding left the target just above the total mass
  if (lane == 0) out[warp] = pick;
}

// ---- activation images ------------------------------------------------------------------------------
// One column of a [rows, history, 4] fp32 RGBA ring-buffer image per call, rows [row0, row0+units):
//   v = max(value, 0); mag = g*v / (g*v + 0.35); mask = v / (v + 0.004); i = (mag*mask)^1.15
//   rgb = (low + (high - low) * i) * i ; alpha = 1 ; head boundaries take max(rgb, separator)
// with low / high / separator already in linear colour (behaviour of the reference's encoder,
// src/viz/encoder.rs:234-298). Rendering it is somebody else's job: the buffer stays on the device
// or is written to a file.
__global__ void viz_encode_units_kernel(const float* __restrict__ values, float* __restrict__ image, int units,
                                        int history, int cursor, int row0, float gain, float3 lo, float3 hi,
                                        float3 sep, int units_per_head) {
  const int u = blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= units) return;
  const float v = fmaxf(values[u], 0.f);
  const float sc = v * gain;
  const float mag = sc / (sc + 0.35f);
  const float mask = v / (v + 0.004f);
  const float t = powf(mag * mask, 1.15f);
  float r = (lo.x + (hi.x - lo.x) * t) * t, g = (lo.y + (hi.y - lo.y) * t) * t, b = (lo.z + (hi.z - lo.z) * t) * t;
  if (units_per_head > 0 && u > 0 && u % units_per_head == 0) {
    r = fmaxf(r, sep.x); g = fmaxf(g, sep.y); b = fmaxf(b, sep.z);
  }
  float* px = image + (static_cast<long long>(row0 + u) * history + cursor) * 4;
  px[0] = r; px[1] = g; px[2] = b; px[3] = 1.f;
}

// RoPE table row for graph-captured decoding: table[2i] = cos, table[2i+1] = sin (fp16) of
// 2*pi*frac(pos * freq_i) with the position read from device memory, so a captured graph needs no
// new kernel arguments as the position advances.
__global__ void rope_table_step_kernel(const int* pos, const float* __restrict__ pair_freqs, __half* table,
                                       int n_pairs) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  float raw = static_cast<float>(*pos) * pair_freqs[i];
  float ph = (raw - floorf(raw)) * 6.283185307179586f;
  float s, c;
  sincosf(ph, &s, &c);
  table[2 * i] = __float2half_rn(c);
  table[2 * i + 1] = __float2half_rn(s);
}
__global__ void bump_counter_kernel(int* counter, int by) { *counter += by; }

}  // namespace bdh

using namespace bdh;

extern "C" int bdh_decode_state_update(const void* q, const void* v, float* rho, float* a, const float* slopes,
                                       int* last, const int* step_dev, int B, int H, int Np, int D, cudaStream_t s) {
  if (D % 64 || D > 1024 || Np <= 0 || B <= 0 || (last != nullptr) != (step_dev != nullptr)) return BDH_ERR_ARGUMENT;
  dim3 grid((Np + DEC_ROWS_PER_CTA - 1) / DEC_ROWS_PER_CTA, H, B);
  // 64 threads per row when possible (D/64 floats each): VEC = D / 256, at least 1
  typedef const __nv_bfloat16* bp;
  if (D % 256 == 0 && D / 256 == 1)
    decode_state_update_kernel<1><<<grid, DEC_THREADS, 0, s>>>((bp)q, (bp)v, rho, a, slopes, last, step_dev, B, H, Np, D);
  else if (D % 256 == 0 && D / 256 == 2)
    decode_state_update_kernel<2><<<grid, DEC_THREADS, 0, s>>>((bp)q, (bp)v, rho, a, slopes, last, step_dev, B, H, Np, D);
  else if (D % 256 == 0 && D / 256 == 4)
    decode_state_update_kernel<4><<<grid, DEC_THREADS, 0, s>>>((bp)q, (bp)v, rho, a, slopes, last, step_dev, B, H, Np, D);
  else if (DEC_THREADS % (D / 4) == 0)
    decode_state_update_kernel<1><<<grid, DEC_THREADS, 0, s>>>((bp)q, (bp)v, rho, a, slopes, last, step_dev, B, H, Np, D);
  else
    return BDH_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_sample_tokens(const float* logits, long long* out, int B, int V, float temperature, int top_k,
                                 int greedy, unsigned seed, const int* step_dev, int step_host, cudaStream_t s) {
  if (V <= 0 || V > 1024 || B <= 0) return BDH_ERR_ARGUMENT;
  const int warps_per_block = 4;
  sample_tokens_kernel<<<(B + warps_per_block - 1) / warps_per_block, warps_per_block * 32, 0, s>>>(
      logits, out, B, V, temperature, top_k, greedy, seed, step_dev, step_host);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_viz_encode_units(const float* values, float* image, int units, int history, int cursor,
                                    int row0, float gain, const float* lo_rgb, const float* hi_rgb,
                                    const float* sep_rgb, int units_per_head, cudaStream_t s) {
  if (units <= 0 || history <= 0 || cursor < 0 || cursor >= history || row0 < 0) return BDH_ERR_ARGUMENT;
  float3 lo = make_float3(lo_rgb[0], lo_rgb[1], lo_rgb[2]), hi = make_float3(hi_rgb[0], hi_rgb[1], hi_rgb[2]);
  float3 sep = make_float3(sep_rgb[0], sep_rgb[1], sep_rgb[2]);
  viz_encode_units_kernel<<<(units + 255) / 256, 256, 0, s>>>(values, image, units, history, cursor, row0, gain, lo,
                                                              hi, sep, units_per_head);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_rope_table_step(const int* pos, const float* pair_freqs, void* table_f16, int n_pairs,
                                   cudaStream_t s) {
  if (n_pairs <= 0) return BDH_ERR_ARGUMENT;
  rope_table_step_kernel<<<(n_pairs + 255) / 256, 256, 0, s>>>(pos, pair_freqs, (__half*)table_f16, n_pairs);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}
extern "C" int bdh_bump_counter(int* counter, int by, cudaStream_t s) {
  bump_counter_kernel<<<1, 1, 0, s>>>(counter, by);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}
