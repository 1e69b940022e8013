// Elementwise parts of a Mamba-2 block around the SSD scan, fp32, forward and backward:
//   * causal depthwise conv1d (width k <= 8) + bias + SiLU over [B, T + k - 1, C] (the k - 1 leading rows are
//     the tail of the previous segment, or zeros),
//   * the gated RMSNorm behind the scan, out = rmsnorm(v * silu(z)) * w.
// Both are bandwidth-bound: every tensor is read once (neighbouring taps come from L1 / L2) and written once;
// the parameter gradients are reduced per block before they touch global memory.
#include <cuda_runtime.h>

#include "bdh_kernels.h"

namespace bdh {

constexpr int CONV_MAX_K = 8;
constexpr int CONV_THREADS = 128;     // channels per block (contiguous: coalesced rows)
constexpr int CONV_ROWS = 64;         // (batch, time) rows per block in the backward pass

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// out[b, t, c] = silu(bias[c] + sum_j w[c, j] * seq[b, t + j, c])
__global__ void __launch_bounds__(CONV_THREADS)
conv1d_silu_fwd_kernel(const float* __restrict__ seq, const float* __restrict__ w, const float* __restrict__ bias,
                       float* __restrict__ out, long long rows, int T, int C, int k) {
  const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
  if (c >= C) return;
  float wk[CONV_MAX_K];
#pragma unroll
  for (int j = 0; j < CONV_MAX_K; ++j) wk[j] = (j < k) ? w[static_cast<long long>(c) * k + j] : 0.f;
  const float bc = bias ? bias[c] : 0.f;
  for (long long row = blockIdx.y; row < rows; row += gridDim.y) {
    const long long b = row / T;
    const int t = static_cast<int>(row % T);
    const float* p = seq + (b * (T + k - 1) + t) * C + c;
    float pre = bc;
#pragma unroll
    for (int j = 0; j < CONV_MAX_K; ++j)
      if (j < k) pre += wk[j] * p[static_cast<long long>(j) * C];
    out[row * C + c] = pre * sigmoidf_(pre);
  }
}

// dpre[b, t, c] = dout * silu'(pre) (pre recomputed); dw[c, j] += sum dpre * seq[b, t + j, c]; db[c] += sum dpre.
// One thread per channel walks CONV_ROWS rows, so the parameter gradients cost k + 1 atomics per thread.
__global__ void __launch_bounds__(CONV_THREADS)
conv1d_silu_bwd_pre_kernel(const float* __restrict__ seq, const float* __restrict__ w, const float* __restrict__ bias,
                           const float* __restrict__ dout, float* __restrict__ dpre, float* __restrict__ dw,
                           float* __restrict__ db, long long rows, int T, int C, int k) {
  const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
  if (c >= C) return;
  float wk[CONV_MAX_K], gw[CONV_MAX_K];
#pragma unroll
  for (int j = 0; j < CONV_MAX_K; ++j) {
    wk[j] = (j < k) ? w[static_cast<long long>(c) * k + j] : 0.f;
    gw[j] = 0.f;
  }
  const float bc = bias ? bias[c] : 0.f;
  float gb = 0.f;
  const long long r0 = static_cast<long long>(blockIdx.y) * CONV_ROWS;
  const long long r1 = (r0 + CONV_ROWS < rows) ? r0 + CONV_ROWS : rows;
  for (long long row = r0; row < r1; ++row) {
    const long long b = row / T;
    const int t = static_cast<int>(row % T);
    const float* p = seq + (b * (T + k - 1) + t) * C + c;
    float x[CONV_MAX_K];
    float pre = bc;
#pragma unroll
    for (int j = 0; j < CONV_MAX_K; ++j) {
      x[j] = (j < k) ? p[static_cast<long long>(j) * C] : 0.f;
      pre += wk[j] * x[j];
    }
    const float s = sigmoidf_(pre);
    const float g = dout[row * C + c] * s * (1.f + pre * (1.f - s));
    dpre[row * C + c] = g;
    gb += g;
#pragma unroll
    for (int j = 0; j < CONV_MAX_K; ++j) gw[j] += g * x[j];
  }
#pragma unroll
  for (int j = 0; j < CONV_MAX_K; ++j)
    if (j < k) atomicAdd(dw + static_cast<long long>(c) * k + j, gw[j]);
  if (db) atomicAdd(db + c, gb);
}

// dseq[b, tau, c] = sum_j w[c, j] * dpre[b, tau - j, c] over 0 <= tau - j < T
__global__ void __launch_bounds__(CONV_THREADS)
conv1d_silu_bwd_seq_kernel(const float* __restrict__ dpre, const float* __restrict__ w, float* __restrict__ dseq,
                           long long rows_in, int T, int C, int k) {
  const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
  if (c >= C) return;
  float wk[CONV_MAX_K];
#pragma unroll
  for (int j = 0; j < CONV_MAX_K; ++j) wk[j] = (j < k) ? w[static_cast<long long>(c) * k + j] : 0.f;
  const int Tin = T + k - 1;
  for (long long row = blockIdx.y; row < rows_in; row += gridDim.y) {
    const long long b = row / Tin;
    const int tau = static_cast<int>(row % Tin);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_K; ++j) {
      const int t = tau - j;
      if (j < k && t >= 0 && t < T) acc += wk[j] * dpre[(b * T + t) * C + c];
    }
    dseq[row * C + c] = acc;
  }
}

// ---- gated RMSNorm ---------------------------------------------------------------------------------
constexpr int NORM_WARPS = 8;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// out = g * rstd * w with g = v * silu(z), rstd = rsqrt(mean(g^2) + eps); one warp per row.
__global__ void __launch_bounds__(NORM_WARPS * 32)
gated_rmsnorm_fwd_kernel(const float* __restrict__ v, const float* __restrict__ z, const float* __restrict__ w,
                         float* __restrict__ out, float* __restrict__ rstd, long long rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * NORM_WARPS;
  for (; row < rows; row += stride) {
    const float* pv = v + row * D;
    const float* pz = z + row * D;
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) {
      const float zz = pz[c];
      const float g = pv[c] * zz * sigmoidf_(zz);
      ss += g * g;
    }
    const float r = rsqrtf(warp_sum_f(ss) / D + eps);
    if (lane == 0) rstd[row] = r;
    for (int c = lane; c < D; c += 32) {
      const float zz = pz[c];
      out[row * D + c] = pv[c] * zz * sigmoidf_(zz) * r * w[c];
    }
  }
}

// dg = r (w dout) - g r^3 mean(g w dout); dv = dg silu(z); dz = dg v silu'(z); dw += dout g r (block-reduced in
// shared memory, one global atomic per column and block).
__global__ void __launch_bounds__(NORM_WARPS * 32)
gated_rmsnorm_bwd_kernel(const float* __restrict__ v, const float* __restrict__ z, const float* __restrict__ w,
                         const float* __restrict__ rstd, const float* __restrict__ dout, float* __restrict__ dv,
                         float* __restrict__ dz, float* __restrict__ dw, long long rows, int D) {
  extern __shared__ float dw_acc[];
  for (int c = threadIdx.x; c < D; c += blockDim.x) dw_acc[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * NORM_WARPS;
  for (; row < rows; row += stride) {
    const float* pv = v + row * D;
    const float* pz = z + row * D;
    const float* pd = dout + row * D;
    const float r = rstd[row];
    float dot = 0.f;
    for (int c = lane; c < D; c += 32) {
      const float zz = pz[c];
      dot += pv[c] * zz * sigmoidf_(zz) * w[c] * pd[c];
    }
    const float m = warp_sum_f(dot) / D * r * r * r;
    for (int c = lane; c < D; c += 32) {
      const float zz = pz[c], vv = pv[c], dd = pd[c];
      const float s = sigmoidf_(zz);
      const float sl = zz * s;
      const float g = vv * sl;
      const float dg = r * w[c] * dd - g * m;
      dv[row * D + c] = dg * sl;
      dz[row * D + c] = dg * vv * s * (1.f + zz * (1.f - s));
      atomicAdd(dw_acc + c, dd * g * r);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += blockDim.x) atomicAdd(dw + c, dw_acc[c]);
}

}  // namespace bdh

using namespace bdh;

static inline int launch_ok() { return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH; }

extern "C" int bdh_conv1d_silu_fwd(const float* seq, const float* w, const float* bias, float* out, int B, int T,
                                   int C, int k, cudaStream_t s) {
  if (k < 1 || k > CONV_MAX_K || B < 0 || T < 0 || C < 1) return BDH_ERR_ARGUMENT;
  const long long rows = static_cast<long long>(B) * T;
  if (rows == 0) return BDH_OK;
  dim3 grid((C + CONV_THREADS - 1) / CONV_THREADS, static_cast<unsigned>(rows < 16384 ? rows : 16384));
  conv1d_silu_fwd_kernel<<<grid, CONV_THREADS, 0, s>>>(seq, w, bias, out, rows, T, C, k);
  return launch_ok();
}

extern "C" int bdh_conv1d_silu_bwd(const float* seq, const float* w, const float* bias, const float* dout,
                                   float* dpre, float* dseq, float* dw, float* db, int B, int T, int C, int k,
                                   cudaStream_t s) {
  if (k < 1 || k > CONV_MAX_K || B < 0 || T < 0 || C < 1) return BDH_ERR_ARGUMENT;
  const long long rows = static_cast<long long>(B) * T;
  if (rows == 0) return BDH_OK;
  const long long chunks = (rows + CONV_ROWS - 1) / CONV_ROWS;
  if (chunks > 65535) return BDH_ERR_TOO_LARGE;
  dim3 g1((C + CONV_THREADS - 1) / CONV_THREADS, static_cast<unsigned>(chunks));
  conv1d_silu_bwd_pre_kernel<<<g1, CONV_THREADS, 0, s>>>(seq, w, bias, dout, dpre, dw, db, rows, T, C, k);
  if (cudaGetLastError() != cudaSuccess) return BDH_ERR_LAUNCH;
  const long long rows_in = static_cast<long long>(B) * (T + k - 1);
  dim3 g2((C + CONV_THREADS - 1) / CONV_THREADS, static_cast<unsigned>(rows_in < 16384 ? rows_in : 16384));
  conv1d_silu_bwd_seq_kernel<<<g2, CONV_THREADS, 0, s>>>(dpre, w, dseq, rows_in, T, C, k);
  return launch_ok();
}

extern "C" int bdh_gated_rmsnorm_fwd(const float* v, const float* z, const float* w, float* out, float* rstd,
                                     long long rows, int D, float eps, cudaStream_t s) {
  if (D < 1 || rows < 0) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  const long long blocks = (rows + NORM_WARPS - 1) / NORM_WARPS;
  gated_rmsnorm_fwd_kernel<<<static_cast<unsigned>(blocks < 4096 ? blocks : 4096), NORM_WARPS * 32, 0, s>>>(
      v, z, w, out, rstd, rows, D, eps);
  return launch_ok();
}

extern "C" int bdh_gated_rmsnorm_bwd(const float* v, const float* z, const float* w, const float* rstd,
                                     const float* dout, float* dv, float* dz, float* dw, long long rows, int D,
                                     cudaStream_t s) {
  if (D < 1 || D > 12288 || rows < 0) return BDH_ERR_ARGUMENT;       // the column sums live in 48 KB of shared memory
  if (rows == 0) return BDH_OK;
  const long long blocks = (rows + NORM_WARPS - 1) / NORM_WARPS;
  gated_rmsnorm_bwd_kernel<<<static_cast<unsigned>(blocks < 592 ? blocks : 592), NORM_WARPS * 32,
                             static_cast<size_t>(D) * sizeof(float), s>>>(v, z, w, rstd, dout, dv, dz, dw, rows, D);
  return launch_ok();
}
