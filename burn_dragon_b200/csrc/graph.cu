// Block-ELL sparse neuron-graph propagation for the BDH-graph model path:
//     y[m, n] = relu( sum over the active column blocks j of neuron block nb:  x[m, j*64 : j*64+64] . W[n, same] - theta )
// W is [N_total, D] row-major (one row per neuron) and only the listed 64x64 blocks are touched;
// `ell_cols` [N_total/64, ell_width] holds the active column-block indices of each neuron block,
// padded with -1. With every block listed this equals the dense encoder relu(x W^T - theta)
// (reference semantics: src/kernel/relu_lowrank.rs:7-37). The reference has no sparse-graph path.
#include "bdh_kernels.h"
#include "sm100_ptx.cuh"
#include "debug_bounds.cuh"

namespace bdh {

constexpr int GB = 64;            // block edge (neurons x embedding columns)
constexpr int G_THREADS = 256;

__global__ void __launch_bounds__(G_THREADS)
graph_spmm_relu_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       const int* __restrict__ ell_cols, __nv_bfloat16* __restrict__ y, int M, int Ntot, int D,
                       int ell_width, float theta) {
  __shared__ float sx[GB][GB + 1];
  __shared__ float sw[GB][GB + 1];
  const int mb = blockIdx.x, nb = blockIdx.y;
  const int tm = (threadIdx.x / 16) * 4, tn = (threadIdx.x % 16) * 4;
  float acc[4][4] = {};
  for (int e = 0; e < ell_width; ++e) {
    const int cb = ell_cols[nb * ell_width + e];
    if (cb < 0) break;
    BDH_BOUNDS_CHECK(cb, (D + GB - 1) / GB, BOUNDS_GRAPH_COLUMN, static_cast<long long>(nb) * ell_width + e);
    for (int i = threadIdx.x; i < GB * GB; i += G_THREADS) {
      const int r = i / GB, c = i % GB;
      const int m = mb * GB + r, n = nb * GB + r, d = cb * GB + c;
      sx[r][c] = (m < M && d < D) ? __bfloat162float(x[static_cast<long long>(m) * D + d]) : 0.f;
      sw[r][c] = (n < Ntot && d < D) ? __bfloat162float(w[static_cast<long long>(n) * D + d]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < GB; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = sx[tm + i][k]; b[i] = sw[tn + i][k]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = mb * GB + tm + i, n = nb * GB + tn + j;
      if (m < M && n < Ntot)
        y[static_cast<long long>(m) * Ntot + n] = __float2bfloat16_rn(fmaxf(acc[i][j] - theta, 0.f));
    }
}

}  // namespace bdh

extern "C" int bdh_graph_spmm_relu(const void* x_bf16, const void* w_bf16, const int* ell_cols, void* y_bf16, int M,
                                   int Ntot, int D, int ell_width, float theta, cudaStream_t s) {
  if (M <= 0 || Ntot <= 0 || D <= 0 || ell_width <= 0) return BDH_ERR_ARGUMENT;
  dim3 grid((M + bdh::GB - 1) / bdh::GB, (Ntot + bdh::GB - 1) / bdh::GB);
  bdh::graph_spmm_relu_kernel<<<grid, bdh::G_THREADS, 0, s>>>((const __nv_bfloat16*)x_bf16, (const __nv_bfloat16*)w_bf16,
                                                             ell_cols, (__nv_bfloat16*)y_bf16, M, Ntot, D, ell_width,
                                                             theta);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

// First data-dependent index of this file's kernels that was out of range since the last clear:
// out = {checked build?, site, index, extent, where} (csrc/debug_bounds.cuh).
extern "C" int bdh_bounds_record_graph(long long* out5, int clear) { return bdh::bounds_record_read(out5, clear) ? BDH_ERR_LAUNCH : BDH_OK; }
